"""Grouped-query attention over the paged cache.

One part covers what the reference spreads over project_qkv (ampere_kv/runner.py:60-77),
apply_rope (runner.py:80-98), the cache write and the three attention paths of
decoder_layer_forward (runner.py:122-152) and o_proj (runner.py:163-165): q/k/v projection
(one product over the row-concatenated matrices), per-head RMSNorm of q and k before the
rotation, post-rotation K and plain V written to the request's pages, causal attention of
every new token over the pages (optionally only the last ``window`` keys), output projection.
Prompt portions and decoded tokens of many requests go through the same two kernels.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import (POSITION_ENCODINGS, CacheSpec, Mixer, ParamSpec, build_part, register_mixer)


@register_mixer("attention")
class PagedAttention(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``qk_norm`` (bool), ``qk_norm_eps``,
    ``bias`` (bool), ``window`` (keys visible including the query's own, or None),
    ``scale`` (None = head_dim ** -0.5), ``position_encoding`` (a PartSpec)."""

    graph_safe = True
    takes_lazy_norm = True
    adds_residual = True
    takes_stream_norm = True

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        p = spec.params
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.bias = bool(p.get("bias", False))
        self.window = p.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError(f"attention: window must be positive, got {self.window}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.head_dim ** -0.5
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"attention: {self.num_heads} heads are not a multiple of {self.num_kv_heads} kv heads")
        if self.head_dim % 16 or self.head_dim > 256:
            raise ValueError(f"attention: head_dim must be a multiple of 16 up to 256 for the attention kernels, "
                             f"got {self.head_dim}")
        self.position_encoding = build_part(POSITION_ENCODINGS, p["position_encoding"], hidden_size=self.hidden_size,
                                            dtype=self.dtype, device=self.device)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_norm_weight = self.k_norm_weight = None

    def children(self):
        return (self.position_encoding,)

    def preferred_q_tile(self):
        return ops.attention_q_tile(self.head_dim, self.num_heads // self.num_kv_heads)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(kind="window" if self.window is not None else "full", num_kv_heads=self.num_kv_heads,
                         head_dim=self.head_dim, window=None if self.window is None else int(self.window))

    def param_specs(self):
        h, d = self.hidden_size, self.head_dim
        specs = {
            "q_proj.weight": ParamSpec((self.num_heads * d, h)),
            "k_proj.weight": ParamSpec((self.num_kv_heads * d, h)),
            "v_proj.weight": ParamSpec((self.num_kv_heads * d, h)),
            "o_proj.weight": ParamSpec((h, self.num_heads * d)),
        }
        if self.bias:
            specs["q_proj.bias"] = ParamSpec((self.num_heads * d,), kind="bias")
            specs["k_proj.bias"] = ParamSpec((self.num_kv_heads * d,), kind="bias")
            specs["v_proj.bias"] = ParamSpec((self.num_kv_heads * d,), kind="bias")
            specs["o_proj.bias"] = ParamSpec((h,), kind="bias")
        if self.qk_norm:
            specs["q_norm.weight"] = ParamSpec((d,), kind="vector", init="norm")
            specs["k_norm.weight"] = ParamSpec((d,), kind="vector", init="norm")
        return specs

    def load(self, tensors):
        self.w_qkv = torch.cat((tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]),
                               dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.bias:
            self.b_qkv = torch.cat((tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"])).contiguous()
            self.b_o = tensors["o_proj.bias"].contiguous()
        if self.qk_norm:
            self.q_norm_weight = tensors["q_norm.weight"]
            self.k_norm_weight = tensors["k_norm.weight"]

    def forward(self, x, ctx, cache, residual=None):
        group = ctx.groups[cache.group]
        slots = group.slot_mapping if cache.writes else None
        k_cache = cache.k_cache if cache.writes else None
        v_cache = cache.v_cache if cache.writes else None
        fused = self.position_encoding.fused_rotary()
        q = None
        if isinstance(x, ops.StreamNorm):
            # a few decoded tokens: the projection goes behind the products that are still queued (the layer
            # before's output projection and feed-forward), all in one launch of the chained-product kernel
            on_tile = (fused is not None and self.b_qkv is None and self.head_dim == 128
                       and (fused[0] is None or fused[1] == 128) and ops.stream_takes(x.shape[0], self.w_qkv))
            if on_tile:
                q = torch.empty((x.shape[0], self.num_heads * 128), dtype=torch.bfloat16, device=self.w_qkv.device)
                x.pending.add(x.normed_phase(
                    self.w_qkv, epilogue="qkv", q_out=q, positions=ctx.positions, slots=slots,
                    q_weight=self.q_norm_weight, k_weight=self.k_norm_weight, inv_freq=fused[0], k_cache=k_cache,
                    v_cache=v_cache, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                    qk_eps=self.qk_norm_eps))
                x.pending.launch()
            else:
                x = x.materialize()
        if q is not None:
            pass        # the chained-product kernel made q and wrote K and V
        elif fused is not None:
            inv_freq, rotary_dim = fused
            q = ops.project_qkv(
                x, self.w_qkv, self.b_qkv, ctx.positions, slots, self.q_norm_weight, self.k_norm_weight, inv_freq,
                k_cache, v_cache, num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                rotary_dim=rotary_dim, eps=self.qk_norm_eps, status=ctx.status)
        else:
            # an encoding that is not a fused rotation: norm, encode on dense q/k, then write the pages
            qkv = ops.linear(x, self.w_qkv, self.b_qkv, partial_ok=True, status=ctx.status)
            q, k, v = ops.qk_norm_rope_write(
                qkv, ctx.positions, None, self.q_norm_weight, self.k_norm_weight, None, None, None,
                num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, rotary_dim=0,
                eps=self.qk_norm_eps, want_kv=True, status=ctx.status)
            q, k = self.position_encoding.apply(q, k, ctx.positions)
            if cache.writes:
                ops.kv_write(k.contiguous(), v, group.slot_mapping, cache.k_cache, cache.v_cache, status=ctx.status)
            q = q.contiguous()
        group_size = self.num_heads // self.num_kv_heads
        tensor_core = ops.attention_takes_tensor_cores(self.dtype, self.head_dim, group_size, cache.page_size)
        out = torch.empty_like(q)
        # decoded tokens beside prompt portions: the single-token tiles (they come first) run apart, with their keys
        # split over several CTAs; as one-row tiles of the prompt kernel each would walk its whole context alone
        first = getattr(ctx, "num_decode_tiles", 0)
        for lo, hi, q_tile in ((0, first, 1), (first, ctx.num_tiles, ctx.q_tile)):
            if hi <= lo:
                continue
            # the keys that the longest and the average tile walks: the context, or the window if that is shorter
            longest, mean = ctx.decode_contexts if q_tile == 1 else (ctx.max_context, ctx.max_context)
            if self.window:
                longest, mean = min(longest, self.window), min(mean, self.window)
            splits = 1 if q_tile > 1 and tensor_core else ops.choose_splits(
                hi - lo, self.num_kv_heads, q_tile * group_size, longest, tensor_core, mean_context=mean)
            ops.paged_attention(
                q, cache.k_cache, cache.v_cache, group.block_table, ctx.cu_q, ctx.ctx_lens, ctx.tile_seq[lo:hi],
                ctx.tile_q0[lo:hi], ctx.tile_nq[lo:hi], num_tiles=hi - lo, q_tile=q_tile, num_splits=splits,
                num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, window=self.window or 0, scale=self.scale,
                status=ctx.status, out=out)
        if residual is not None and self.b_o is None and ops.stream_takes(out.shape[0], self.w_o) \
                and residual.dtype == torch.float32 and residual.is_contiguous() \
                and residual.shape == (out.shape[0], self.w_o.shape[0]):
            # queued, not launched: the feed-forward and the next layer's projection join it
            pending = ops.PendingPhases(residual, ctx.status)
            pending.add(dict(w=self.w_o, x=out, epilogue="residual"))
            return pending
        if residual is not None and self.b_o is None:
            summed = ops.linear_into_residual(out, self.w_o, residual, status=ctx.status)
            if summed is not None:
                return summed
        return ops.linear(out, self.w_o, self.b_o, partial_ok=True, status=ctx.status)
