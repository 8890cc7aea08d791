"""A stand-in for the CUDA extension, for tests that run without a GPU.

It has the extension's functions with the same arguments and writes the same outputs, computed
with plain tensor operations on whatever device the tensors are on.  Tests install it with
``monkeypatch.setattr(ops, "_EXT", FakeExt())`` to drive the engine's host logic (batch layout,
cache manager, step function, scheduler, replay) on the CPU.  The package itself never uses it:
without the real extension the product path raises.
"""

from __future__ import annotations

import math

import torch


class FakeExt:
    def smoke_add(self, a, b):
        return a + b

    def embedding(self, ids, table, hidden, status=None, sampled=None):
        ids = ids.long()
        if sampled is not None:
            ids = torch.where(ids < 0, sampled.long()[(-ids - 1).clamp(min=0)], ids)
        hidden.copy_(table[ids].float())

    def add_rmsnorm(self, hidden, delta, weight, out, rows, eps, status=None):
        if delta is not None and delta.dim() == 3:
            delta = delta.sum(0)
        if rows is None:
            if delta is not None:
                hidden += delta.float()
            x = hidden
        else:
            x = hidden[rows.long()]
            if delta is not None:
                x = x + delta[rows.long()].float()
        inv = torch.rsqrt(x.square().mean(-1, keepdim=True) + eps)
        out.copy_((x * inv * weight).to(out.dtype))

    def silu_mul(self, gate_up, out, block=0):
        if gate_up.dim() == 3:
            gate_up = gate_up.sum(0)
        inter = gate_up.shape[1] // 2
        block = block or inter
        pairs = gate_up.float().view(gate_up.shape[0], inter // block, 2, block)
        g, u = pairs[:, :, 0].reshape(-1, inter), pairs[:, :, 1].reshape(-1, inter)
        out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))

    def qk_norm_rope_write(self, qkv, positions, slots, q_weight, k_weight, inv_freq, q_out, k_out, v_out, k_cache,
                           v_cache, num_heads, num_kv_heads, head_dim, rotary_dim, eps, status=None):
        if qkv.dim() == 3:
            qkv = qkv.sum(0)
        n = qkv.shape[0]
        x = qkv.float().view(n, num_heads + 2 * num_kv_heads, head_dim)
        q, k, v = x[:, :num_heads], x[:, num_heads:num_heads + num_kv_heads], x[:, num_heads + num_kv_heads:]

        def norm(t, w):
            if w is None:
                return t
            return t * torch.rsqrt(t.square().mean(-1, keepdim=True) + eps) * w

        def rotate(t):
            if inv_freq is None or rotary_dim == 0:
                return t
            ang = positions.float()[:, None] * inv_freq[None, :]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            half = rotary_dim // 2
            a, b = t[..., :half], t[..., half:rotary_dim]
            return torch.cat((a * cos - b * sin, b * cos + a * sin, t[..., rotary_dim:]), dim=-1)

        q, k = rotate(norm(q, q_weight)), rotate(norm(k, k_weight))
        q_out.copy_(q.reshape(n, -1).to(q_out.dtype))
        if k_out is not None:
            k_out.copy_(k.reshape(n, -1).to(k_out.dtype))
        if v_out is not None:
            v_out.copy_(v.reshape(n, -1).to(v_out.dtype))
        if k_cache is not None and slots is not None:
            self._write(k.to(k_cache.dtype), v.to(v_cache.dtype), slots, k_cache, v_cache)

    @staticmethod
    def _write(k, v, slots, k_cache, v_cache):
        page_size = k_cache.shape[2]
        keep = slots >= 0
        s = slots[keep].long()
        k_cache[s // page_size, :, s % page_size] = k[keep]
        v_cache[s // page_size, :, s % page_size] = v[keep]

    def kv_write(self, k, v, slots, k_cache, v_cache, status=None):
        nkv, d = k_cache.shape[1], k_cache.shape[3]
        self._write(k.view(-1, nkv, d), v.view(-1, nkv, d), slots, k_cache, v_cache)

    def paged_attention(self, q, k_cache, v_cache, out, block_table, cu_q, ctx_lens, tile_seq, tile_q0, tile_nq,
                        partials, num_tiles, q_tile, num_splits, num_heads, num_kv_heads, window, scale, status=None,
                        kernel=0):
        page_size, d = k_cache.shape[2], k_cache.shape[3]
        group = num_heads // num_kv_heads
        cu = cu_q.tolist()
        for s, ctx in enumerate(ctx_lens.tolist()):
            q0, q1 = cu[s], cu[s + 1]
            n = q1 - q0
            first_pos = ctx - n
            lo = max(0, first_pos - window + 1) if window else 0
            keys = torch.arange(lo, ctx)
            pages = block_table[s].long()[keys // page_size]
            assert (pages >= 0).all(), "attention would read a page that is not held"
            k = k_cache[pages, :, keys % page_size].float()     # [keys, nkv, d]
            v = v_cache[pages, :, keys % page_size].float()
            qs = q[q0:q1].float().view(n, num_heads, d)
            scores = torch.einsum("thd,shd->hts", qs, k.repeat_interleave(group, dim=1)) * scale
            pos = torch.arange(first_pos, ctx)[:, None]
            visible = keys[None, :] <= pos
            if window:
                visible &= keys[None, :] > pos - window
            scores = scores.masked_fill(~visible[None], -math.inf)
            o = torch.einsum("hts,shd->thd", torch.softmax(scores, -1), v.repeat_interleave(group, dim=1))
            out[q0:q1] = o.reshape(n, -1).to(out.dtype)

    def sample_slices(self):
        return 8

    def sample(self, logits, temperature, uniform, tokens, parts=None, tickets=None):
        for r in range(logits.shape[0]):
            t = float(temperature[r])
            if t <= 0:
                tokens[r] = int(logits[r].argmax())
                continue
            p = torch.softmax(logits[r].double() / t, -1)
            cdf = torch.cumsum(p, -1)
            target = float(uniform[r]) * float(cdf[-1])
            tokens[r] = min(int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True)),
                            logits.shape[1] - 1)
