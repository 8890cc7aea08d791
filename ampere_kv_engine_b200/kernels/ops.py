"""Tensor-level entry points of the kernels.

Each function checks nothing twice (the extension validates its arguments) and allocates
only its result, from the caller's device.  Matrix products are library calls
(:func:`linear`), as they are in the reference (``F.linear`` at ampere_kv/runner.py:64-66,
165, 174-177, 297); everything else on the step's path is a kernel of ``_C``.  There is no
fallback: without the extension these functions raise.
"""

from __future__ import annotations

import math
import os

import torch

from . import build

#: query tokens of one sequence that one attention tile covers (the kernels cut it further as they need)
ATTENTION_Q_TILE = 32

_EXT = None

#: kernels of this package launched since the last reset (the benchmark reports it)
launch_count = 0


def _launched(n: int = 1) -> None:
    global launch_count
    launch_count += n


def ext():
    """The loaded extension module (built on first use)."""
    global _EXT
    if _EXT is None:
        _EXT = build.load()
    return _EXT


def smoke_add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return ext().smoke_add(a, b)


def embedding(ids: torch.Tensor, table: torch.Tensor, status: torch.Tensor | None = None,
              sampled: torch.Tensor | None = None) -> torch.Tensor:
    """float32 residual stream [tokens, hidden] gathered from ``table`` rows.  With ``sampled`` (int32, on the
    device) an id of ``-(r + 1)`` stands for ``sampled[r]``: the token the previous step chose in its row r."""
    hidden = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    ext().embedding(ids, table, hidden, status, sampled)
    _launched()
    return hidden


def add_rmsnorm(hidden: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, rows: torch.Tensor | None = None,
                status: torch.Tensor | None = None) -> torch.Tensor:
    """``hidden += delta`` in place (whole-batch form), then RMSNorm times ``weight``.

    With ``rows`` only those rows are normalised (``hidden`` is left as it is) and the
    result is [len(rows), hidden].
    """
    n = hidden.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, hidden.shape[1]), dtype=out_dtype, device=hidden.device)
    ext().add_rmsnorm(hidden, delta, weight, out, rows, float(eps), status)
    _launched()
    return out


GATE_UP_RUN = 64   # gate and up rows alternate in runs of this many when one GEMM tile is to hold both


def silu_mul(gate_up: torch.Tensor, out_dtype: torch.dtype | None = None, block: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` of [tokens, 2 * intermediate].  Gate and up columns alternate in runs of ``block``
    columns (0: all gate columns first).  A 3-D float32 input is a stack of split-K partial sums that are added
    up first; then ``out_dtype`` names the result's type."""
    if gate_up.dim() == 3:
        out_dtype = out_dtype or torch.bfloat16
    else:
        out_dtype = gate_up.dtype
    out = torch.empty((gate_up.shape[-2], gate_up.shape[-1] // 2), dtype=out_dtype, device=gate_up.device)
    ext().silu_mul(gate_up, out, int(block))
    _launched()
    return out


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, block: int) -> torch.Tensor:
    """One matrix [2 * intermediate, k] whose rows are ``block`` gate rows, then the ``block`` up rows of the same
    outputs, and so on."""
    inter, k = gate.shape
    return torch.stack((gate.view(inter // block, block, k), up.view(inter // block, block, k)), dim=1).reshape(2 * inter, k)


def gated_linear(x: torch.Tensor, gate_up: torch.Tensor, block: int, status: torch.Tensor | None = None) -> torch.Tensor:
    """``silu(x @ gate.T) * (x @ up.T)`` with gate and up rows stored in alternating runs of ``block`` (0: all gate
    rows first).  Few bfloat16 tokens and ``block == GATE_UP_RUN``: one tcgen05 kernel that applies the activation
    to its output tile; otherwise the product and the activation kernel."""
    x, normed, small = _operand(x, gate_up)
    if block == GATE_UP_RUN and small and gate_up.shape[0] % 128 == 0:
        return small_m_gemm(x, gate_up, status=status, gated=True, normed=normed)
    if normed:
        return silu_mul(small_m_gemm(None, gate_up, status=status, normed=normed), torch.bfloat16, block)
    return silu_mul(linear(x, gate_up, partial_ok=True, status=status), x.dtype, block)


def qk_norm_rope_write(qkv, positions, slots, q_weight, k_weight, inv_freq, k_cache, v_cache, *, num_heads,
                       num_kv_heads, head_dim, rotary_dim, eps, want_kv: bool = False, status=None):
    """Per-head RMSNorm of q and k, rotation by position, K/V written to their cache slots.

    Returns q [tokens, heads * head_dim] (and the dense k, v when ``want_kv``).
    """
    n = qkv.shape[-2]
    out_dtype = torch.bfloat16 if qkv.dim() == 3 else qkv.dtype      # 3-D: float32 split-K partial sums
    q_out = torch.empty((n, num_heads * head_dim), dtype=out_dtype, device=qkv.device)
    k_out = v_out = None
    if want_kv:
        k_out = torch.empty((n, num_kv_heads * head_dim), dtype=out_dtype, device=qkv.device)
        v_out = torch.empty_like(k_out)
    ext().qk_norm_rope_write(qkv, positions, slots, q_weight, k_weight, inv_freq, q_out, k_out, v_out, k_cache,
                             v_cache, num_heads, num_kv_heads, head_dim, rotary_dim, float(eps), status)
    _launched()
    return (q_out, k_out, v_out) if want_kv else q_out


def project_qkv(x, w_qkv, bias, positions, slots, q_weight, k_weight, inv_freq, k_cache, v_cache, *, num_heads,
                num_kv_heads, head_dim, rotary_dim, eps, status=None):
    """The q/k/v projection of ``x``, then per-head RMSNorm of q and k, rotation of the first ``rotary_dim`` dims
    by position, and K/V written to their cache slots.  Returns q [tokens, heads * head_dim].

    Few bfloat16 tokens with heads of 128 dims that are rotated whole: one tcgen05 kernel whose 128-row tile is
    one head and does all of it on the tile.  Otherwise the product, then ``qk_norm_rope_write``.
    """
    on_tile = (bias is None and head_dim == 128 and (inv_freq is None or rotary_dim == 128)
               and w_qkv.shape[0] == (num_heads + 2 * num_kv_heads) * 128)
    if on_tile:
        x, normed, small = _operand(x, w_qkv)
        if small:
            q_out = torch.empty((positions.shape[0], num_heads * 128), dtype=torch.bfloat16, device=w_qkv.device)
            ext().small_m_gemm_qkv(x, w_qkv, q_out, positions, slots, q_weight, k_weight, inv_freq, k_cache,
                                   v_cache, num_heads, num_kv_heads, float(eps), _cluster_splits(w_qkv), status,
                                   **normed)
            _launched()
            return q_out
    qkv = linear(x, w_qkv, bias, partial_ok=True, status=status)
    return qk_norm_rope_write(qkv, positions, slots, q_weight, k_weight, inv_freq, k_cache, v_cache,
                              num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                              rotary_dim=rotary_dim, eps=eps, status=status)


def kv_write(k, v, slots, k_cache, v_cache, status=None) -> None:
    ext().kv_write(k, v, slots, k_cache, v_cache, status)
    _launched()


#: streaming multiprocessors assumed when no device can be asked (planning on a host without a GPU): a B200's
FALLBACK_SM_COUNT = 148
_SM_COUNT: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of ``device`` (default: the current CUDA device), asked once per device."""
    if not torch.cuda.is_available():
        return FALLBACK_SM_COUNT
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    if index not in _SM_COUNT:
        _SM_COUNT[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return _SM_COUNT[index]


def attention_q_tile(head_dim: int, group_size: int) -> int:
    """Query tokens per attention tile that suit a mixer of this shape: the tcgen05 prompt kernel's CTAs take
    128 // group tokens (128 rows), so a group that does not divide 128 gets tiles of exactly that many."""
    if head_dim == 128 and 1 <= group_size <= 16 and 128 % group_size:
        return 128 // group_size
    return ATTENTION_Q_TILE


def attention_takes_tensor_cores(dtype: torch.dtype, head_dim: int, group_size: int, page_size: int) -> bool:
    """Whether the TMA + tensor-core attention kernels take these sizes (else the general kernel runs)."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and 1 <= group_size <= 16 and page_size >= 8
            and page_size & (page_size - 1) == 0)


def choose_splits(num_tiles: int, num_kv_heads: int, rows_per_tile: int, max_context: int,
                  tensor_core: bool = False, mean_context: int | None = None, sms: int | None = None) -> int:
    """How many key ranges each decoded token's attention is cut into so that a small batch still fills the GPU
    and a long sequence among short ones does not keep one CTA walking alone.  ``max_context`` / ``mean_context``:
    the keys the longest and the average token of the batch walks (the mean defaults to the maximum).

    The tensor-core decode kernel runs one CTA per (token, kv head, split), four to an SM; the general kernel
    one warp per (token, kv head, 8 rows, split), sixteen to an SM.
    """
    sms = sms or sm_count()
    if tensor_core:
        # 1, 2, 4 or 8 splits (merged inside the kernel by a cluster).  A cost in microseconds, fitted to
        # measurements on B200 (32 q-heads, 8 kv-heads, head size 128, batches of 4 to 64, 1,088 to 8,000 keys,
        # equal and mixed lengths): a CTA spends about 1.1 us on a 32-key block and a fixed 5.5 us (7.5 us in a
        # cluster) on start-up and merge; the GPU holds four CTAs per SM at a time.  With equal lengths all CTAs end
        # together, so a grid that needs a further round of CTAs pays for a whole one; with mixed lengths slots
        # free up all the time and only the fraction counts.  The longest sequences' CTAs start first (the batch
        # layout orders the tiles so), so the step takes the longest walk or the rounds of mean walks, whichever
        # is more, and never less than the bytes need to cross the memory system.
        # Measured (us at 1/2/4/8 splits): batch 8 at 1,088 keys 35/24/15/12; batch 24: 40/27/32/36; batch 64:
        # 48/57/68/95; batch 48 at 4,096 keys 169/172/142/159; batch 64 with 300 to 4,600 keys (mean 2,500):
        # 171/110/119/144; batch 40 likewise: 160/94/75/88; batch 20: 144/81/48/46.
        items, slots = max(1, num_tiles * num_kv_heads), sms * 4
        blocks_max = max(1, (max_context + 31) // 32)
        blocks_mean = blocks_max if mean_context is None else max(1, min(blocks_max, (int(mean_context) + 31) // 32))
        evenness = (blocks_mean / blocks_max) ** 2
        moved = items * blocks_mean * 16384 / 6.0e6       # us for the K/V bytes (heads of 128 dims) at 6 TB/s
        best, best_cost = 1, None
        for i, s in enumerate((1, 2, 4, 8)):
            if s > 1 and blocks_max // s < 2:
                break
            fixed = 5.5 if s == 1 else 7.5
            walk_max = -(-blocks_max // s) * 1.1 + fixed
            walk_mean = -(-blocks_mean // s) * 1.1 + fixed
            rounds = items * s / slots
            rounds += (math.ceil(rounds) - rounds) * evenness
            cost = max(walk_max, rounds * walk_mean, moved) * (1.0 + 0.03 * i)
            if best_cost is None or cost < best_cost:
                best, best_cost = s, cost
        return best
    items, target, min_keys = max(1, num_tiles * num_kv_heads * ((rows_per_tile + 7) // 8)), sms * 16, 128
    if items >= target or max_context <= min_keys:
        return 1
    want = target // items
    return int(max(1, min(want, (max_context + min_keys - 1) // min_keys, 64)))


def paged_attention(q, k_cache, v_cache, block_table, cu_q, ctx_lens, tile_seq, tile_q0, tile_nq, *, num_tiles,
                    q_tile, num_splits, num_heads, num_kv_heads, window, scale, partials=None, status=None,
                    kernel: str = "auto", out=None):
    """Causal attention of the batch's new tokens over the paged cache.  ``kernel``: ``"auto"`` takes the
    tensor-core kernels where they fit (bfloat16, head size 64 or 128; prompt portions at head size 128 and groups
    of up to 16 q-heads on tcgen05) and the general kernel elsewhere; ``"general"`` forces the latter, ``"mma"``
    keeps prompt portions on the mma.sync kernel, ``"tcgen05-narrow"`` / ``"tcgen05-wide"`` pick the form of the
    tcgen05 prompt kernel that the grid's size otherwise decides.  Only the rows of the given tiles are written; with ``out`` they
    go into that tensor (a batch may be covered by two calls with different tile sizes)."""
    if out is None:
        out = torch.empty_like(q)
    if num_splits > 1 and partials is None:
        head_dim = q.shape[1] // num_heads
        partials = torch.empty((q.shape[0] * num_heads * num_splits * (head_dim + 2),), dtype=torch.float32,
                               device=q.device)
    ext().paged_attention(q, k_cache, v_cache, out, block_table, cu_q, ctx_lens, tile_seq, tile_q0, tile_nq,
                          partials, num_tiles, q_tile, num_splits, num_heads, num_kv_heads, int(window or 0),
                          float(scale), status, {"auto": 0, "general": 1, "mma": 2, "tcgen05-narrow": 3, "tcgen05-wide": 4}[kernel])
    _launched(2 if num_splits > 1 else 1)
    return out


_SAMPLE_TICKETS: dict = {}      # per device: zeroed row counters of the sampling kernel (it leaves them zero)


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """int32 token per row: the arg-max where ``temperature`` is 0, else the inverse-CDF draw of
    ``softmax(logits / temperature)`` at ``uniform``.  With ``out`` (int32, contiguous, at least a row each) the
    tokens are written there."""
    rows = logits.shape[0]
    if out is None:
        tokens = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    else:
        if out.dtype != torch.int32 or out.device != logits.device or out.dim() != 1 or out.shape[0] < rows \
                or not out.is_contiguous():
            raise ValueError("sample: out must be a contiguous int32 vector on the logits' device with a row each")
        tokens = out[:rows]
    tickets = _SAMPLE_TICKETS.get(logits.device)
    if tickets is None or tickets.numel() < rows:
        tickets = torch.zeros((max(rows, 512),), dtype=torch.int32, device=logits.device)
        _SAMPLE_TICKETS[logits.device] = tickets
    parts = torch.empty((4 * rows * ext().sample_slices(),), dtype=torch.float32, device=logits.device)
    ext().sample(logits, temperature, uniform, tokens, parts, tickets)
    _launched()
    return tokens


class Summed:
    """What a product leaves behind when it has added its result to the residual stream itself
    (``linear_into_residual``): ``hidden`` holds the sum already, and ``ssq`` [tiles, tokens] the sums of squares
    of its new values per 128-feature tile, from which the next RMS norm needs no pass over ``hidden``."""

    def __init__(self, hidden: torch.Tensor, ssq: torch.Tensor):
        self.hidden, self.ssq = hidden, ssq


class LazyNorm:
    """An RMS norm that is not computed yet: ``hidden * rsqrt(mean(hidden^2) + eps) * weight`` with the sums of
    squares already known (``Summed``).  ``linear``, ``gated_linear`` and ``project_qkv`` take it in place of a
    tensor and let the small-batch product kernel apply it to its token operand; ``materialize`` runs the norm
    kernel."""

    def __init__(self, summed: Summed, weight: torch.Tensor, eps: float, dtype: torch.dtype, status=None):
        self.hidden, self.ssq, self.weight, self.eps, self.dtype, self.status = (
            summed.hidden, summed.ssq, weight, float(eps), dtype, status)

    @property
    def shape(self):
        return self.hidden.shape

    def materialize(self) -> torch.Tensor:
        return add_rmsnorm(self.hidden, None, self.weight, self.eps, self.dtype, status=self.status)


def _operand(x, weight: torch.Tensor):
    """(tensor or None, normed-x keyword arguments of the extension, fused?) for a token operand that may be a
    ``LazyNorm``.  A lazy norm that the small-batch kernel cannot take is materialized."""
    if not isinstance(x, LazyNorm):
        return x, {}, _takes_small_m(x, weight)
    h = x.hidden
    fused = (use_small_m_gemm and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and h.is_cuda
             and h.shape[0] <= SMALL_M_LIMIT and h.is_contiguous() and weight.is_contiguous()
             and h.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and x.weight.data_ptr() % 16 == 0
             and h.shape[1] == weight.shape[1]
             and ext().small_m_gemm_supported(h.shape[0], weight.shape[0], weight.shape[1]))
    if not fused:
        t = x.materialize()
        return t, {}, _takes_small_m(t, weight)
    return None, {"nx_hidden": h, "nx_ssq": x.ssq, "nx_weight": x.weight, "nx_eps": x.eps}, True


#: products of at most this many bfloat16 tokens go through the package's own tcgen05 kernel: all it takes.
#: Measured per decode step on B200 against the library product with the row-wise kernels around it: 5.08 against
#: 5.21 ms at 40 tokens, 5.21 against 5.36 ms at 56, 5.17 against 5.37 ms at 64.
SMALL_M_LIMIT = 64
use_small_m_gemm = True
#: up to this many tokens a decode branch adds to the residual stream inside its last product and the next product
#: applies the norm to its own token operand.  Every CTA of that product re-reads the float32 stream for its K
#: range, which grows with the tokens: measured per decode step on B200 against the norm as a kernel of its own,
#: 3.64 against 3.67 ms at 12 tokens, 3.71 against 3.76 ms at 16, but 4.98 against 4.25 ms at 32 and 7.0 against
#: 5.2 ms at 64.
LAZY_NORM_LIMIT = 16
#: hand split-K partial sums to the consuming kernel instead of adding them up inside the product kernel
prefer_partials = False


def _cluster_splits(weight: torch.Tensor) -> int:
    splits = min(ext().small_m_gemm_splits(weight.shape[0], weight.shape[1]), (weight.shape[1] + 63) // 64)
    while splits not in (1, 2, 4, 8):
        splits -= 1
    return splits


def small_m_gemm(x: torch.Tensor | None, weight: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                 splits: int | None = None, parts: bool = False, status: torch.Tensor | None = None,
                 gated: bool = False, normed: dict | None = None) -> torch.Tensor:
    """``x @ weight.T`` for 1..64 bfloat16 tokens on the tcgen05 tensor cores, K cut into ``splits`` ranges.

    Default: [tokens, features] in ``out_dtype`` (float32 or bfloat16); the splits (1, 2, 4 or 8 CTAs of a
    cluster) add their float32 partial tiles up through distributed shared memory.  ``parts=True``: the float32
    partial sums themselves, [splits, tokens, features], for a consumer kernel that adds them up.
    ``gated=True``: ``weight`` holds gate and up rows in alternating runs of 64 and the result is
    ``silu(gate) * up``, [tokens, features / 2] bfloat16.  ``normed`` (with ``x`` None): the kernel makes its token
    operand from a residual stream and its sums of squares (``LazyNorm``).
    """
    normed = normed or {}
    tokens = x.shape[0] if x is not None else normed["nx_hidden"].shape[0]
    kb_total = (weight.shape[1] + 63) // 64
    if splits is None:
        splits = ext().small_m_gemm_splits(weight.shape[0], weight.shape[1])
    splits = max(1, min(int(splits), kb_total))
    if parts:
        out = torch.empty((splits, tokens, weight.shape[0]), dtype=torch.float32, device=weight.device)
    else:
        while splits not in (1, 2, 4, 8):
            splits -= 1
        out = torch.empty((tokens, weight.shape[0] // 2 if gated else weight.shape[0]),
                          dtype=torch.bfloat16 if gated else out_dtype, device=weight.device)
    ext().small_m_gemm(x, weight, out, splits, status, gated, **normed)
    _launched()
    return out


def linear_into_residual(x: torch.Tensor, weight: torch.Tensor, hidden: torch.Tensor,
                         status: torch.Tensor | None = None) -> Summed | None:
    """``hidden += bfloat16(x @ weight.T)`` inside the small-batch product kernel, which also leaves the sums of
    squares of the new ``hidden`` for the next norm.  None when that kernel does not take the sizes: the caller
    then computes the product and hands it to the norm as a pending delta."""
    if not (x.shape[0] <= LAZY_NORM_LIMIT and _takes_small_m(x, weight) and hidden.dtype == torch.float32
            and hidden.is_contiguous() and hidden.shape == (x.shape[0], weight.shape[0])):
        return None
    ssq = torch.empty(((weight.shape[0] + 127) // 128, x.shape[0]), dtype=torch.float32, device=x.device)
    ext().small_m_gemm_residual(x, weight, hidden, ssq, _cluster_splits(weight), status)
    _launched()
    return Summed(hidden, ssq)


def _takes_small_m(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (use_small_m_gemm and x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and x.dim() == 2 and x.shape[0] <= SMALL_M_LIMIT and x.is_contiguous() and weight.is_contiguous()
            and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and ext().small_m_gemm_supported(x.shape[0], weight.shape[0], weight.shape[1]))


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           out_dtype: torch.dtype | None = None, partial_ok: bool = False,
           status: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)``, float32 accumulation.

    Few bfloat16 tokens (decode steps) go through this package's tcgen05 kernel; everything else is the library
    GEMM, as in the reference.  With ``partial_ok`` the result may be a 3-D float32 stack
    ``[parts, tokens, features]`` of split-K partial sums, for a consumer kernel that adds them up;
    ``out_dtype=torch.float32`` keeps the accumulator's precision in the result (used for the logits).
    ``x`` may be a ``LazyNorm``.
    """
    if isinstance(x, LazyNorm) and bias is not None:
        x = x.materialize()
    x, normed, small = _operand(x, weight)
    if bias is None and small:
        if partial_ok and prefer_partials and not normed:
            return small_m_gemm(x, weight, parts=True, status=status)
        return small_m_gemm(x, weight, out_dtype=out_dtype or torch.bfloat16, status=status, normed=normed)
    if out_dtype is not None and out_dtype != x.dtype:
        out = torch.mm(x, weight.t(), out_dtype=out_dtype)
        if bias is not None:
            out += bias.to(out_dtype)
        return out
    return torch.nn.functional.linear(x, weight, bias)


# ----------------------------------------------------------------------------- chains of products in one kernel

#: a decode step of at most this many bfloat16 tokens may run the tail of each layer and the head of the next (output
#: projection, gate/up, down, the next q/k/v projection) as ONE persistent kernel that never stops streaming weights
STREAM_LIMIT = 8
#: Off unless AKV_STREAM_PHASES=1: measured on B200 at the benchmark model's sizes the chain of a layer takes 100 us
#: in the persistent kernel against 76 us as four kernels (a decode step of 8 tokens: 4.26 ms against 3.37 ms).  Its
#: weights do stream at the memory's rate (0.37 us per 16 KB block per SM), but each of the three places where a
#: phase needs the one before it finished everywhere costs 5 to 6 us (the last tile's sum over the cluster, a
#: releasing count in global memory, the slowest SM, the operand built anew) against the 3.7 us of weights that the
#: ring holds, and whole tiles per cluster of four leave a share of the SMs idle at the end of each phase (48 tiles
#: over 33 clusters).  Asking the L2 for blocks ahead of the ring made it slower still.
use_stream_phases = os.environ.get("AKV_STREAM_PHASES", "0") == "1"
_STREAM_SYNC_INTS = 1 << 16


class _StreamScratch:
    """Per device: sums of squares, whatever scratch the kernel asks for and its zeroed counters.  The counters
    are handed out slice by slice and zeroed again at the start of every step (``stream_begin_step``)."""

    def __init__(self, device):
        self.device = device
        self.ssq = torch.empty((1,), dtype=torch.float32, device=device)
        self.parts = torch.empty((1,), dtype=torch.float32, device=device)
        self.sync = torch.zeros((_STREAM_SYNC_INTS,), dtype=torch.int32, device=device)
        self.cursor = 0
        self.high_water = 0      # counters ever handed out: a replayed graph may have used them behind our back


_STREAM_SCRATCH: dict = {}


def _device_key(device) -> torch.device:
    """``cuda`` and ``cuda:0`` name the same device: always the form with an index."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def _stream_scratch(device) -> _StreamScratch:
    key = _device_key(device)
    if key not in _STREAM_SCRATCH:
        _STREAM_SCRATCH[key] = _StreamScratch(key)
    return _STREAM_SCRATCH[key]


def stream_begin_step(device) -> None:
    """Zero every counter the chained-product kernel has ever been handed on this device (one small memset; nothing
    before the kernel's first use).  Called at the start of every step, so a captured step carries its own."""
    if not _STREAM_SCRATCH:
        return
    scratch = _STREAM_SCRATCH.get(_device_key(device))
    if scratch is not None and scratch.high_water:
        scratch.sync[:scratch.high_water].zero_()
        scratch.cursor = 0


def stream_phases(hidden: torch.Tensor, phases: list[dict], status: torch.Tensor | None = None,
                  trace: torch.Tensor | None = None) -> None:
    """Run ``phases`` (1 to 4 products, each depending on the one before) on the float32 residual stream ``hidden``
    [tokens <= 16, width] in one persistent kernel.  A phase is a dict: ``w`` [features, k] bfloat16; ``x``
    [tokens, k] bfloat16, or ``norm_weight`` and ``eps`` for the RMS norm of ``hidden``; ``epilogue`` "residual" (adds
    the product, rounded to bfloat16, into ``hidden``), "gated" (``out`` = silu(gate) * up over rows alternating in
    runs of 64), "plain" (``out``) or "qkv" (the arguments of the fused q/k/v projection).  Outputs are written into
    the tensors the phases name."""
    scratch = _stream_scratch(hidden.device)
    part_floats, sync_ints = ext().stream_phases_scratch([(int(p["w"].shape[0]), int(p["w"].shape[1])) for p in phases])
    ssq_floats = (hidden.shape[1] + 127) // 128 * 16
    if scratch.ssq.numel() < ssq_floats:
        scratch.ssq = torch.empty((ssq_floats,), dtype=torch.float32, device=hidden.device)
    if scratch.parts.numel() < part_floats:
        scratch.parts = torch.empty((part_floats,), dtype=torch.float32, device=hidden.device)
    if scratch.cursor + sync_ints > scratch.sync.numel():
        raise RuntimeError("the chained-product kernel ran out of counters: stream_begin_step() was not called "
                           "between steps")
    sync = scratch.sync[scratch.cursor:scratch.cursor + sync_ints]
    scratch.cursor += sync_ints
    scratch.high_water = max(scratch.high_water, scratch.cursor)
    ext().stream_phases(hidden, phases, scratch.ssq, scratch.parts, sync, status, trace)
    _launched()


def stream_takes(tokens: int, *weights: torch.Tensor) -> bool:
    """Whether the chained-product kernel takes a step of ``tokens`` tokens over these matrices."""
    return (use_stream_phases and 1 <= tokens <= STREAM_LIMIT and all(
        w is not None and w.is_cuda and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous()
        and w.data_ptr() % 16 == 0 and w.shape[1] % 8 == 0 and w.shape[1] >= 64 for w in weights))


class PendingPhases:
    """Products that are decided but not launched yet: the tail of one layer (output projection, feed-forward) waits
    here for the head of the next (its q/k/v projection) so that all of them go into one launch of the
    chained-product kernel.  Whoever needs the residual stream itself calls :meth:`launch` first."""

    def __init__(self, hidden: torch.Tensor, status: torch.Tensor | None = None):
        self.hidden, self.status = hidden, status
        self.phases: list[dict] = []
        self._max = None

    def room(self, count: int = 1) -> bool:
        if self._max is None:
            self._max = int(ext().stream_phases_max())
        return len(self.phases) + count <= self._max

    def add(self, phase: dict) -> None:
        if not self.room():
            self.launch()
        self.phases.append(phase)

    def launch(self) -> None:
        if self.phases:
            stream_phases(self.hidden, self.phases, status=self.status)
            self.phases = []


class StreamNorm:
    """An RMS norm of the residual stream that is not computed: the consumer adds a phase whose token operand the
    chained-product kernel makes from the stream itself, after the phases queued before it."""

    def __init__(self, pending: PendingPhases, weight: torch.Tensor, eps: float, dtype: torch.dtype):
        self.pending, self.weight, self.eps, self.dtype = pending, weight, float(eps), dtype

    @property
    def hidden(self) -> torch.Tensor:
        return self.pending.hidden

    @property
    def shape(self):
        return self.pending.hidden.shape

    def normed_phase(self, w: torch.Tensor, **epilogue) -> dict:
        return dict(w=w, norm_weight=self.weight, eps=self.eps, **epilogue)

    def materialize(self) -> torch.Tensor:
        """Launch what is queued and run the norm kernel after all."""
        self.pending.launch()
        return add_rmsnorm(self.pending.hidden, None, self.weight, self.eps, self.dtype, status=self.pending.status)
