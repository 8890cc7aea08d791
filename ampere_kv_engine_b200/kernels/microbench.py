"""Times one kernel at a time on the GPU, with CUDA events, on inputs larger than L2.

    python -m ampere_kv_engine_b200.kernels.microbench gemm --tokens 8 --features 24576 --k 4096 [--gated]
    python -m ampere_kv_engine_b200.kernels.microbench decode-attention --batch 64 --context 1152
    python -m ampere_kv_engine_b200.kernels.microbench prefill-attention --tokens 2048
    python -m ampere_kv_engine_b200.kernels.microbench norm --tokens 2048
    python -m ampere_kv_engine_b200.kernels.microbench chain --tokens 8 [--trace]

The counterpart of the reference's kernel micro-benchmark (``python -m ampere_kv.paged_decode --benchmark``,
ampere_kv/paged_decode.py:19-100, CUDA-event windows at 64/256/1024/4096 keys).  Each case cycles through
enough distinct copies of its large operand that no call finds it in the 126 MB L2, warms up, then reports
the mean time per call and the achieved bytes or FLOPs per second.  It is also the small, self-ending
workload that the profiler captures are taken on.
"""

from __future__ import annotations

import argparse
import json
import sys

import torch

from . import ops

L2_BYTES = 126 * 1024 * 1024


def timed(fn, calls: int, warmup: int = 3) -> float:
    """Mean microseconds per call of ``fn(i)``."""
    for i in range(warmup):
        fn(i)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(calls):
        fn(warmup + i)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1000.0 / calls


def timed_graph(fn, calls: int, warmup: int = 3) -> float:
    """Mean microseconds per call of ``fn(i)`` with the calls captured in one CUDA graph: the figure for kernels
    so short that launching them one by one from Python would measure the host."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(calls):
            fn(warmup + i)
    graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1000.0 / calls


def copies_for(nbytes: int) -> int:
    return max(2, (2 * L2_BYTES + nbytes - 1) // nbytes + 1)


def bench_gemm(args) -> dict:
    g = torch.Generator(device="cuda").manual_seed(0)
    n = copies_for(args.features * args.k * 2)
    weights = [torch.randn(args.features, args.k, generator=g, device="cuda", dtype=torch.bfloat16) * args.k ** -0.5
               for _ in range(n)]
    x = torch.randn(args.tokens, args.k, generator=g, device="cuda", dtype=torch.bfloat16)
    out = {}
    small = args.tokens <= 64
    if small and args.gated:
        # the weight read as gate and up rows in alternating runs of 64; the kernel applies SiLU-mul to its tile
        out["tcgen05_us"] = timed(lambda i: ops.small_m_gemm(x, weights[i % n], gated=True), args.calls)
        full = (x.float() @ weights[0].float().t()).to(torch.bfloat16).float().view(args.tokens, -1, 2, 64)
        ref = (torch.nn.functional.silu(full[:, :, 0]) * full[:, :, 1]).reshape(args.tokens, -1)
        got = ops.small_m_gemm(x, weights[0], gated=True).float()
        out["max_abs_error"] = float((got - ref).abs().max())
    elif small:
        out["tcgen05_us"] = timed(lambda i: ops.small_m_gemm(x, weights[i % n]), args.calls)
        ref = x.float() @ weights[0].float().t()
        got = ops.small_m_gemm(x, weights[0], out_dtype=torch.float32)
        out["max_abs_error"] = float((got - ref).abs().max())
    out["library_us"] = timed(lambda i: torch.nn.functional.linear(x, weights[i % n]), args.calls)
    nbytes = args.features * args.k * 2
    for key in ("tcgen05_us", "library_us"):
        if key in out:
            out[key.replace("_us", "_gbs")] = round(nbytes / out[key] / 1e3, 1)
            out[key.replace("_us", "_tflops")] = round(2.0 * args.tokens * args.features * args.k / out[key] / 1e6, 2)
    out["splits"] = ops.ext().small_m_gemm_splits(args.features, args.k) if small else None
    return out


def _paged_case(batch: int, context: int, q_len: int, heads: int, kv_heads: int, head_dim: int, page: int, copies: int):
    """``copies`` independent page pools holding ``batch`` sequences of ``context`` keys each."""
    g = torch.Generator(device="cuda").manual_seed(1)
    pages_per_seq = (context + page - 1) // page
    pool = batch * pages_per_seq
    caches = [(torch.randn(pool, kv_heads, page, head_dim, generator=g, device="cuda", dtype=torch.bfloat16),
               torch.randn(pool, kv_heads, page, head_dim, generator=g, device="cuda", dtype=torch.bfloat16))
              for _ in range(copies)]
    table = torch.randperm(pool, generator=g, device="cuda").to(torch.int32).view(batch, pages_per_seq)
    n = batch * q_len
    q = torch.randn(n, heads * head_dim, generator=g, device="cuda", dtype=torch.bfloat16)
    cu = torch.arange(0, n + 1, q_len, device="cuda", dtype=torch.int32)
    ctx = torch.full((batch,), context, device="cuda", dtype=torch.int32)
    tile_rows = 1 if q_len == 1 else ops.ATTENTION_Q_TILE
    tiles = [(s, s * q_len + q0, min(tile_rows, q_len - q0)) for s in range(batch) for q0 in range(0, q_len, tile_rows)]
    cols = [torch.tensor([t[i] for t in tiles], device="cuda", dtype=torch.int32) for i in range(3)]
    return caches, table, q, cu, ctx, cols, tile_rows


def bench_attention(args, q_len: int, batch: int, context: int) -> dict:
    kv_bytes = batch * context * args.kv_heads * args.head_dim * 2 * 2
    copies = copies_for(kv_bytes)
    caches, table, q, cu, ctx, tiles, tile_rows = _paged_case(batch, context, q_len, args.heads, args.kv_heads,
                                                              args.head_dim, args.page_size, copies)
    group = args.heads // args.kv_heads
    out = {}
    for kernel in ("auto", "mma", "general"):
        tensor_core = kernel != "general" and ops.attention_takes_tensor_cores(torch.bfloat16, args.head_dim, group,
                                                                            args.page_size)
        splits = args.splits or (1 if q_len > 1 and tensor_core else ops.choose_splits(
            len(tiles[0]), args.kv_heads, tile_rows * group, context, tensor_core))

        def run(i, kernel=kernel, splits=splits):
            k_cache, v_cache = caches[i % copies]
            return ops.paged_attention(q, k_cache, v_cache, table, cu, ctx, tiles[0], tiles[1], tiles[2],
                                       num_tiles=len(tiles[0]), q_tile=tile_rows, num_splits=splits,
                                       num_heads=args.heads, num_kv_heads=args.kv_heads, window=0,
                                       scale=args.head_dim ** -0.5, kernel=kernel)
        if kernel == "general" and q_len > 1 and not args.with_general:
            continue
        if kernel == "mma" and q_len == 1:
            continue
        us = timed(run, args.calls)
        out[f"{kernel}_us"] = us
        out[f"{kernel}_splits"] = splits
        if q_len == 1:
            out[f"{kernel}_gbs"] = round(kv_bytes / us / 1e3, 1)
        else:
            flops = 4.0 * args.heads * args.head_dim * batch * q_len * (context - q_len + (q_len + 1) / 2)
            out[f"{kernel}_tflops"] = round(flops / us / 1e6, 1)
    return out


def bench_rowwise(args) -> dict:
    g = torch.Generator(device="cuda").manual_seed(2)
    n, h, inter = args.tokens, args.hidden, args.intermediate
    copies = copies_for(n * h * 10)
    hidden = [torch.randn(n, h, generator=g, device="cuda") for _ in range(copies)]
    delta = [torch.randn(n, h, generator=g, device="cuda").to(torch.bfloat16) for _ in range(copies)]
    weight = torch.ones(h, device="cuda")
    out = {"norm_us": timed_graph(lambda i: ops.add_rmsnorm(hidden[i % copies], delta[i % copies], weight, 1e-6,
                                                      torch.bfloat16), args.calls)}
    out["norm_gbs"] = round(n * h * (4 + 2 + 4 + 2) / out["norm_us"] / 1e3, 1)
    gate_up = [torch.randn(n, 2 * inter, generator=g, device="cuda").to(torch.bfloat16)
               for _ in range(copies_for(n * inter * 6))]
    out["silu_mul_us"] = timed_graph(lambda i: ops.silu_mul(gate_up[i % len(gate_up)]), args.calls)
    out["silu_mul_gbs"] = round(n * inter * 6 / out["silu_mul_us"] / 1e3, 1)
    heads, kv, d = args.heads, args.kv_heads, args.head_dim
    qkv = [torch.randn(n, (heads + 2 * kv) * d, generator=g, device="cuda").to(torch.bfloat16)
           for _ in range(copies_for(n * (heads + 2 * kv) * d * 4))]
    pages = (n + args.page_size - 1) // args.page_size + 1
    k_cache = torch.zeros(pages, kv, args.page_size, d, device="cuda", dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    positions = torch.arange(n, device="cuda", dtype=torch.int32)
    ones = torch.ones(d, device="cuda")
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2).float() / d))).cuda()
    out["qk_rope_write_us"] = timed_graph(lambda i: ops.qk_norm_rope_write(
        qkv[i % len(qkv)], positions, positions, ones, ones, inv_freq, k_cache, v_cache, num_heads=heads,
        num_kv_heads=kv, head_dim=d, rotary_dim=d, eps=1e-6), args.calls)
    out["qk_rope_write_gbs"] = round(n * (heads + 2 * kv) * d * 4 / out["qk_rope_write_us"] / 1e3, 1)
    return out


def bench_chain(args) -> dict:
    """A layer's chain of products (output projection + residual -> norm + gate/up + SiLU-mul -> down + residual ->
    norm + next q/k/v + rotation + cache write) as ONE launch of the chained-product kernel against the four
    separate kernels, each on three copies of the weights in turn.  ``--trace``: where the persistent kernel's
    CTAs are in each phase, from its nanosecond stamps (minimum / median / maximum over the CTAs, microseconds)."""
    g = torch.Generator(device="cuda").manual_seed(3)
    t, h, inter, heads, kv = args.tokens, args.hidden, args.intermediate, args.heads, args.kv_heads
    rand = lambda *shape, scale=0.02: torch.randn(*shape, generator=g, device="cuda") * scale
    copies = []
    for _ in range(3):
        gate_up = ops.interleave_gate_up(rand(inter, h).bfloat16(), rand(inter, h).bfloat16(), ops.GATE_UP_RUN)
        copies.append((rand(h, heads * 128).bfloat16(), gate_up.contiguous(), rand(h, inter).bfloat16(),
                       rand((heads + 2 * kv) * 128, h).bfloat16()))
    norm_a, norm_b = 1 + rand(h, scale=0.1), 1 + rand(h, scale=0.1)
    qn, kn = 1 + rand(128, scale=0.1), 1 + rand(128, scale=0.1)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, 128, 2).float() / 128))).cuda()
    hidden = rand(t, h, scale=1.0)
    attn_out = rand(t, heads * 128, scale=1.0).bfloat16()
    positions = torch.arange(1000, 1000 + t, device="cuda", dtype=torch.int32)
    slots = torch.arange(t, device="cuda", dtype=torch.int32)
    k_cache = torch.zeros((t // args.page_size + 2, kv, args.page_size, 128), device="cuda", dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    act = torch.empty((t, inter), dtype=torch.bfloat16, device="cuda")
    q_out = torch.empty((t, heads * 128), dtype=torch.bfloat16, device="cuda")

    def phases(i):
        o, gu, down, qkv = copies[i % 3]
        return [dict(w=o, x=attn_out, epilogue="residual"),
                dict(w=gu, norm_weight=norm_a, eps=1e-6, epilogue="gated", out=act),
                dict(w=down, x=act, epilogue="residual"),
                dict(w=qkv, norm_weight=norm_b, eps=1e-6, epilogue="qkv", q_out=q_out, positions=positions,
                     slots=slots, q_weight=qn, k_weight=kn, inv_freq=inv_freq, k_cache=k_cache, v_cache=v_cache,
                     num_heads=heads, num_kv_heads=kv, qk_eps=1e-6)]
    lists = [phases(i) for i in range(3)]

    def chained(i):
        ops.stream_begin_step("cuda")
        ops.stream_phases(hidden, lists[i % 3], status=status)

    def separate(i):
        o, gu, down, qkv = copies[i % 3]
        summed = ops.linear_into_residual(attn_out, o, hidden, status=status)
        x = ops.LazyNorm(summed, norm_a, 1e-6, torch.bfloat16, status)
        a = ops.gated_linear(x, gu, ops.GATE_UP_RUN, status=status)
        summed = ops.linear_into_residual(a, down, hidden, status=status)
        x = ops.LazyNorm(summed, norm_b, 1e-6, torch.bfloat16, status)
        ops.project_qkv(x, qkv, None, positions, slots, qn, kn, inv_freq, k_cache, v_cache, num_heads=heads,
                        num_kv_heads=kv, head_dim=128, rotary_dim=128, eps=1e-6, status=status)

    nbytes = sum(w.numel() * 2 for w in copies[0])
    out = {"weight_mb": round(nbytes / 1e6, 1), "chained_us": timed_graph(chained, args.calls),
           "separate_us": timed_graph(separate, args.calls)}
    out["chained_gbs"] = round(nbytes / out["chained_us"] / 1e3, 1)
    out["separate_gbs"] = round(nbytes / out["separate_us"] / 1e3, 1)
    if args.trace:
        grid = int(ops.ext().stream_phases_grid())
        trace = torch.zeros((grid, 4, 16), dtype=torch.int64, device="cuda")
        ops.stream_begin_step("cuda")
        ops.stream_phases(hidden, lists[0], status=status, trace=trace)
        torch.cuda.synchronize()
        stamps = trace.cpu().double()
        stamps = (stamps - stamps[stamps > 0].min()) / 1000.0
        names = ("first copy", "last copy", "first mma", "last mma", "operand may start", "operand first group",
                 "operand done", "last epilogue")
        out["trace_us"] = {f"phase{ph} {name}": [round(float(f(stamps[:, ph, e])), 2) for f in
                                               (torch.min, torch.median, torch.max)]
                           for ph in range(4) for e, name in enumerate(names)}
    out["status"] = int(status.item())
    return out


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("kernel", choices=("gemm", "decode-attention", "prefill-attention", "norm", "chain"))
    parser.add_argument("--tokens", type=int, default=8)
    parser.add_argument("--features", type=int, default=24576)
    parser.add_argument("--k", type=int, default=4096)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=1152)
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv-heads", type=int, default=8)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--hidden", type=int, default=4096)
    parser.add_argument("--intermediate", type=int, default=12288)
    parser.add_argument("--splits", type=int, default=0, help="key splits of decode attention (0 = the engine's choice)")
    parser.add_argument("--with-general", action="store_true", help="also time the general attention kernel on prompts")
    parser.add_argument("--gated", action="store_true", help="gemm: the SiLU-mul epilogue (gate/up rows in runs of 64)")
    parser.add_argument("--trace", action="store_true", help="chain: the persistent kernel's per-phase time stamps")
    parser.add_argument("--calls", type=int, default=50)
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        raise RuntimeError("the micro-benchmark needs a CUDA device")
    ops.ext()
    if args.kernel == "gemm":
        result = bench_gemm(args)
    elif args.kernel == "decode-attention":
        result = bench_attention(args, 1, args.batch, args.context)
    elif args.kernel == "chain":
        result = bench_chain(args)
    elif args.kernel == "prefill-attention":
        result = bench_attention(args, args.tokens, 1, max(args.context, args.tokens) if args.context > args.tokens
                                 else args.tokens)
    else:
        result = bench_rowwise(args)
    shape = {k: v for k, v in vars(args).items() if k not in ("calls", "with_general")}
    print(json.dumps({"shape": shape, **{k: (round(v, 2) if isinstance(v, float) else v) for k, v in result.items()}}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
