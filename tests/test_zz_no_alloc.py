"""The entry point for callers that must not allocate device memory (csrc/noalloc_entry.h).

Some hosts of this library cannot call cudaMalloc: their device memory was handed out in full by a pool of their
own, or they sit in a real-time loop or a graph capture where the allocator is off limits.  For them the library
exports one C function that runs the split paged attention with its workspace in a fixed 16 MiB array inside the
library.  This test calls it the way such a host does, through the exported C symbol with raw device pointers,
twice in a row, and compares with the ordinary entry point (whose Python wrapper allocates the workspace).

The file is named so that it is collected last: if it fails, a run that stops at the first failure has already
run every other test.  It does not depend on them: it also passes alone in a fresh process.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from ampere_kv_engine_b200.kernels import build, ops
    ops.ext()                                   # builds the extension if needed and loads libtorch first
    lib = ctypes.CDLL(build.build(verbose=False))
    fn = lib.akv_paged_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_int64] + [ctypes.c_int] * 9 + [ctypes.c_int64, ctypes.c_int,
                                                                                    ctypes.c_float, ctypes.c_int,
                                                                                    ctypes.c_void_p, ctypes.c_void_p]
    lib.akv_noalloc_last_error.restype = ctypes.c_char_p
    lib.akv_noalloc_scratch_bytes.restype = ctypes.c_int64
    return lib, ops


def _case(dtype, seed, nh=8, nkv=2, d=64, page=16, ctxs=(300, 17, 129, 64, 1)):
    g = torch.Generator().manual_seed(seed)
    pages_per = [(c + page - 1) // page for c in ctxs]
    pool = sum(pages_per) + 3
    k_cache = torch.randn(pool, nkv, page, d, generator=g).to(dtype).cuda()
    v_cache = torch.randn(pool, nkv, page, d, generator=g).to(dtype).cuda()
    order = torch.randperm(pool, generator=g).tolist()
    table = torch.full((len(ctxs), max(pages_per)), -1, dtype=torch.int32)
    for s, n in enumerate(pages_per):
        for lp in range(n):
            table[s, lp] = order.pop()
    q = torch.randn(len(ctxs), nh * d, generator=g).to(dtype).cuda()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    n = len(ctxs)
    return dict(q=q, k=k_cache, v=v_cache, table=table.cuda(), cu=i32(list(range(n + 1))), ctx=i32(list(ctxs)),
                tile_seq=i32(list(range(n))), tile_q0=i32(list(range(n))), tile_nq=i32([1] * n), nh=nh, nkv=nkv, d=d,
                page=page, pool=pool, n=n)


def _call(lib, c, out, splits, dtype):
    code = 0 if dtype == torch.float32 else 1
    return lib.akv_paged_attention_noalloc(
        c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), out.data_ptr(), c["table"].data_ptr(),
        c["cu"].data_ptr(), c["ctx"].data_ptr(), c["tile_seq"].data_ptr(), c["tile_q0"].data_ptr(),
        c["tile_nq"].data_ptr(), c["n"], c["n"], 1, splits, c["n"], c["table"].shape[1], c["nh"], c["nkv"], c["d"],
        c["page"], c["pool"], 0, c["d"] ** -0.5, code, None, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_entry_matches_the_ordinary_entry_point(dtype):
    lib, ops = _library()
    assert lib.akv_noalloc_scratch_bytes() == 16 * 1024 * 1024
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=1.6e-2, rtol=1.6e-2)
    # two calls in a row on different data: the second finds the first one's partials in the shared workspace
    for seed, splits in ((1, 5), (2, 3)):
        c = _case(dtype, seed)
        want = ops.paged_attention(c["q"], c["k"], c["v"], c["table"], c["cu"], c["ctx"], c["tile_seq"], c["tile_q0"],
                                   c["tile_nq"], num_tiles=c["n"], q_tile=1, num_splits=splits, num_heads=c["nh"],
                                   num_kv_heads=c["nkv"], window=0, scale=c["d"] ** -0.5, kernel="general")
        out = torch.full_like(c["q"], float("nan"))
        before = torch.cuda.memory_allocated()
        rc = _call(lib, c, out, splits, dtype)
        assert rc == 0, lib.akv_noalloc_last_error().decode()
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float().cpu(), want.float().cpu(), **tol)


def test_no_alloc_entry_refuses_what_does_not_fit():
    lib, _ = _library()
    c = _case(torch.float32, 3)
    out = torch.zeros_like(c["q"])
    big = dict(c, n=70000)            # 70,000 tokens x 8 heads x 4 splits x 66 floats is far beyond 16 MiB
    rc = _call(lib, big, out, 4, torch.float32)
    assert rc != 0
    message = lib.akv_noalloc_last_error().decode()
    assert "workspace" in message and "16777216" in message
    rc = lib.akv_paged_attention_noalloc(None, *([None] * 9), 1, 1, 1, 1, 1, 1, 8, 2, 64, 16, 4, 0, 1.0, 0, None, None)
    assert rc != 0 and "null" in lib.akv_noalloc_last_error().decode()
