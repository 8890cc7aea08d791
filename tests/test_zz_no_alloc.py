"""The entry point for callers that must not allocate device memory (csrc/noalloc_entry.h).

Some hosts of this library cannot call cudaMalloc: their device memory was handed out in full by a pool of their
own, or they sit in a real-time loop where the allocator is off limits, or they may only touch the buffers they
were given.  For them the library exports one C function that runs the split paged attention with its workspace
in a fixed 16 MiB array inside the library.  This test calls it the way such a host does, through the exported C
symbol with raw device pointers, several times in a row, and compares with the ordinary entry point (whose Python
wrapper allocates the workspace) and with the plain attention formula.

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
    """One decoded token per request over a shuffled pool whose unheld pages are NaN (a read outside the
    request's own pages would show), with the plain formula's answer beside it."""
    from paged_case import PagedCase
    case = PagedCase(dtype, nh, nkv, d, page, q_lens=[1] * len(ctxs), ctx_lens=list(ctxs), seed=seed)
    i32 = lambda v: torch.as_tensor(v, dtype=torch.int32).cuda()
    n = len(ctxs)
    q = torch.cat([x.reshape(x.shape[0], -1) for x in case.q_seq]).cuda()
    return dict(case=case, q=q, k=case.k_cache.cuda(), v=case.v_cache.cuda(), table=case.table.cuda(), cu=i32(case.cu),
                ctx=i32(list(ctxs)), tile_seq=i32(case.tiles[0]), tile_q0=i32(case.tiles[1]), tile_nq=i32(case.tiles[2]),
                nh=nh, nkv=nkv, d=d, page=page, pool=case.k_cache.shape[0], n=n)


def _call(lib, c, out, splits, dtype, window=0, status=None):
    code = 0 if dtype == torch.float32 else 1
    return lib.akv_paged_attention_noalloc(
        c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), out.data_ptr(), c["table"].data_ptr(),
        c["cu"].data_ptr(), c["ctx"].data_ptr(), c["tile_seq"].data_ptr(), c["tile_q0"].data_ptr(),
        c["tile_nq"].data_ptr(), c["n"], c["n"], 1, splits, c["n"], c["table"].shape[1], c["nh"], c["nkv"], c["d"],
        c["page"], c["pool"], window, c["d"] ** -0.5, code, None if status is None else status.data_ptr(),
        torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_entry_matches_the_ordinary_entry_point(dtype):
    lib, ops = _library()
    assert lib.akv_noalloc_scratch_bytes() == 16 * 1024 * 1024
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=1.6e-2, rtol=1.6e-2)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # calls in a row on different data: each finds the one before's partials in the shared workspace.  The last
    # needs no workspace at all (one split); the third looks back over a window only.
    for seed, splits, window in ((1, 5, 0), (2, 3, 0), (3, 4, 40), (4, 1, 0)):
        c = _case(dtype, seed)
        want = ops.paged_attention(c["q"], c["k"], c["v"], c["table"], c["cu"], c["ctx"], c["tile_seq"], c["tile_q0"],
                                   c["tile_nq"], num_tiles=c["n"], q_tile=1, num_splits=splits, num_heads=c["nh"],
                                   num_kv_heads=c["nkv"], window=window, scale=c["d"] ** -0.5, kernel="general")
        out = torch.full_like(c["q"], float("nan"))
        rc = _call(lib, c, out, splits, dtype, window, status)
        assert rc == 0, lib.akv_noalloc_last_error().decode()
        torch.cuda.synchronize()
        assert int(status.item()) == 0          # no block-table entry or slot was out of range
        torch.testing.assert_close(out.float().cpu(), want.float().cpu(), **tol)
        # and both against the attention formula itself, not only against each other
        torch.testing.assert_close(out.float().cpu(), c["case"].reference(window), **tol)


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
