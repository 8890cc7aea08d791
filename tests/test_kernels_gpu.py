"""Each kernel alone against a plain float32 reference of the same operation, at sizes other than the
tiny models' (head sizes 48/80/128/256, group sizes 1/2/3/8, widths and vocabularies that are no power
of two), in float32 and bfloat16."""


import pytest
import torch

from paged_case import PagedCase, dev, status_word
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=1.6e-2, rtol=1.6e-2)


@pytest.fixture(scope="module")
def ops():
    from ampere_kv_engine_b200.kernels import ops as module
    module.ext()
    return module


def test_smoke_add(ops):
    a, b = torch.randn(1000), torch.randn(1000)
    torch.testing.assert_close(ops.smoke_add(dev(a), dev(b)).cpu(), a + b, atol=0, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(ops, dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(777, 200, generator=g).to(dtype)
    ids = torch.randint(0, 777, (53,), generator=g, dtype=torch.int32)
    status = status_word()
    out = ops.embedding(dev(ids), dev(table), status=status)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), table.float()[ids.long()], atol=0, rtol=0)
    assert int(status.item()) == 0


def test_embedding_reports_a_bad_token_without_faulting(ops):
    table = torch.randn(10, 32)
    ids = torch.tensor([1, 10, 3], dtype=torch.int32)     # 10 is outside the vocabulary
    status = status_word()
    out = ops.embedding(dev(ids), dev(table), status=status)
    assert int(status.item()) == 3
    torch.testing.assert_close(out.cpu()[[0, 2]], table[[1, 3]], atol=0, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [72, 200, 4096, 5120])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rmsnorm(ops, dtype, hidden, with_delta):
    g = torch.Generator().manual_seed(hidden)
    h = torch.randn(19, hidden, generator=g)
    delta = torch.randn(19, hidden, generator=g).to(dtype) if with_delta else None
    w = 1 + 0.1 * torch.randn(hidden, generator=g)
    eps = 1e-5
    h_dev = dev(h.clone())
    out = ops.add_rmsnorm(h_dev, dev(delta) if with_delta else None, dev(w), eps, dtype)
    summed = h + (delta.float() if with_delta else 0)
    torch.testing.assert_close(h_dev.cpu(), summed, atol=0, rtol=0)       # the residual sum is exact float32
    want = plain.rms_norm(summed, w, eps)
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))
    # gathered form: chosen rows only, the stream is left alone
    rows = torch.tensor([18, 0, 7], dtype=torch.int32)
    h_dev = dev(h.clone())
    out = ops.add_rmsnorm(h_dev, dev(delta) if with_delta else None, dev(w), eps, dtype, rows=dev(rows))
    torch.testing.assert_close(h_dev.cpu(), h, atol=0, rtol=0)
    torch.testing.assert_close(out.float().cpu(), want[rows.long()], **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(ops, dtype):
    g = torch.Generator().manual_seed(1)
    gu = (3 * torch.randn(37, 2 * 300, generator=g)).to(dtype)
    out = ops.silu_mul(dev(gu))
    want = torch.nn.functional.silu(gu.float()[:, :300]) * gu.float()[:, 300:]
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter,block", [(320, 64), (300, 4), (96, 32), (66, 3)])
def test_silu_mul_with_alternating_runs(ops, dtype, inter, block):
    """Gate and up columns in alternating runs (the layout of the fused decode GEMM), vector and scalar paths."""
    g = torch.Generator().manual_seed(inter)
    gate, up = (3 * torch.randn(2, 23, inter, generator=g)).to(dtype)
    mixed = torch.stack((gate.view(23, inter // block, block), up.view(23, inter // block, block)), dim=2)
    out = ops.silu_mul(dev(mixed.reshape(23, 2 * inter).contiguous()), block=block)
    want = torch.nn.functional.silu(gate.float()) * up.float()
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))
    with pytest.raises(RuntimeError, match="run length"):
        ops.silu_mul(dev(mixed.reshape(23, 2 * inter).contiguous()), block=7)


@pytest.mark.parametrize("tokens,inter,k", [(1, 64, 64), (8, 192, 320), (17, 640, 1024), (32, 128, 4096), (5, 12288, 512)])
def test_gated_gemm_applies_the_activation(ops, tokens, inter, k):
    """The decode GEMM with the gated epilogue equals product, rounding, then the activation kernel."""
    g = torch.Generator().manual_seed(tokens + inter)
    gate = (torch.randn(inter, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    up = (torch.randn(inter, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    x = (2 * torch.randn(tokens, k, generator=g)).to(torch.bfloat16)
    w = ops.interleave_gate_up(gate, up, ops.GATE_UP_RUN).contiguous()
    status = status_word()
    out = ops.gated_linear(dev(x), dev(w), ops.GATE_UP_RUN, status=status)
    assert int(status.item()) == 0 and out.shape == (tokens, inter) and out.dtype == torch.bfloat16
    gf = (x.float() @ gate.float().t()).to(torch.bfloat16).float()
    uf = (x.float() @ up.float().t()).to(torch.bfloat16).float()
    want = torch.nn.functional.silu(gf) * uf
    torch.testing.assert_close(out.float().cpu(), want, atol=3e-2, rtol=3e-2)
    # every split count gives the same kind of answer, and the unfused pair agrees
    for splits in (1, 2, 4, 8):
        if splits <= (k + 63) // 64:
            got = ops.small_m_gemm(dev(x), dev(w), splits=splits, gated=True)
            torch.testing.assert_close(got.float().cpu(), want, atol=3e-2, rtol=3e-2)
    unfused = ops.silu_mul(torch.nn.functional.linear(dev(x), dev(w)), block=ops.GATE_UP_RUN)
    torch.testing.assert_close(out.float().cpu(), unfused.float().cpu(), atol=3e-2, rtol=3e-2)
    # all gate rows first: the product and the activation kernel
    halves = ops.gated_linear(dev(x), dev(torch.cat((gate, up))), 0)
    torch.testing.assert_close(halves.float().cpu(), want, atol=3e-2, rtol=3e-2)


def _qkv_reference(qkv, positions, q_w, k_w, nh, nkv, d, eps, theta):
    n = qkv.shape[0]
    x = qkv.float().view(n, nh + 2 * nkv, d)
    q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]
    q, k = plain.rms_norm(q, q_w, eps), plain.rms_norm(k, k_w, eps)
    inv = plain.rope_inverse_frequencies(d, theta)
    return plain.apply_rope(q, positions, inv), plain.apply_rope(k, positions, inv), v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,page", [(6, 3, 48, 8), (8, 1, 128, 16), (4, 4, 80, 32), (2, 1, 256, 16), (5, 5, 64, 8),
                                           (7, 1, 128, 32)])
def test_qk_norm_rope_write(ops, dtype, nh, nkv, d, page):
    g = torch.Generator().manual_seed(d)
    n, pages, eps, theta = 29, 12, 1e-5, 50000.0
    qkv = torch.randn(n, (nh + 2 * nkv) * d, generator=g).to(dtype)
    positions = torch.randint(0, 3000, (n,), generator=g, dtype=torch.int32)
    q_w = 1 + 0.1 * torch.randn(d, generator=g)
    k_w = 1 + 0.1 * torch.randn(d, generator=g)
    slots = torch.randperm(pages * page, generator=g)[:n].to(torch.int32)
    slots[5] = -1                                            # a token whose K/V must not be written
    k_cache = torch.full((pages, nkv, page, d), float("nan")).to(dtype)
    v_cache = k_cache.clone()
    k_dev, v_dev = dev(k_cache), dev(v_cache)
    inv_freq = plain.rope_inverse_frequencies(d, theta)
    status = status_word()
    q, k_dense, v_dense = ops.qk_norm_rope_write(
        dev(qkv), dev(positions), dev(slots), dev(q_w), dev(k_w), dev(inv_freq), k_dev, v_dev, num_heads=nh,
        num_kv_heads=nkv, head_dim=d, rotary_dim=d, eps=eps, want_kv=True, status=status)
    assert int(status.item()) == 0
    q_ref, k_ref, v_ref = _qkv_reference(qkv, positions, q_w, k_w, nh, nkv, d, eps, theta)
    torch.testing.assert_close(q.float().cpu().view(n, nh, d), q_ref, **tol(dtype))
    torch.testing.assert_close(k_dense.float().cpu().view(n, nkv, d), k_ref, **tol(dtype))
    torch.testing.assert_close(v_dense.float().cpu().view(n, nkv, d), v_ref, atol=0, rtol=0)
    k_host, v_host = k_dev.cpu(), v_dev.cpu()
    written = torch.zeros(pages, page, dtype=torch.bool)
    for t in range(n):
        s = int(slots[t])
        if s < 0:
            continue
        written[s // page, s % page] = True
        # the pages hold exactly what the dense outputs hold: post-rotation K, un-rotated V
        torch.testing.assert_close(k_host[s // page, :, s % page], k_dense.cpu().view(n, nkv, d)[t], atol=0, rtol=0)
        torch.testing.assert_close(v_host[s // page, :, s % page], v_dense.cpu().view(n, nkv, d)[t], atol=0, rtol=0)
    untouched = ~written[:, None, :, None].expand_as(k_host)
    assert bool(torch.isnan(k_host.float()[untouched]).all()), "a slot that no token owns was written"
    assert bool(torch.isnan(v_host.float()[untouched]).all())


@pytest.mark.parametrize("tokens,nh,nkv,k,page", [(1, 2, 1, 64, 16), (8, 4, 2, 320, 8), (19, 3, 3, 1024, 32), (32, 8, 2, 2048, 16)])
def test_project_qkv_on_the_gemm_tile(ops, tokens, nh, nkv, k, page):
    """Few tokens with heads of 128 dims: the projection kernel norms, rotates and writes the cache on its output
    tile.  It must equal the product followed by qk_norm_rope_write, and the plain reference."""
    d, eps, theta, pages = 128, 1e-5, 50000.0, 9
    g = torch.Generator().manual_seed(tokens + k)
    w = (torch.randn((nh + 2 * nkv) * d, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    x = (2 * torch.randn(tokens, k, generator=g)).to(torch.bfloat16)
    positions = torch.randint(0, 9000, (tokens,), generator=g, dtype=torch.int32)
    q_w = 1 + 0.1 * torch.randn(d, generator=g)
    k_w = 1 + 0.1 * torch.randn(d, generator=g)
    slots = torch.randperm(pages * page, generator=g)[:tokens].to(torch.int32)
    if tokens > 5:
        slots[5] = -1
    inv_freq = plain.rope_inverse_frequencies(d, theta)
    results = []
    for fused in (True, False):
        ops.use_small_m_gemm = fused
        try:
            k_dev = dev(torch.full((pages, nkv, page, d), float("nan")).to(torch.bfloat16))
            v_dev = k_dev.clone()
            status = status_word()
            before = ops.launch_count
            q = ops.project_qkv(dev(x), dev(w), None, dev(positions), dev(slots), dev(q_w), dev(k_w), dev(inv_freq),
                                k_dev, v_dev, num_heads=nh, num_kv_heads=nkv, head_dim=d, rotary_dim=d, eps=eps,
                                status=status)
            assert ops.launch_count - before == 1      # one kernel of this package either way (the other
        finally:                                       # route's product is the library's)
            ops.use_small_m_gemm = True
        assert int(status.item()) == 0
        results.append((q.float().cpu(), k_dev.float().cpu(), v_dev.float().cpu()))
    qkv = (x.float() @ w.float().t()).to(torch.bfloat16)
    q_ref, k_ref, v_ref = _qkv_reference(qkv, positions, q_w, k_w, nh, nkv, d, eps, theta)
    for q, k_host, v_host in results:
        torch.testing.assert_close(q.view(tokens, nh, d), q_ref, atol=3e-2, rtol=3e-2)
        written = torch.zeros(pages, page, dtype=torch.bool)
        for t in range(tokens):
            s_ = int(slots[t])
            if s_ < 0:
                continue
            written[s_ // page, s_ % page] = True
            torch.testing.assert_close(k_host[s_ // page, :, s_ % page], k_ref[t], atol=3e-2, rtol=3e-2)
            torch.testing.assert_close(v_host[s_ // page, :, s_ % page], v_ref[t], atol=3e-2, rtol=3e-2)
        untouched = ~written[:, None, :, None].expand_as(k_host)
        assert bool(torch.isnan(k_host[untouched]).all()) and bool(torch.isnan(v_host[untouched]).all())
    # the two routes differ only by the order in which each adds up K
    torch.testing.assert_close(results[0][0], results[1][0], atol=3e-2, rtol=3e-2)
    # no norm weights, no rotation, no cache: q is the plain product
    q = ops.project_qkv(dev(x), dev(w), None, dev(positions), None, None, None, None, None, None, num_heads=nh,
                        num_kv_heads=nkv, head_dim=d, rotary_dim=0, eps=eps)
    torch.testing.assert_close(q.float().cpu(), qkv[:, :nh * d].float(), atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("tokens,hidden_size,k", [(1, 64, 64), (8, 96, 160), (19, 4096, 512), (32, 1000, 1024)])
def test_product_adds_to_the_residual_and_the_next_applies_the_norm(ops, monkeypatch, tokens, hidden_size, k):
    """A decode branch ends in a product that adds to the float32 residual stream itself and leaves per-tile sums
    of squares; the next product makes its token operand from them (the RMS norm inside the kernel).  Both must
    equal the unfused kernels: product, add + norm, product."""
    monkeypatch.setattr(ops, "LAZY_NORM_LIMIT", ops.SMALL_M_LIMIT)     # the engine stops at fewer tokens; the kernels do not
    g = torch.Generator().manual_seed(tokens + hidden_size)
    eps = 1e-5
    x = torch.randn(tokens, k, generator=g).to(torch.bfloat16)
    w_out = (torch.randn(hidden_size, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    hidden = 3 * torch.randn(tokens, hidden_size, generator=g)
    norm_w = 1 + 0.1 * torch.randn(hidden_size, generator=g)
    h_dev = dev(hidden.clone())
    status = status_word()
    summed = ops.linear_into_residual(dev(x), dev(w_out), h_dev, status=status)
    assert summed is not None and summed.hidden is h_dev and int(status.item()) == 0
    delta = (x.float() @ w_out.float().t()).to(torch.bfloat16).float()
    want_hidden = hidden + delta
    # the product's float32 sums differ from the host's in their last bits, and a bfloat16 rounding may flip
    torch.testing.assert_close(h_dev.cpu(), want_hidden, atol=2e-2, rtol=2e-2)
    got_hidden = h_dev.cpu()
    assert summed.ssq.shape == ((hidden_size + 127) // 128, tokens)
    torch.testing.assert_close(summed.ssq.sum(0).cpu(), got_hidden.square().sum(-1), atol=1e-3, rtol=1e-5)
    for tile in range(summed.ssq.shape[0]):
        torch.testing.assert_close(summed.ssq[tile].cpu(), got_hidden[:, tile * 128:(tile + 1) * 128].square().sum(-1),
                                   atol=1e-3, rtol=1e-5)

    lazy = ops.LazyNorm(summed, dev(norm_w), eps, torch.bfloat16, status)
    normed = plain.rms_norm(got_hidden, norm_w, eps).to(torch.bfloat16)
    torch.testing.assert_close(lazy.materialize().float().cpu(), normed.float(), **tol(torch.bfloat16))
    if hidden_size % 8:
        return
    # plain product of the lazy norm, in both output types
    w_next = (torch.randn(200, hidden_size, generator=g) * hidden_size ** -0.5).to(torch.bfloat16)
    want = normed.float() @ w_next.float().t()
    torch.testing.assert_close(ops.linear(lazy, dev(w_next), out_dtype=torch.float32, status=status).cpu(), want,
                               atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(ops.linear(lazy, dev(w_next), status=status).float().cpu(), want, atol=4e-2, rtol=4e-2)
    # gated product
    gate = (torch.randn(128, hidden_size, generator=g) * hidden_size ** -0.5).to(torch.bfloat16)
    up = (torch.randn(128, hidden_size, generator=g) * hidden_size ** -0.5).to(torch.bfloat16)
    gu = ops.interleave_gate_up(gate, up, ops.GATE_UP_RUN).contiguous()
    gf = (normed.float() @ gate.float().t()).to(torch.bfloat16).float()
    uf = (normed.float() @ up.float().t()).to(torch.bfloat16).float()
    torch.testing.assert_close(ops.gated_linear(lazy, dev(gu), ops.GATE_UP_RUN, status=status).float().cpu(),
                               torch.nn.functional.silu(gf) * uf, atol=4e-2, rtol=4e-2)
    torch.testing.assert_close(ops.gated_linear(lazy, dev(torch.cat((gate, up))), 0, status=status).float().cpu(),
                               torch.nn.functional.silu(gf) * uf, atol=4e-2, rtol=4e-2)
    # q/k/v projection with norm, rotation and cache write on the tile
    nh, nkv, d, page, pages = 2, 1, 128, 16, 6
    w_qkv = (torch.randn((nh + 2 * nkv) * d, hidden_size, generator=g) * hidden_size ** -0.5).to(torch.bfloat16)
    positions = torch.randint(0, 5000, (tokens,), generator=g, dtype=torch.int32)
    slots = torch.randperm(pages * page, generator=g)[:tokens].to(torch.int32)
    q_w, k_w = 1 + 0.1 * torch.randn(d, generator=g), 1 + 0.1 * torch.randn(d, generator=g)
    inv_freq = plain.rope_inverse_frequencies(d, 10000.0)
    k_dev = dev(torch.full((pages, nkv, page, d), float("nan")).to(torch.bfloat16))
    v_dev = k_dev.clone()
    q = ops.project_qkv(lazy, dev(w_qkv), None, dev(positions), dev(slots), dev(q_w), dev(k_w), dev(inv_freq), k_dev,
                        v_dev, num_heads=nh, num_kv_heads=nkv, head_dim=d, rotary_dim=d, eps=eps, status=status)
    qkv = (normed.float() @ w_qkv.float().t()).to(torch.bfloat16)
    q_ref, k_ref, v_ref = _qkv_reference(qkv, positions, q_w, k_w, nh, nkv, d, eps, 10000.0)
    torch.testing.assert_close(q.float().cpu().view(tokens, nh, d), q_ref, atol=4e-2, rtol=4e-2)
    for t_ in range(tokens):
        s_ = int(slots[t_])
        torch.testing.assert_close(k_dev.float().cpu()[s_ // page, :, s_ % page], k_ref[t_], atol=4e-2, rtol=4e-2)
        torch.testing.assert_close(v_dev.float().cpu()[s_ // page, :, s_ % page], v_ref[t_], atol=4e-2, rtol=4e-2)
    assert int(status.item()) == 0
    # more tokens than the small-batch kernel takes, or float32: the caller keeps the unfused route
    big = dev(torch.zeros(ops.SMALL_M_LIMIT + 1, k, dtype=torch.bfloat16))
    assert ops.linear_into_residual(big, dev(w_out), dev(torch.zeros(ops.SMALL_M_LIMIT + 1, hidden_size))) is None


def test_qk_partial_rotation_and_no_rotation(ops):
    """rotary_dim < head_dim rotates pairs (j, j + rotary_dim/2) of the first rotary_dim dims only; no table = no rotation."""
    g = torch.Generator().manual_seed(4)
    n, nh, nkv, d, rd = 7, 3, 1, 64, 32
    qkv = torch.randn(n, (nh + 2 * nkv) * d, generator=g)
    positions = torch.arange(100, 100 + n, dtype=torch.int32)
    inv = plain.rope_inverse_frequencies(rd, 10000.0)
    q = ops.qk_norm_rope_write(dev(qkv), dev(positions), None, None, None, dev(inv), None, None, num_heads=nh,
                               num_kv_heads=nkv, head_dim=d, rotary_dim=rd, eps=1e-6).cpu().view(n, nh, d)
    x = qkv.view(n, nh + 2 * nkv, d)[:, :nh]
    want = torch.cat((plain.apply_rope(x[..., :rd], positions, inv), x[..., rd:]), dim=-1)
    torch.testing.assert_close(q, want, atol=2e-5, rtol=1e-4)
    q = ops.qk_norm_rope_write(dev(qkv), dev(positions), None, None, None, None, None, None, num_heads=nh,
                               num_kv_heads=nkv, head_dim=d, rotary_dim=0, eps=1e-6).cpu().view(n, nh, d)
    torch.testing.assert_close(q, x, atol=0, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_kv_write(ops, dtype):
    g = torch.Generator().manual_seed(2)
    n, nkv, d, page, pages = 11, 3, 48, 8, 5
    k = torch.randn(n, nkv * d, generator=g).to(dtype)
    v = torch.randn(n, nkv * d, generator=g).to(dtype)
    slots = torch.randperm(pages * page, generator=g)[:n].to(torch.int32)
    k_cache = dev(torch.full((pages, nkv, page, d), float("nan")).to(dtype))
    v_cache = k_cache.clone()
    ops.kv_write(dev(k), dev(v), dev(slots), k_cache, v_cache)
    for t in range(n):
        s = int(slots[t])
        torch.testing.assert_close(k_cache.cpu()[s // page, :, s % page].reshape(-1), k[t], atol=0, rtol=0)
        torch.testing.assert_close(v_cache.cpu()[s // page, :, s % page].reshape(-1), v[t], atol=0, rtol=0)
    assert int(torch.isnan(k_cache.float()).sum()) == (pages * page - n) * nkv * d


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,page", [(6, 3, 48, 8), (8, 1, 128, 16), (4, 4, 80, 32), (4, 2, 256, 16), (9, 3, 16, 64)])
@pytest.mark.parametrize("window", [0, 17])
def test_paged_attention_mixed_batch(ops, dtype, nh, nkv, d, page, window):
    case = PagedCase(dtype, nh, nkv, d, page, q_lens=[1, 37, 5, 1, 2], ctx_lens=[200, 37, 150, 1, 66], seed=d + page)
    want = case.reference(window)
    for splits in (1, 3):
        torch.testing.assert_close(case.run(ops, window, splits), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kernel", ["auto", "general"])
def test_a_batch_covered_by_two_calls_with_different_splits(ops, dtype, kernel):
    """A step that holds decoded tokens beside prompt portions runs attention twice, over different tiles and with
    different numbers of key splits, into one output.  A call writes the rows of its own tiles only: the other
    call's rows have no partial sums in its workspace (here the workspaces are filled with NaN beforehand)."""
    case = PagedCase(dtype, 8, 2, 64, 16, q_lens=[1, 40, 1, 23, 1], ctx_lens=[300, 90, 77, 400, 1], seed=5)
    want = case.reference(0)
    q = dev(torch.cat([x.reshape(x.shape[0], -1) for x in case.q_seq]))
    ctx_lens = dev(torch.tensor(case.ctx_lens, dtype=torch.int32))
    cu = case.cu.tolist()
    single = [(s, cu[s], 1) for s, n in enumerate(case.q_lens) if n == 1]
    portions = [(s, cu[s] + q0, min(16, n - q0)) for s, n in enumerate(case.q_lens) if n > 1 for q0 in range(0, n, 16)]
    for first_splits, second_splits in ((3, 2), (2, 5), (1, 4), (4, 1)):
        out = torch.full_like(q, float("nan"))
        status = status_word()
        for tiles, q_tile, splits in ((single, 1, first_splits), (portions, 16, second_splits)):
            cols = [dev(torch.tensor([t[i] for t in tiles], dtype=torch.int32)) for i in range(3)]
            partials = torch.full((q.shape[0] * 8 * splits * (64 + 2),), float("nan"), device=q.device)
            ops.paged_attention(q, dev(case.k_cache), dev(case.v_cache), dev(case.table), dev(case.cu), ctx_lens,
                                cols[0], cols[1], cols[2], num_tiles=len(tiles), q_tile=q_tile, num_splits=splits,
                                num_heads=8, num_kv_heads=2, window=0, scale=64 ** -0.5, partials=partials,
                                status=status, kernel=kernel, out=out)
        assert int(status.item()) == 0
        torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("nh,nkv,d,page", [(32, 8, 128, 16), (8, 8, 64, 32), (16, 1, 128, 64), (6, 2, 128, 8)])
@pytest.mark.parametrize("window", [0, 50])
def test_tensor_core_and_general_kernels_agree(ops, nh, nkv, d, page, window):
    """bfloat16 at head sizes 64 and 128 takes the TMA + tensor-core kernels; forcing the general kernel on the
    same problem must give the same answer (both are also held against the plain reference)."""
    dtype = torch.bfloat16
    mixed = PagedCase(dtype, nh, nkv, d, page, q_lens=[1, 37, 5, 1, 16, 70], ctx_lens=[200, 37, 150, 1, 16, 333],
                      seed=nh + page)
    want = mixed.reference(window)
    torch.testing.assert_close(mixed.run(ops, window, 1, kernel="auto"), want, **tol(dtype))
    torch.testing.assert_close(mixed.run(ops, window, 1, kernel="mma"), want, **tol(dtype))
    torch.testing.assert_close(mixed.run(ops, window, 1, kernel="general"), want, **tol(dtype))
    decode = PagedCase(dtype, nh, nkv, d, page, q_lens=[1] * 6, ctx_lens=[1, 31, 32, 33, 700, 129], seed=nh)
    want = decode.reference(window)
    for splits in (1, 2, 7):
        torch.testing.assert_close(decode.run(ops, window, splits, kernel="auto"), want, **tol(dtype))
    torch.testing.assert_close(decode.run(ops, window, 3, kernel="general"), want, **tol(dtype))


@pytest.mark.parametrize("nh,nkv,page,q_tile", [(32, 8, 16, 32), (16, 8, 32, 64), (8, 1, 64, 16), (32, 8, 16, 16),
                                                 (32, 8, 16, 64), (8, 2, 16, 96), (16, 2, 32, 64), (8, 4, 64, 128),
                                                 # groups that do not divide 128 (dead rows at a tile's end), one
                                                 # q-head per kv head, sixteen
                                                 (40, 8, 16, 25), (40, 8, 16, 32), (6, 2, 16, 42), (4, 4, 16, 32),
                                                 (16, 1, 16, 32), (12, 2, 32, 21), (14, 2, 16, 64), (8, 2, 64, 32),
                                                 (8, 2, 128, 32)])
@pytest.mark.parametrize("window", [0, 100, 37])
def test_tcgen05_prompt_attention(ops, nh, nkv, page, q_tile, window):
    """Prompt portions at head size 128 with groups of 1 to 16 q-heads run on the tcgen05 kernel: whole
    prompts, portions after a long history, tiles that end mid-way, a portion of one token beside them.  Batch
    tiles of one, two, three or four of the kernel's 128-row query tiles (the last one whole, partial or empty),
    windows longer and shorter than a tile's span."""
    dtype = torch.bfloat16
    case = PagedCase(dtype, nh, nkv, 128, page, q_lens=[300, 77, 33, 1, 128], ctx_lens=[300, 500, 33, 40, 128],
                     seed=page + nh, q_tile=q_tile)
    want = case.reference(window)
    # both forms of the kernel (the grid's size picks one otherwise), and the mma.sync kernel
    for kernel in ("tcgen05-narrow", "tcgen05-wide", "auto", "mma"):
        torch.testing.assert_close(case.run(ops, window, 1, kernel=kernel), want, **tol(dtype))


@pytest.mark.parametrize("q_tile", [32, 64])
def test_tcgen05_prompt_attention_repeats_and_rescales(ops, q_tile):
    """The tcgen05 kernel keeps a stale running maximum and rescales its accumulator only when a score exceeds it
    by 2^8: keys of growing norm force that path in every block, a dominant key early and late in a long history
    tests both sides of it, and repeated launches must agree bit for bit (its warps run at different speeds)."""
    dtype = torch.bfloat16
    case = PagedCase(dtype, 8, 2, 128, 16, q_lens=[96, 200, 40], ctx_lens=[900, 200, 1500], seed=77, q_tile=q_tile)
    # sequence 0: key norms grow along the sequence, so that later blocks keep raising the maximum
    ramp = torch.linspace(0.2, 6.0, 900).view(900, 1, 1)
    case.k_seq[0] = (case.k_seq[0].float() * ramp).to(dtype)
    # sequence 2: one dominant key near the start and one near the end, seen by every query of the portion
    for far, gain in ((5, 6.0), (1490, 9.0)):
        for kv in range(2):
            direction = torch.nn.functional.normalize(case.k_seq[2][far, kv].float(), dim=0)
            case.k_seq[2][far, kv] = (gain * direction).to(dtype)
            for h in range(4 * kv, 4 * kv + 4):
                case.q_seq[2][:, h] = (case.q_seq[2][:, h].float() + 25.0 * direction).to(dtype)
    case.rewrite_cache()
    want = case.reference(0)
    for form in ("tcgen05-narrow", "tcgen05-wide"):
        first = case.run(ops, 0, 1, kernel=form)
        torch.testing.assert_close(first, want, **tol(dtype))
        for _ in range(8):
            assert torch.equal(case.run(ops, 0, 1, kernel=form), first)
    torch.testing.assert_close(case.run(ops, 0, 1, kernel="mma"), want, **tol(dtype))


def _last_rows_reference(case, window=0):
    """The plain attention formula for the last q_len positions of each sequence only (float64), for contexts too
    long for the whole-sequence form: query i sees key j iff j <= i (and j > i - window)."""
    outs = []
    group = case.nh // case.nkv
    for s, (n, c) in enumerate(zip(case.q_lens, case.ctx_lens)):
        q = case.q_seq[s].double()                                            # [n, NH, D]
        k = case.k_seq[s].double().repeat_interleave(group, dim=1)            # [c, NH, D]
        v = case.v_seq[s].double().repeat_interleave(group, dim=1)
        scores = torch.einsum("thd,shd->hts", q, k) * case.d ** -0.5
        i = torch.arange(c - n, c)[:, None]
        j = torch.arange(c)[None, :]
        visible = j <= i
        if window:
            visible &= j > i - window
        probs = torch.softmax(scores.masked_fill(~visible[None], -torch.inf), dim=-1)
        outs.append(torch.einsum("hts,shd->thd", probs, v).reshape(n, -1).float())
    return torch.cat(outs)


@pytest.mark.parametrize("q_tile", [32, 64])
@pytest.mark.parametrize("window", [0, 3000])
def test_attention_over_thousands_of_keys(ops, window, q_tile):
    """Contexts of several thousand keys, where the K/V rings of the tensor-core kernels wrap hundreds of times:
    prompt portions after a long history (tcgen05 and mma.sync kernels), and decoded tokens with every way of
    splitting the keys.  One far key is made to matter in the longest sequence."""
    dtype = torch.bfloat16
    case = PagedCase(dtype, 8, 2, 128, 16, q_lens=[200, 37, 64], ctx_lens=[6000, 4100, 2500], seed=41, q_tile=q_tile)
    far = 77
    for kv in range(2):
        direction = torch.nn.functional.normalize(case.k_seq[0][far, kv].float(), dim=0)
        case.k_seq[0][far, kv] = (7.0 * direction).to(dtype)
        for h in range(4 * kv, 4 * kv + 4):
            case.q_seq[0][:, h] = (case.q_seq[0][:, h].float() + 20.0 * direction).to(dtype)
    case.rewrite_cache()
    want = _last_rows_reference(case, window)
    for kernel in ("tcgen05-narrow", "tcgen05-wide", "auto", "mma"):
        torch.testing.assert_close(case.run(ops, window, 1, kernel=kernel), want, **tol(dtype))
    decode = PagedCase(dtype, 8, 2, 128, 16, q_lens=[1, 1, 1, 1], ctx_lens=[6000, 4100, 1, 2500], seed=42)
    want = _last_rows_reference(decode, window)
    for splits in (1, 2, 4, 8):
        torch.testing.assert_close(decode.run(ops, window, splits), want, **tol(dtype))
    torch.testing.assert_close(decode.run(ops, window, 5, kernel="general"), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_decode_batch_and_scale(ops, dtype):
    case = PagedCase(dtype, 8, 2, 64, 16, q_lens=[1] * 7, ctx_lens=[1, 15, 16, 17, 300, 64, 65], seed=9)
    for splits in (1, 4):
        torch.testing.assert_close(case.run(ops, 0, splits, scale=0.2), case.reference(0, scale=0.2), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [1, 5])
def test_paged_attention_finds_a_far_key(ops, dtype, splits):
    """One key among 700 is made to dominate: the output must be (almost) that key's value row.  A kernel that
    dropped, duplicated or misplaced a page would miss it."""
    case = PagedCase(dtype, 4, 2, 64, 16, q_lens=[1, 3], ctx_lens=[700, 300], seed=3)
    far = 37
    for s in range(2):
        for kv in range(2):
            direction = torch.nn.functional.normalize(case.k_seq[s][far, kv].float(), dim=0)
            for h in (2 * kv, 2 * kv + 1):
                case.q_seq[s][:, h] = (60.0 * direction).to(dtype)
            case.k_seq[s][far, kv] = (8.0 * direction).to(dtype)
            pp = int(case.table[s, far // 16])
            case.k_cache[pp, kv, far % 16] = case.k_seq[s][far, kv]
    out = case.run(ops, 0, splits)
    want = case.reference(0)
    torch.testing.assert_close(out, want, **tol(dtype))
    row = out[0].view(4, 64)
    for h in range(4):
        torch.testing.assert_close(row[h], case.v_seq[0][far, h // 2].float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_window_edge(ops, dtype):
    """The key just inside the window dominates one query, the key just outside would dominate if it were seen."""
    window = 24
    case = PagedCase(dtype, 2, 1, 32, 8, q_lens=[4], ctx_lens=[100], seed=5)
    pos = 99                                   # last query; sees keys 76..99
    inside, outside = pos - window + 1, pos - window
    direction = torch.nn.functional.normalize(torch.randn(32, generator=torch.Generator().manual_seed(1)), dim=0)
    for key, gain in ((inside, 6.0), (outside, 12.0)):
        case.k_seq[0][key, 0] = (gain * direction).to(dtype)
        case.k_cache[int(case.table[0, key // 8]), 0, key % 8] = case.k_seq[0][key, 0]
    case.q_seq[0][:, :] = (40.0 * direction).to(dtype)
    out = case.run(ops, window)
    torch.testing.assert_close(out, case.reference(window), **tol(dtype))
    torch.testing.assert_close(out[3].view(2, 32)[0], case.v_seq[0][inside, 0].float(), atol=2e-2, rtol=2e-2)


def test_paged_attention_reports_a_bad_page_without_faulting(ops):
    case = PagedCase(torch.float32, 2, 1, 32, 8, q_lens=[1], ctx_lens=[20], seed=6)
    case.table[0, 1] = 10 ** 6                   # far outside the pool
    q = case.q_seq[0].reshape(1, -1)
    status = status_word()
    ops.paged_attention(dev(q), dev(case.k_cache), dev(case.v_cache), dev(case.table), dev(case.cu),
                        dev(torch.tensor([20], dtype=torch.int32)), dev(case.tiles[0]), dev(case.tiles[1]),
                        dev(case.tiles[2]), num_tiles=1, q_tile=1, num_splits=1, num_heads=2, num_kv_heads=1,
                        window=0, scale=1.0, status=status)
    assert int(status.item()) == 1


def test_kernels_refuse_sizes_they_do_not_take(ops):
    q = torch.zeros(1, 2 * 24, device="cuda")
    cache = torch.zeros(2, 1, 8, 24, device="cuda")
    i32 = lambda *v: torch.tensor(v, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="multiple of 16"):
        ops.paged_attention(q, cache, cache, i32(0).view(1, 1), i32(0, 1), i32(1), i32(0), i32(0), i32(1),
                            num_tiles=1, q_tile=1, num_splits=1, num_heads=2, num_kv_heads=1, window=0, scale=1.0)
    with pytest.raises(RuntimeError, match="exceeds"):
        h = torch.zeros(1, 60000, device="cuda")
        ops.add_rmsnorm(h, None, torch.ones(60000, device="cuda"), 1e-6, torch.float32)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.silu_mul(torch.zeros(2, 8))


def _cdf_interval_ok(logits, temperature, u, token):
    cdf = plain.temperature_cdf(logits, temperature)
    lo = float(cdf[token - 1]) if token > 0 else 0.0
    hi = float(cdf[token])
    slack = 1e-5
    return lo - slack <= u * float(cdf[-1]) <= hi + slack


@pytest.mark.parametrize("vocab", [13, 1000, 1001, 151936])
def test_sample_greedy_and_temperature(ops, vocab):
    """A row is cut into slices, a block each: vocabularies smaller than the slices' granularity (empty slices), no
    multiple of four (scalar reads) and the benchmark model's; a tie between the first and the last slice."""
    g = torch.Generator().manual_seed(vocab)
    rows = 9
    logits = 3 * torch.randn(rows, vocab, generator=g)
    logits[0, min(17, vocab // 3)] = logits[0, vocab - 2] = 50.0     # a tie across slices: the lowest index wins
    logits[1, vocab - 1] = 60.0                                      # the maximum in the last slice
    temps = torch.tensor([0.0, 0.0, 0.8, 0.8, 1.5, 0.1, 1.0, 0.8, 0.8])
    us = torch.tensor([0.0, 0.0, 0.0, 0.999999, 0.5, 0.3, 0.77, 0.123, 0.5])
    tokens = ops.sample(dev(logits), dev(temps), dev(us)).cpu().tolist()
    assert tokens[0] == min(17, vocab // 3)
    assert tokens[1] == vocab - 1 == int(logits[1].argmax())
    for r in range(2, rows):
        assert _cdf_interval_ok(logits[r], float(temps[r]), float(us[r]), tokens[r]), (r, tokens[r])
    again = ops.sample(dev(logits), dev(temps), dev(us)).cpu().tolist()
    assert again == tokens


def test_sample_distribution(ops):
    """Many draws over a small vocabulary follow softmax(logits / T)."""
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]])
    n = 4000
    us = (torch.arange(n) + 0.5) / n
    tokens = ops.sample(dev(logits.expand(n, 5).contiguous()), dev(torch.full((n,), 0.7)), dev(us)).cpu()
    freq = torch.bincount(tokens.long(), minlength=5).float() / n
    torch.testing.assert_close(freq, torch.softmax(logits[0] / 0.7, -1), atol=2e-3, rtol=0)


@pytest.mark.parametrize("tokens", [1, 8, 17, 64])
@pytest.mark.parametrize("features,k", [(128, 64), (200, 200), (6144, 4096), (4096, 12288), (1000, 4096),
                                        (1001, 1024), (3, 200)])
def test_small_m_gemm_on_tcgen05(ops, tokens, features, k):
    """The weight-streaming tcgen05 kernel: partial sums of every split add up to x @ w^T (float32 reference on the
    same bfloat16 values), for token counts that pad to 16/32/64, feature counts that are no multiple of the
    128-row tile (nor of the four features a lane stores at once) and K that is no multiple of the 64-element
    stage."""
    g = torch.Generator().manual_seed(tokens * 1000 + features)
    x = torch.randn(tokens, k, generator=g).to(torch.bfloat16)
    w = (torch.randn(features, k, generator=g) * k ** -0.5).to(torch.bfloat16)
    want = x.float() @ w.float().t()
    status = status_word()
    for splits in (None, 1, 3):
        parts = ops.small_m_gemm(dev(x), dev(w), splits=splits, parts=True, status=status)
        assert parts.dtype == torch.float32 and parts.shape[1:] == (tokens, features)
        torch.testing.assert_close(parts.sum(0).cpu(), want, atol=2e-3, rtol=2e-3)
    # the splits of a tile as a cluster: partial tiles added up through distributed shared memory
    for splits in (None, 1, 2, 4, 8):
        if splits is not None and splits > (k + 63) // 64:
            continue
        out = ops.small_m_gemm(dev(x), dev(w), out_dtype=torch.float32, splits=splits, status=status)
        torch.testing.assert_close(out.cpu(), want, atol=2e-3, rtol=2e-3)
    out = ops.small_m_gemm(dev(x), dev(w), out_dtype=torch.bfloat16, status=status)
    torch.testing.assert_close(out.float().cpu(), want, atol=3e-2, rtol=3e-2)
    assert int(status.item()) == 0
    # the public product goes through the same kernel; with a bias it is the library's
    torch.testing.assert_close(ops.linear(dev(x), dev(w), out_dtype=torch.float32).cpu(), want, atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(ops.linear(dev(x), dev(w)).float().cpu(), want, atol=3e-2, rtol=3e-2)
    bias = torch.randn(features, generator=g).to(torch.bfloat16)
    torch.testing.assert_close(ops.linear(dev(x), dev(w), dev(bias)).float().cpu(), want + bias.float(), atol=3e-2,
                               rtol=3e-2)


def test_consumers_add_up_partial_sums(ops):
    """Norm, q/k-norm and SiLU-mul take a 3-D float32 stack of split-K partial sums and add it up themselves."""
    g = torch.Generator().manual_seed(77)
    parts = torch.randn(3, 5, 256, generator=g)
    total = parts.sum(0)
    h = torch.randn(5, 256, generator=g)
    w = 1 + 0.1 * torch.randn(256, generator=g)
    h_dev = dev(h.clone())
    out = ops.add_rmsnorm(h_dev, dev(parts), dev(w), 1e-6, torch.bfloat16)
    torch.testing.assert_close(h_dev.cpu(), h + total, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(out.float().cpu(), plain.rms_norm(h + total, w, 1e-6), **tol(torch.bfloat16))
    out = ops.silu_mul(dev(parts), torch.bfloat16)
    want = torch.nn.functional.silu(total[:, :128]) * total[:, 128:]
    torch.testing.assert_close(out.float().cpu(), want, **tol(torch.bfloat16))
    nh, nkv, d = 2, 1, 64
    positions = torch.arange(5, dtype=torch.int32)
    inv = plain.rope_inverse_frequencies(d, 10000.0)
    qw, kw = torch.ones(d), torch.ones(d)
    q = ops.qk_norm_rope_write(dev(parts), dev(positions), None, dev(qw), dev(kw), dev(inv), None, None, num_heads=nh,
                               num_kv_heads=nkv, head_dim=d, rotary_dim=d, eps=1e-6)
    q_ref, _, _ = _qkv_reference(total, positions, qw, kw, nh, nkv, d, 1e-6, 10000.0)
    torch.testing.assert_close(q.float().cpu().view(5, nh, d), q_ref, **tol(torch.bfloat16))
