"""The chained-product kernel (one persistent launch for a list of dependent products) against plain float32
arithmetic with the kernels' rounding points, at the benchmark model's layer sizes and at sizes that divide nothing
evenly; repeated launches agree bit for bit whichever CTA finishes a tile last."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def bf(t):
    return t.to(torch.bfloat16).float()


def reference_chain(hidden, attn_out, w, cfg, positions):
    """o-projection + residual -> norm + gate/up + SiLU-mul -> down + residual -> norm + q/k/v with per-head norm and
    rotation, in float64 with every stored tensor rounded to bfloat16 where the kernels round."""
    d = torch.float64
    h = hidden.to(d) + bf((attn_out.to(d) @ w["o"].to(d).t()).float()).to(d)

    def normed(x, weight, eps):
        return bf((x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * weight.to(d)).float()).to(d)

    x2 = normed(h, w["post_norm"], cfg["eps"])
    inter = w["gate"].shape[0]
    g = bf((x2 @ w["gate"].to(d).t()).float()).to(d)
    u = bf((x2 @ w["up"].to(d).t()).float()).to(d)
    act = bf((g / (1 + torch.exp(-g)) * u).float()).to(d)
    h2 = h + bf((act @ w["down"].to(d).t()).float()).to(d)
    x3 = normed(h2, w["next_norm"], cfg["eps"])
    qkv = bf((x3 @ w["qkv"].to(d).t()).float()).to(d)
    nh, nkv = cfg["heads"], cfg["kv_heads"]
    heads = qkv.view(-1, nh + 2 * nkv, 128)
    q, k, v = heads[:, :nh], heads[:, nh:nh + nkv], heads[:, nh + nkv:]

    def head_norm(t, weight):
        return t * torch.rsqrt(t.square().mean(-1, keepdim=True) + cfg["qk_eps"]) * weight.to(d)

    def rotate(t):
        ang = positions.to(d)[:, None] * w["inv_freq"].to(d)[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        a, b = t[..., :64], t[..., 64:]
        return torch.cat((a * cos - b * sin, b * cos + a * sin), -1)

    q, k = rotate(head_norm(q, w["q_norm"])), rotate(head_norm(k, w["k_norm"]))
    return h2.float(), act.float(), q.reshape(q.shape[0], -1).float(), k.float(), v.float()


def make_case(tokens, hidden, inter, heads, kv_heads, seed, page=16):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, scale=0.02: (torch.randn(*s, generator=g) * scale)
    w = {"o": bf(r(hidden, heads * 128)), "gate": bf(r(inter, hidden)), "up": bf(r(inter, hidden)),
         "down": bf(r(hidden, inter)), "qkv": bf(r((heads + 2 * kv_heads) * 128, hidden)),
         "post_norm": 1 + r(hidden, scale=0.1), "next_norm": 1 + r(hidden, scale=0.1),
         "q_norm": 1 + r(128, scale=0.1), "k_norm": 1 + r(128, scale=0.1),
         "inv_freq": 1.0 / (1e6 ** (torch.arange(0, 128, 2).float() / 128))}
    hidden_in = r(tokens, hidden, scale=1.0)
    attn_out = bf(r(tokens, heads * 128, scale=1.0))
    positions = torch.randint(0, 3000, (tokens,), generator=g, dtype=torch.int32)
    pages = tokens + 3
    slots = (torch.randperm(pages * page, generator=g)[:tokens]).to(torch.int32)
    return w, hidden_in, attn_out, positions, slots, pages, page


@pytest.mark.parametrize("tokens,hidden,inter,heads,kv_heads", [
    (8, 4096, 12288, 32, 8), (1, 4096, 12288, 32, 8), (5, 512, 1152, 8, 2), (3, 320, 448, 3, 1), (7, 1024, 2048, 8, 8)])
def test_chain_of_four_products_matches_float_arithmetic(tokens, hidden, inter, heads, kv_heads):
    from ampere_kv_engine_b200.kernels import ops
    cfg = {"eps": 1e-6, "qk_eps": 1e-5, "heads": heads, "kv_heads": kv_heads}
    w, hidden_in, attn_out, positions, slots, pages, page = make_case(tokens, hidden, inter, heads, kv_heads, tokens)
    dev = lambda t, dt=None: (t if dt is None else t.to(dt)).cuda().contiguous()
    gate_up = ops.interleave_gate_up(dev(w["gate"], torch.bfloat16), dev(w["up"], torch.bfloat16), 64).contiguous()
    want_h, want_act, want_q, want_k, want_v = reference_chain(hidden_in, attn_out, w, cfg, positions)
    outs = []
    for attempt in range(3):
        h = dev(hidden_in)
        act = torch.full((tokens, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
        q_out = torch.full((tokens, heads * 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        k_cache = torch.full((pages, kv_heads, page, 128), float("nan"), dtype=torch.bfloat16, device="cuda")
        v_cache = k_cache.clone()
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        phases = [
            {"w": dev(w["o"], torch.bfloat16), "x": dev(attn_out, torch.bfloat16), "epilogue": "residual"},
            {"w": gate_up, "norm_weight": dev(w["post_norm"]), "eps": cfg["eps"], "epilogue": "gated", "out": act},
            {"w": dev(w["down"], torch.bfloat16), "x": act, "epilogue": "residual"},
            {"w": dev(w["qkv"], torch.bfloat16), "norm_weight": dev(w["next_norm"]), "eps": cfg["eps"],
             "epilogue": "qkv", "q_out": q_out, "positions": dev(positions), "slots": dev(slots),
             "q_weight": dev(w["q_norm"]), "k_weight": dev(w["k_norm"]), "inv_freq": dev(w["inv_freq"]),
             "k_cache": k_cache, "v_cache": v_cache, "num_heads": heads, "num_kv_heads": kv_heads,
             "qk_eps": cfg["qk_eps"]},
        ]
        ops.stream_begin_step("cuda")
        ops.stream_phases(h, phases, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        s = slots.long()
        got_k = k_cache[s // page, :, s % page].float().cpu()
        got_v = v_cache[s // page, :, s % page].float().cpu()
        outs.append((h.cpu(), act.float().cpu(), q_out.float().cpu(), got_k, got_v))
        # nothing but the tokens' own slots was written
        written = torch.zeros(pages * page, dtype=torch.bool)
        written[s] = True
        assert bool(torch.isnan(k_cache.float().cpu().permute(0, 2, 1, 3).reshape(pages * page, -1)[~written]).all())
    h, act, q, k, v = outs[0]
    tol = dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(act, want_act, **tol)
    # the products that go into the stream are rounded to bfloat16 first and reach magnitudes of 4 to 8, where one
    # step of bfloat16 is 0.031: two float32 sums cut at different places may round to neighbouring steps
    torch.testing.assert_close(h, want_h, atol=4e-2, rtol=2e-2)
    torch.testing.assert_close(q, want_q, atol=4e-2, rtol=3e-2)
    torch.testing.assert_close(k, want_k, atol=4e-2, rtol=3e-2)
    torch.testing.assert_close(v, want_v, **tol)
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert torch.equal(a, b), "two launches of the same chain differ"


def test_single_phases_match_the_per_product_kernels():
    """Each kind of phase alone against the existing one-product kernel with the same epilogue (the sums are cut at
    other places, so the results agree to rounding, not bit for bit), and a normed first phase without sums of
    squares from a residual phase (they are added up in the kernel)."""
    from ampere_kv_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    tokens, hidden, inter = 6, 1024, 1536
    x = (torch.randn(tokens, hidden, generator=g)).to(torch.bfloat16).cuda()
    w_res = (torch.randn(hidden, hidden, generator=g) * 0.02).to(torch.bfloat16).cuda()
    w_plain = (torch.randn(inter, hidden, generator=g) * 0.02).to(torch.bfloat16).cuda()
    h0 = torch.randn(tokens, hidden, generator=g).cuda()
    norm_w = (1 + 0.1 * torch.randn(hidden, generator=g)).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # residual
    h_a, h_b = h0.clone(), h0.clone()
    ops.stream_begin_step("cuda")
    ops.stream_phases(h_a, [{"w": w_res, "x": x, "epilogue": "residual"}], status=status)
    assert ops.linear_into_residual(x, w_res, h_b, status=status) is not None
    torch.testing.assert_close(h_a, h_b, atol=1e-2, rtol=1e-2)
    # plain product of the normed stream, sums of squares made in the kernel
    out = torch.empty((tokens, inter), dtype=torch.bfloat16, device="cuda")
    ops.stream_phases(h_a, [{"w": w_plain, "norm_weight": norm_w, "eps": 1e-6, "epilogue": "plain", "out": out}],
                      status=status)
    normed = ops.add_rmsnorm(h_a.clone(), None, norm_w, 1e-6, torch.bfloat16)
    want = ops.linear(normed, w_plain)
    torch.testing.assert_close(out.float(), want.float(), atol=2e-2, rtol=2e-2)
    assert int(status.item()) == 0


@pytest.mark.parametrize("name", ["A", "C"])
def test_engine_with_the_chained_kernel_switched_on(name, monkeypatch):
    """The whole engine with the option on (it is off by default: the four separate kernels are faster): decoded
    tokens, portions of two and three tokens, mixed steps of up to eight tokens and captured decode graphs all take
    the chained-product kernel, and every row must still equal the plain implementation's."""
    import replay_util as ru
    import tiny
    from ampere_kv_engine_b200.kernels import ops
    from models_util import model_folder, plain_logits
    monkeypatch.setattr(ops, "use_stream_phases", True)
    raw, page = tiny.CONFIGS[name]
    folder = model_folder(name)
    requests = ru.make_requests(raw["vocab_size"], (5, 17, 33, 70, 45), seed=11)
    expected = plain_logits(folder, raw, requests, "bfloat16")
    trace = ru.Trace()
    for mode, sub in (("last", ru.trace_last_decoded(requests)), ("portions", ru.trace_portions(requests)),
                      ("mixed", ru.trace_mixed(requests, 64 * 6, seed=5))):
        trace.extend(sub, mode + ":")
    wanted = {f"{mode}:{rid}": logits for mode in ("last", "portions", "mixed") for rid, logits in expected.items()}
    before = ops.launch_count
    outputs, engine = ru.run_on_device(folder, "bfloat16", trace, 64 * 6, page_size=page, max_seqs=8)
    ru.compare(trace, outputs, wanted, "bfloat16")
    assert engine.runner.graph_replays > 20
    scratch = ops._stream_scratch("cuda")
    assert scratch.high_water > 0          # the kernel did run
