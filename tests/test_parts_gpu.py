"""Each part a layer is put together from, built alone from its spec and compared with the plain
implementation's function for that part: norm, position encoding, attention (with a cache of its own),
feed-forward, embedding, head, and the pre-norm block."""

import pytest
import torch

from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=3e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def build(registry, spec, hidden, dtype):
    from ampere_kv_engine_b200.parts.base import build_part
    return build_part(registry, spec, hidden_size=hidden, dtype=dtype, device=torch.device("cuda"))


def random_params(part, seed, dtype):
    """Random tensors for a part: (what the part is given, the same values as float32 on the host)."""
    from ampere_kv_engine_b200.weights.loader import cast_for
    g = torch.Generator().manual_seed(seed)
    given, host = {}, {}
    for name, ps in part.param_specs().items():
        t = torch.randn(ps.shape, generator=g)
        t = 1 + 0.1 * t if ps.init == "norm" else 0.05 * t
        cast = cast_for(ps, t, dtype)
        given[name] = cast.to("cuda")
        host[name] = cast.float()
    part.load(given)
    return host


def attention_setup(spec, hidden, dtype, page_size, q_lens, starts):
    """A cache manager and a step context for one mixer; sequences already hold ``starts`` positions."""
    from ampere_kv_engine_b200.cache.manager import CacheManager
    from ampere_kv_engine_b200.engine.batch import SeqStep, build_context
    from ampere_kv_engine_b200.parts.base import MIXERS
    mixer = build(MIXERS, spec, hidden, dtype)
    manager = CacheManager([mixer.cache_spec()], [None], page_size=page_size, num_pages=64, max_seqs=8, dtype=dtype,
                           device="cuda")
    return mixer, manager


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from ampere_kv_engine_b200.config.spec import PartSpec
    from ampere_kv_engine_b200.parts.base import NORMS
    part = build(NORMS, PartSpec("rmsnorm", {"eps": 3e-5}), 200, dtype)
    host = random_params(part, 0, dtype)
    h = torch.randn(13, 200)
    delta = torch.randn(13, 200).to(dtype)
    h_dev = h.cuda()
    out = part.forward(h_dev, delta.cuda(), None)
    torch.testing.assert_close(h_dev.cpu(), h + delta.float(), atol=0, rtol=0)
    torch.testing.assert_close(out.float().cpu(), plain.rms_norm(h + delta.float(), host["weight"], 3e-5), **tol(dtype))
    assert out.dtype == dtype


def test_rope_part_matches_plain_table():
    from ampere_kv_engine_b200.config.spec import PartSpec
    from ampere_kv_engine_b200.parts.base import POSITION_ENCODINGS
    part = build(POSITION_ENCODINGS, PartSpec("rope", {"theta": 1e6, "rotary_dim": 96}), 64, torch.float32)
    inv, rd = part.fused_rotary()
    assert rd == 96
    torch.testing.assert_close(inv.cpu(), plain.rope_inverse_frequencies(96, 1e6), atol=0, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 21])
def test_attention_part_against_plain(dtype, window):
    """Prompt in two portions, then two decoded tokens, for two sequences at once; outputs of all positions
    equal the plain attention part run on the whole sequences."""
    from ampere_kv_engine_b200.config.spec import PartSpec
    from ampere_kv_engine_b200.engine.batch import SeqStep, build_context
    hidden, nh, nkv, d, eps, theta = 72, 6, 2, 48, 2e-6, 30000.0
    spec = PartSpec("attention", {"num_heads": nh, "num_kv_heads": nkv, "head_dim": d, "qk_norm": True,
                                  "qk_norm_eps": eps, "bias": True, "window": window, "scale": None,
                                  "position_encoding": PartSpec("rope", {"theta": theta, "rotary_dim": d})}, "attn")
    mixer, manager = attention_setup(spec, hidden, dtype, 8, None, None)
    host = random_params(mixer, 1, dtype)
    w = {f"attn.{k}": v for k, v in host.items()}
    g = torch.Generator().manual_seed(2)
    xs = {"a": torch.randn(61, hidden, generator=g).to(dtype), "b": torch.randn(30, hidden, generator=g).to(dtype)}
    want = {k: plain.attention_part(x.float(), torch.arange(x.shape[0]), w, "attn", num_heads=nh, num_kv_heads=nkv,
                                    head_dim=d, eps=eps, theta=theta, window=window) for k, x in xs.items()}
    seqs = {k: manager.open(k) for k in xs}
    view = manager.layer_view(0)
    plan = [{"a": 40, "b": 7}, {"a": 19, "b": 21}, {"a": 1, "b": 1}, {"a": 1, "b": 1}]
    done = {k: 0 for k in xs}
    got = {k: [] for k in xs}
    for step in plan:
        entries = []
        for k, n in step.items():
            manager.reserve(seqs[k], n)
            entries.append(SeqStep(seqs[k], [0] * n))
        ctx = build_context(manager, entries, torch.device("cuda"), status=torch.zeros(1, dtype=torch.int32, device="cuda"))
        x = torch.cat([xs[k][done[k]:done[k] + n] for k, n in step.items()]).cuda()
        out = mixer.forward(x, ctx, view).float().cpu()
        assert int(ctx.status.item()) == 0
        row = 0
        for k, n in step.items():
            got[k].append(out[row:row + n])
            row += n
            done[k] += n
            manager.commit(seqs[k], n)
    for k in xs:
        torch.testing.assert_close(torch.cat(got[k]), want[k], **tol(dtype))
    manager.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_mlp_part(dtype):
    from ampere_kv_engine_b200.config.spec import PartSpec
    from ampere_kv_engine_b200.parts.base import FEED_FORWARDS
    part = build(FEED_FORWARDS, PartSpec("gated_mlp", {"intermediate_size": 136, "activation": "silu"}, "mlp"), 72, dtype)
    host = random_params(part, 3, dtype)
    x = torch.randn(17, 72).to(dtype)
    out = part.forward(x.cuda(), None)
    want = plain.gated_mlp(x.float(), {f"mlp.{k}": v for k, v in host.items()}, "mlp")
    torch.testing.assert_close(out.float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from ampere_kv_engine_b200.config.spec import PartSpec
    from ampere_kv_engine_b200.parts.embedding import LinearHead, TokenEmbedding
    kw = dict(hidden_size=72, dtype=dtype, device=torch.device("cuda"))
    emb = TokenEmbedding(PartSpec("token_embedding", {"vocab_size": 333}, "emb"), **kw)
    host = random_params(emb, 4, dtype)
    ids = torch.tensor([0, 332, 17, 17], dtype=torch.int32)
    torch.testing.assert_close(emb.forward(ids.cuda(), None).cpu(), host["weight"][ids.long()], atol=0, rtol=0)
    tied = LinearHead(PartSpec("linear_head", {"vocab_size": 333, "tied": True}, "head"), **kw)
    tied.load({})
    tied.tie(emb)
    x = torch.randn(5, 72).to(dtype)
    logits = tied.forward(x.cuda())
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.cpu(), x.float() @ host["weight"].t(), **tol(dtype))
    own = LinearHead(PartSpec("linear_head", {"vocab_size": 333, "tied": False}, "head"), **kw)
    host_head = random_params(own, 5, dtype)
    torch.testing.assert_close(own.forward(x.cuda()).cpu(), x.float() @ host_head["weight"].t(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_prenorm_block_against_plain_layer(dtype):
    """One whole layer (norm, attention, residual, norm, feed-forward, residual) on a whole sequence."""
    from ampere_kv_engine_b200.cache.manager import CacheManager
    from ampere_kv_engine_b200.config.spec import LayerSpec, PartSpec
    from ampere_kv_engine_b200.engine.batch import SeqStep, build_context
    from ampere_kv_engine_b200.parts.base import BLOCKS
    cfg = {"hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 32,
           "intermediate_size": 112, "rms_norm_eps": 1e-5, "rope_theta": 12345.0, "num_hidden_layers": 1}
    p = "model.layers.0"
    layer = LayerSpec(
        "prenorm",
        mixer=PartSpec("attention", {
            "num_heads": 5, "num_kv_heads": 5, "head_dim": 32, "qk_norm": True, "qk_norm_eps": 1e-5, "bias": False,
            "window": None, "scale": None, "position_encoding": PartSpec("rope", {"theta": 12345.0, "rotary_dim": 32})},
            f"{p}.self_attn"),
        feed_forward=PartSpec("gated_mlp", {"intermediate_size": 112}, f"{p}.mlp"),
        mixer_norm=PartSpec("rmsnorm", {"eps": 1e-5}, f"{p}.input_layernorm"),
        feed_forward_norm=PartSpec("rmsnorm", {"eps": 1e-5}, f"{p}.post_attention_layernorm"))
    # the block kind builds its own parts from the roles of the layer spec
    block = BLOCKS.get("prenorm")(layer, hidden_size=80, dtype=dtype, device=torch.device("cuda"))
    mixer = block.mixer
    assert [type(x).__name__ for x in block.parts()] == ["RMSNorm", "PagedAttention", "RMSNorm", "GatedMLP"]
    w = {}
    for i, part in enumerate(block.parts()):
        for k, v in random_params(part, 10 + i, dtype).items():
            w[f"{part.spec.prefix}.{k}"] = v
    manager = CacheManager([mixer.cache_spec()], [None], page_size=16, num_pages=8, max_seqs=2, dtype=dtype, device="cuda")
    seq = manager.open("s")
    manager.reserve(seq, 50)
    ctx = build_context(manager, [SeqStep(seq, [0] * 50)], torch.device("cuda"),
                        status=torch.zeros(1, dtype=torch.int32, device="cuda"))
    h = torch.randn(50, 80)
    hidden, delta = block.forward(h.cuda(), None, ctx, manager.layer_view(0))
    got = hidden.cpu() + delta.float().cpu()
    want = plain.decoder_layer(h, torch.arange(50), w, 0, cfg, None)
    torch.testing.assert_close(got, want, **tol(dtype))
