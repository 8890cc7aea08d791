"""The plain implementation itself: against the reference project's own forward pass (committed golden
logits, see tests/golden/make_golden.py), against an independent float64 attention formula, and a few
properties of its parts."""

import importlib.util
import os

import torch
from safetensors.torch import load_file

import tiny
from plain import qwen3_plain as plain

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _golden_cases():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return list(module.cases())


def test_plain_equals_the_references_own_forward():
    golden = load_file(os.path.join(GOLDEN, "reference_logits.safetensors"))
    checked = 0
    for name, cfg, ids in _golden_cases():
        logits = plain.forward_logits(plain.random_weights(cfg, 1), cfg, ids)[-1]
        for key in (f"{name}.len{len(ids)}.whole", f"{name}.len{len(ids)}.portions"):
            if key in golden:
                torch.testing.assert_close(logits, golden[key], atol=2e-6, rtol=1e-5)
                checked += 1
    assert checked == len(golden) == 10


def test_attention_against_float64_formula():
    """Same independent check the reference runs on its own attention (ampere_kv/check_chunked.py:13-26)."""
    g = torch.Generator().manual_seed(7)
    q = torch.randn(65, 4, 8, generator=g)
    k = torch.randn(65, 2, 8, generator=g)
    v = torch.randn(65, 2, 8, generator=g)
    scores = torch.einsum("thd,shd->hts", q.double(), k.double().repeat_interleave(2, dim=1)) / 8 ** 0.5
    future = torch.ones(65, 65, dtype=torch.bool).triu(1)
    want = torch.einsum("hts,shd->thd", scores.masked_fill(future, -torch.inf).softmax(-1),
                        v.double().repeat_interleave(2, dim=1))
    torch.testing.assert_close(plain.causal_attention(q, k, v).double(), want, atol=1e-5, rtol=1e-5)


def test_window_sees_exactly_its_last_keys():
    g = torch.Generator().manual_seed(8)
    q, k, v = (torch.randn(30, 2, 16, generator=g) for _ in range(3))
    out = plain.causal_attention(q, k, v, window=7)
    for t in (0, 5, 6, 7, 29):
        lo = max(0, t - 6)
        alone = plain.causal_attention(q[lo:t + 1], k[lo:t + 1], v[lo:t + 1])[-1]
        torch.testing.assert_close(out[t], alone, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(plain.causal_attention(q, k, v, window=30), plain.causal_attention(q, k, v))


def test_rope_rotates_pairs_and_keeps_norms():
    inv = plain.rope_inverse_frequencies(16, 10000.0)
    assert inv.dtype == torch.float32 and float(inv[0]) == 1.0
    torch.testing.assert_close(inv[1], torch.tensor(10000.0 ** (-2 / 16)))
    x = torch.randn(5, 3, 16)
    pos = torch.tensor([0, 1, 2, 100, 4000])
    y = plain.apply_rope(x, pos, inv)
    torch.testing.assert_close(y[0], x[0])                                   # position 0 is the identity
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5, rtol=1e-5)
    # scores depend on the distance only
    a, b = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    s1 = (plain.apply_rope(a, torch.tensor([10]), inv) * plain.apply_rope(b, torch.tensor([3]), inv)).sum()
    s2 = (plain.apply_rope(a, torch.tensor([107]), inv) * plain.apply_rope(b, torch.tensor([100]), inv)).sum()
    torch.testing.assert_close(s1, s2, atol=1e-4, rtol=1e-4)


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    want = x / ((9 + 16) / 2 + 1e-6) ** 0.5 * w
    torch.testing.assert_close(plain.rms_norm(x, w, 1e-6), want)


def test_later_tokens_do_not_change_earlier_logits():
    for name in ("A", "B"):
        cfg = tiny.config(name)
        w = plain.random_weights(cfg, 2)
        ids = torch.randint(0, cfg["vocab_size"], (60,), generator=torch.Generator().manual_seed(1)).tolist()
        full = plain.forward_logits(w, cfg, ids)
        torch.testing.assert_close(plain.forward_logits(w, cfg, ids[:41]), full[:41], atol=1e-5, rtol=1e-5)
        assert full.shape == (60, cfg["vocab_size"]) and full.dtype == torch.float32


def test_window_layers_change_the_result_only_past_the_window():
    cfg = tiny.config("B")
    w = plain.random_weights(cfg, 2)
    ids = torch.randint(0, cfg["vocab_size"], (70,), generator=torch.Generator().manual_seed(3)).tolist()
    windowed = plain.forward_logits(w, cfg, ids)
    cfg_full = dict(cfg, use_sliding_window=False)
    full = plain.forward_logits(w, cfg_full, ids)
    torch.testing.assert_close(windowed[:40], full[:40], atol=1e-6, rtol=1e-5)
    assert float((windowed[60:] - full[60:]).abs().max()) > 1e-4


def test_sampling_helpers():
    assert plain.uniform_from_key(1, 2, 3) == plain.uniform_from_key(1, 2, 3) != plain.uniform_from_key(1, 2, 4)
    us = [plain.uniform_from_key(5, 0, i) for i in range(2000)]
    assert 0 <= min(us) and max(us) < 1 and abs(sum(us) / 2000 - 0.5) < 0.03
    logits = torch.tensor([0.0, 1.0, 2.0])
    p = torch.softmax(logits / 0.5, -1)
    assert plain.sample_temperature(logits, 0.5, float(p[0]) - 1e-6) == 0
    assert plain.sample_temperature(logits, 0.5, float(p[0]) + 1e-6) == 1
    assert plain.sample_temperature(logits, 0.5, 0.999999) == 2
    assert plain.sample_temperature(logits, 0.0, 0.3) == 2
