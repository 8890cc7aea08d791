"""The benchmark model's layer sizes (Qwen3-8B: hidden 4096, 32 q-heads / 8 kv-heads of 128 dims, intermediate
12288, 16-token pages) with two layers and a small vocabulary, through bin/trace_run: float32 against the plain
implementation, and bfloat16 (tcgen05 prompt attention, fused decode kernels, split-K at K = 4096 and 12288)
against float32 on the same bfloat16-stored weights, whole, decoded one by one, and mixed with page reuse."""

import tempfile

import pytest
import torch

import replay_util as ru
from models_util import plain_weights
from plain import qwen3_plain

pytestmark = pytest.mark.gpu

FLAGSHIP_LAYERS = {
    "architectures": ["Qwen3ForCausalLM"],
    "model_type": "qwen3",
    "num_hidden_layers": 2,
    "hidden_size": 4096,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "intermediate_size": 12288,
    "vocab_size": 4096,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "max_position_embeddings": 8192,
    "tie_word_embeddings": False,
    "hidden_act": "silu",
    "attention_bias": False,
    "use_sliding_window": False,
    "eos_token_id": 1,
}


def test_flagship_layer_sizes_in_both_precisions():
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    _, cfg = config_from_dict(dict(FLAGSHIP_LAYERS))
    folder = tempfile.mkdtemp(prefix="flagship_layers_")
    write_random_model(cfg, 5, folder, torch.bfloat16)
    requests = ru.make_requests(FLAGSHIP_LAYERS["vocab_size"], (70, 33, 130, 9, 64), seed=3)
    trace = ru.Trace()
    spans = {}
    for mode, sub in (("whole", ru.trace_whole(requests)), ("last32", ru.trace_last_decoded(requests)),
                      ("mixed", ru.trace_mixed(requests, 64 * 6, seed=9))):
        spans[mode] = trace.extend(sub, mode + ":")
    out32 = ru.run_subprocess(folder, "float32", trace, 64 * 6)
    out16 = ru.run_subprocess(folder, "bfloat16", trace, 64 * 6)
    # float32 against the plain implementation (two requests keep the CPU part short)
    short = {rid: requests[rid] for rid in ("r1", "r3")}
    # The plain model's matrix products run in float64 here: sums of 4,096 to 12,288 float32 terms on the CPU depend
    # on how the library splits them over its threads, which changes with the load of the machine, and the
    # difference between two float32 orders is as large as the one this test measures.
    w64 = {k: v.double() for k, v in plain_weights(folder, "float32").items()}
    plain = {rid: qwen3_plain.forward_logits(w64, FLAGSHIP_LAYERS, toks) for rid, toks in short.items()}
    expected = {f"{mode}:{rid}": logits for mode in spans for rid, logits in plain.items()}
    anchored = ru.Trace()
    anchored.expect = {s: rows for s, rows in trace.expect.items() if all(rid in expected for rid, _ in rows)}
    assert anchored.expect
    # The two float32 implementations differ by the order of their sums, which here have 4,096 to 12,288 terms
    # instead of the tiny models' 64 to 160: the error of such a sum grows with the square root of its length, so
    # the absolute part of the tiny models' tolerance (2e-5 at 96 terms) is scaled by sqrt(4096 / 96).
    scale = (FLAGSHIP_LAYERS["hidden_size"] / 96) ** 0.5
    worst32 = 0.0
    for step, rows in anchored.expect.items():
        got = torch.from_numpy(out32[step].copy()).view(len(rows), -1)
        want = torch.stack([expected[rid][pos] for rid, pos in rows])
        bound = ru.TOL["float32"]["atol"] * scale + ru.TOL["float32"]["rtol"] * want.abs()
        diff = (got - want).abs()
        assert bool((diff <= bound).all()), (f"step {step}: float32 differs from the plain implementation by "
                                             f"{float(diff.max()):.3e} (logits up to {float(want.abs().max()):.2f})")
        worst32 = max(worst32, float(diff.max()))
    print(f"float32 vs plain: worst {worst32:.3e}")
    # bfloat16 against float32, every written row.  Stored activations are rounded to 8 bits of mantissa, and a
    # logit is a sum of 4,096 such products after two layers of them: the error is measured against the row's own
    # scale (its root mean square), as a whole (relative RMS error) and at its worst element.
    vocab = FLAGSHIP_LAYERS["vocab_size"]
    worst_rms = worst_peak = 0.0
    for step, rows in trace.expect.items():
        a = torch.from_numpy(out32[step].copy()).view(len(rows), vocab)
        b = torch.from_numpy(out16[step].copy()).view(len(rows), vocab)
        scale_rows = a.square().mean(dim=1).sqrt()
        rel_rms = (a - b).square().mean(dim=1).sqrt() / scale_rows
        peak = (a - b).abs().max(dim=1).values / scale_rows
        worst_rms, worst_peak = max(worst_rms, float(rel_rms.max())), max(worst_peak, float(peak.max()))
    print(f"bfloat16 vs float32: worst relative RMS error {worst_rms:.4f}, worst element / row RMS {worst_peak:.4f}")
    assert 0.0 < worst_rms < 0.02 and worst_peak < 0.1
