"""Seeded random Qwen3 configurations (heads, groups, head sizes in steps of 16, widths and vocabularies that are
no power of two, windows, biases, tied heads, page sizes) through trace replay on the GPU, mixed with page reuse
and decoded token by token, in both precisions, against the plain implementation: whichever kernels a shape is
dispatched to (general, mma.sync, tcgen05, fused decode epilogues or not), the logits must agree."""

import io
import random
import tempfile

import pytest
import torch

import replay_util as ru
from models_util import plain_logits

pytestmark = pytest.mark.gpu


def random_config(seed: int) -> tuple[dict, int]:
    rng = random.Random(seed)
    head_dim = rng.choice([16, 32, 48, 64, 64, 128, 128, 128])
    group = rng.choice([1, 2, 3, 4, 8] if head_dim < 128 else [1, 2, 4, 4, 8])
    kv_heads = rng.choice([1, 2, 3])
    heads = kv_heads * group
    hidden = rng.choice([64, 72, 96, 136, 192, 320]) if rng.random() < 0.6 else heads * head_dim
    hidden = max(64, hidden // 8 * 8)
    layers = rng.choice([1, 2, 3])
    window = rng.choice([None, None, 24, 70])
    cfg = {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": layers,
        "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": head_dim,
        "intermediate_size": rng.choice([64, 96, 128, 136, 192, 200, 320]), "vocab_size": rng.choice([257, 500, 1000, 1531]),
        "rope_theta": rng.choice([10000.0, 1000000.0]), "rms_norm_eps": rng.choice([1e-6, 1e-5]),
        "max_position_embeddings": 1024, "tie_word_embeddings": rng.random() < 0.5, "hidden_act": "silu",
        "attention_bias": rng.random() < 0.3, "use_sliding_window": window is not None,
        "eos_token_id": 1,
    }
    if window is not None:
        cfg["sliding_window"] = window
        cfg["max_window_layers"] = rng.randrange(0, layers)
    return cfg, rng.choice([8, 16, 16, 32, 64])


@pytest.mark.parametrize("seed", range(16))
def test_random_configuration_matches_plain(seed):
    from ampere_kv_engine_b200 import replay
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.random_init import write_random_model
    raw, page = random_config(seed)
    _, cfg = config_from_dict(dict(raw))
    folder = tempfile.mkdtemp(prefix=f"random_config_{seed}_")
    write_random_model(cfg, seed, folder, torch.float32)
    requests = ru.make_requests(raw["vocab_size"], (2, 45, 90, 131, 17), seed=seed + 100)
    trace = ru.Trace()
    trace.extend(ru.trace_mixed(requests, 64 * 6, seed=seed), "mixed:")
    trace.extend(ru.trace_last_decoded(requests), "last32:")
    for dtype in ("float32", "bfloat16"):
        plain = plain_logits(folder, raw, requests, dtype)
        expected = {f"{mode}:{rid}": logits for mode in ("mixed", "last32") for rid, logits in plain.items()}
        out = tempfile.mkdtemp(prefix="replay_out_")
        sink = io.StringIO()
        argv = ["--model", folder, "--dtype", dtype, "--out", out, "--max-tokens", str(64 * 6), "--page-size", str(page)]
        assert replay.main(argv, stdin=io.StringIO(trace.lines()), stdout=sink) == 0, raw
        try:
            ru.compare(trace, ru.read_outputs(out, trace), expected, dtype)
        except AssertionError as error:
            raise AssertionError(f"configuration {raw}, page size {page}, {dtype}: {error}") from None
