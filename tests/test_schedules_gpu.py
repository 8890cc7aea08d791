"""The schedules that serving and the benchmark run, each compared with the plain implementation in float32 and in
bfloat16:

* a request decoded across the edge of a block-table bucket, so that a second decode graph is captured in the
  middle of it (the benchmark's 1,024-token prompts live beyond the first bucket);
* decode steps of 12, 40 and 70 live sequences of mixed lengths, with requests ending and joining on the way
  (the batch buckets above 8, the 9-to-32-token and the 33-to-64-token regimes of the decode products);
* generation of some forty requests through the scheduler, rounds queued one ahead, an end-of-sequence token that
  stops some of them;
* the benchmark model itself, all 36 layers and all 151,936 logits, float32 and bfloat16 against the plain model
  run on the GPU in true float32.
"""

import gc
import math
import random

import pytest
import torch

import replay_util as ru
import tiny
from models_util import model_folder, plain_logits, plain_weights
from plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


# --------------------------------------------------------------------------- across a block-table bucket

def _long_trace(tokens, portions, decoded):
    """One request: ``portions`` (each wanting its last place and one in the middle), then ``decoded`` single
    tokens, each wanted."""
    trace = ru.Trace()
    p = 0
    for n in portions:
        trace.add([("long", tokens[p:p + n], p, sorted({n // 2, n - 1}))])
        p += n
    for i in range(decoded):
        trace.add([("long", tokens[p:p + 1], p, [0])], end=["long"] if i == decoded - 1 else [])
        p += 1
    assert p == len(tokens)
    return trace


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("A", 16), ("C", 16), ("C", 64)])
def test_decode_crosses_a_block_table_bucket(name, page_size, dtype):
    """1,000 tokens in portions, then 180 one by one.  With 16-token pages the request's block table grows past 64
    pages at position 1,024: the decode graph captured for the first bucket of table widths no longer fits and a
    second one is captured in the middle of the request, with its own table width and split counts."""
    from ampere_kv_engine_b200.engine import step as step_module
    raw, _ = tiny.CONFIGS[name]
    folder = model_folder(name)
    requests = ru.make_requests(raw["vocab_size"], (1180,), seed=31)
    tokens = requests["r0"]
    trace = _long_trace(tokens, (300, 17, 2, 411, 270), 180)
    expected = {"long": plain_logits(folder, raw, requests, dtype)["r0"]}
    outputs, engine = ru.run_on_device(folder, dtype, trace, 1216, page_size=page_size, max_seqs=4)
    ru.check(trace, outputs, expected, dtype, many_rows=True)
    runner = engine.runner
    assert runner.cuda_graphs and runner.graph_replays >= 170
    widths = sorted(key[-1] for key in runner._captured)
    if page_size == 16:
        assert 1180 // page_size > step_module._WIDTH_STEP          # the request did cross the bucket's edge
        assert len(runner._captured) == 2 and widths[0] != widths[1], widths
    else:
        assert len(runner._captured) == 1
    assert runner.manager.free_pages() == [g.pool.count for g in runner.manager.groups]


def test_bucket_edge_through_the_replay_program():
    """The same request through ``bin/trace_run`` as a user runs it (bfloat16, graphs on by default)."""
    raw, _ = tiny.CONFIGS["C"]
    folder = model_folder("C")
    requests = ru.make_requests(raw["vocab_size"], (1180,), seed=31)
    trace = _long_trace(requests["r0"], (1000,), 180)
    outputs = ru.run_subprocess(folder, "bfloat16", trace, 1216, page_size=16)
    ru.check(trace, outputs, {"long": plain_logits(folder, raw, requests, "bfloat16")["r0"]}, "bfloat16", many_rows=True)


# --------------------------------------------------------------------------- many sequences decoding

def _crowd_trace(requests, decode_steps, seed):
    """Prompts in mixed steps of several requests, then ``decode_steps`` rounds in which every live request brings
    one token.  A third of the requests are short and end on the way; one latecomer's prompt arrives in portions
    beside the others' decoded tokens."""
    rng = random.Random(seed)
    trace = ru.Trace()
    ids = list(requests)
    late = ids[-1]
    crowd = ids[:-1]
    decode_from = {r: len(requests[r]) - (decode_steps if i % 3 else decode_steps // 2) for i, r in enumerate(crowd)}
    assert all(v >= 1 for v in decode_from.values())
    fed = {r: 0 for r in ids}
    pending = list(crowd)
    while pending:                                  # prompts: up to six requests a step, portions of mixed sizes
        entries = []
        for r in pending[:6]:
            n = min(decode_from[r] - fed[r], rng.choice((3, 17, 40, 64)))
            entries.append((r, requests[r][fed[r]:fed[r] + n], fed[r], [n - 1]))
            fed[r] += n
        trace.add(entries)
        pending = [r for r in pending if fed[r] < decode_from[r]]
    for round_index in range(decode_steps):
        entries, ended = [], []
        for r in crowd:
            if fed[r] < len(requests[r]):
                entries.append((r, requests[r][fed[r]:fed[r] + 1], fed[r], [0]))
                fed[r] += 1
                if fed[r] == len(requests[r]):
                    ended.append(r)
        if round_index >= 3 and fed[late] < len(requests[late]):     # the latecomer: portions, then single tokens
            left = len(requests[late]) - fed[late]
            n = 1 if left <= 4 else min(left - 4, rng.choice((5, 9, 24)))
            entries.append((late, requests[late][fed[late]:fed[late] + n], fed[late], [n - 1]))
            fed[late] += n
            if fed[late] == len(requests[late]):
                ended.append(late)
        trace.add(entries, end=ended)
    left_open = [r for r in ids if fed[r] < len(requests[r])]
    assert not left_open, left_open
    return trace


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("live", [12, 40, 70])
def test_decode_steps_of_many_sequences(live, dtype):
    """12, 40 and 70 sequences decode together for 24 rounds (config C: the benchmark model's head shape, so the
    bfloat16 run takes the tensor-core attention and the package's own decode products up to 32 tokens and the
    library products with separate norm, activation and q/k kernels above).  Pure decode rounds are replayed
    graphs of the batch buckets 12/16, 48/32, 96/64; rounds with the latecomer's portion run as they come."""
    raw, page = tiny.CONFIGS["C"]
    folder = model_folder("C")
    rng = random.Random(live)
    lengths = [rng.choice((26, 31, 47, 64, 90, 133, 200)) for _ in range(live - 1)] + [61]
    requests = ru.make_requests(raw["vocab_size"], lengths, seed=live)
    trace = _crowd_trace(requests, 24, seed=live)
    assert max(len(s["entries"]) for s in trace.steps) == live
    expected = plain_logits(folder, raw, requests, dtype)
    max_tokens = sum((n + 63) // 64 * 64 for n in lengths)
    outputs, engine = ru.run_on_device(folder, dtype, trace, max_tokens, page_size=page, max_seqs=live + 2)
    ru.check(trace, outputs, expected, dtype, many_rows=True)
    buckets = sorted({key[0] for key in engine.runner._captured})
    assert engine.runner.graph_replays >= 4 and buckets, buckets
    assert max(buckets) >= live - 1 and len(buckets) >= 2, buckets       # the batch shrank into a smaller bucket
    engine.runner.manager.check_invariants()


def test_many_sequences_through_the_replay_program():
    """``bin/trace_run --max-seqs``: forty live requests through the program itself."""
    raw, page = tiny.CONFIGS["B"]
    folder = model_folder("B")
    rng = random.Random(5)
    lengths = [rng.choice((26, 31, 47, 64, 90, 133)) for _ in range(39)] + [61]
    requests = ru.make_requests(raw["vocab_size"], lengths, seed=40)
    trace = _crowd_trace(requests, 24, seed=2)
    max_tokens = sum((n + 63) // 64 * 64 for n in lengths)
    outputs = ru.run_subprocess(folder, "float32", trace, max_tokens, page_size=page, max_seqs=42)
    ru.compare(trace, outputs, plain_logits(folder, raw, requests, "float32"), "float32")


# --------------------------------------------------------------------------- forty requests through the scheduler

@pytest.mark.parametrize("name", ["A", "C"])
def test_forty_requests_queued_ahead_with_an_end_of_sequence_token(name):
    """float32, greedy: every request's tokens equal the same request generated alone, and the plain
    implementation's for a few.  The end-of-sequence ids are chosen so that they stop a third of the requests or more
    part-way; rounds are queued one ahead, so those requests have a speculative token dropped."""
    from ampere_kv_engine_b200.config.engine_config import EngineConfig
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = tiny.CONFIGS[name]
    folder = model_folder(name)
    rng = random.Random(17)
    prompts = [torch.randint(0, raw["vocab_size"], (rng.choice((1, 3, 8, 21, 40, 77)),),
                             generator=torch.Generator().manual_seed(100 + i)).tolist() for i in range(41)]
    engine = Engine.from_pretrained(folder, config=EngineConfig(
        dtype="float32", page_size=page, max_tokens=41 * 160, max_seqs=48, max_batch_tokens=96))
    assert engine.config.lookahead
    free = engine.generate(prompts, max_new_tokens=30, ignore_eos=True)
    assert all(len(out) == 30 for out in free)
    # end-of-sequence ids taken from the middle of every third request's free run: those requests stop there (or
    # earlier, at another of the ids), the others mostly run to their limit
    eos = tuple(sorted({free[i][8 + i % 12] for i in range(0, len(free), 3)}))
    engine.eos_token_ids = eos
    assert engine.new_scheduler().lookahead
    together = engine.generate(prompts, max_new_tokens=30)

    def cut(out):
        first = min((out.index(t) for t in eos if t in out), default=None)
        return out if first is None else out[:first + 1]

    want = [cut(out) for out in free]
    assert together == want
    stopped = [i for i, out in enumerate(want) if len(out) < 30]
    assert len(stopped) >= 10 and len(stopped) < len(prompts)
    # alone, one request at a time
    for i in stopped[:4] + [j for j in range(len(prompts)) if j not in stopped][:3]:
        assert engine.generate([prompts[i]], max_new_tokens=30)[0] == want[i]
    # against the plain implementation
    w = plain_weights(folder, "float32")
    for i in stopped[:2]:
        assert plain.greedy_generate(w, raw, prompts[i], 30, eos_ids=eos, ignore_eos=False) == want[i]
    assert engine.manager.free_pages() == [g.pool.count for g in engine.manager.groups]
    engine.manager.check_invariants()


# --------------------------------------------------------------------------- the benchmark model itself

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 40960, "tie_word_embeddings": False,
    "hidden_act": "silu", "attention_bias": False,
}


def test_benchmark_model_whole_depth_and_vocabulary():
    """Qwen3-8B's sizes, all 36 layers, all 151,936 logits, seeded random weights that bfloat16 holds exactly.  The
    plain model runs on the GPU in true float32 (no reduced-precision matrix mode).  One 300-token request whole,
    16 tokens decoded one by one (captured graphs), and a step that mixes its next token with a portion of a second
    request: the float32 engine against the plain logits, then the bfloat16 engine against the same."""
    from ampere_kv_engine_b200.config.engine_config import EngineConfig
    from ampere_kv_engine_b200.engine.engine import Engine, set_exact_matmul
    from ampere_kv_engine_b200.models.decoder import DecoderModel
    from ampere_kv_engine_b200.models.registry import config_from_dict
    from ampere_kv_engine_b200.weights.loader import cast_for
    from ampere_kv_engine_b200.weights.random_init import random_tensors
    if torch.cuda.get_device_properties(0).total_memory < 100 * 2 ** 30:
        pytest.skip("needs about 80 GB of device memory")
    set_exact_matmul()
    arch, cfg = config_from_dict(dict(QWEN3_8B))
    spec = arch.build_spec(cfg)
    probe = DecoderModel(spec, dtype=torch.float32, device="cuda")
    specs = probe.param_specs()
    weights = {name: t.bfloat16().float() for name, t in random_tensors(specs, 11, device="cuda").items()}
    vocab = QWEN3_8B["vocab_size"]
    requests = ru.make_requests(vocab, (317, 41), seed=2)
    first, second = requests["r0"], requests["r1"]
    trace = ru.Trace()
    trace.add([("r0", first[:300], 0, [0, 150, 299])])
    for p in range(300, 316):
        trace.add([("r0", first[p:p + 1], p, [0])])
    trace.add([("r0", first[316:317], 316, [0]), ("r1", second[:40], 0, [0, 39])], end=["r0"])
    trace.add([("r1", second[40:41], 40, [0])], end=["r1"])
    expected = {rid: plain.forward_logits(weights, QWEN3_8B, toks).cpu() for rid, toks in requests.items()}
    row_scale = float(expected["r0"].square().mean().sqrt())

    def run(dtype):
        model = DecoderModel(spec, dtype=dtype, device="cuda")
        model.load_tensors({name: cast_for(specs[name], t, dtype) for name, t in weights.items()})
        engine = Engine(model, EngineConfig(dtype=dtype, page_size=16, num_pages=64, max_seqs=4))
        outputs = ru.replay_on(engine, trace)
        assert engine.runner.graph_replays >= 14
        return outputs

    def errors(outputs):
        worst_abs = worst_rms = 0.0
        for step, rows in trace.expect.items():
            got = torch.from_numpy(outputs[step].copy()).view(len(rows), vocab)
            want = torch.stack([expected[rid][pos] for rid, pos in rows])
            worst_abs = max(worst_abs, float((got - want).abs().max()))
            worst_rms = max(worst_rms, float(((got - want).square().mean(dim=1).sqrt()
                                              / want.square().mean(dim=1).sqrt()).max()))
        return worst_abs, worst_rms

    out32 = run(torch.float32)
    abs32, rms32 = errors(out32)
    print(f"float32 engine vs plain, 36 layers x 151,936 logits: worst |diff| {abs32:.3e}, "
          f"worst relative RMS {rms32:.3e} (logit RMS {row_scale:.3f})")
    # Two float32 implementations that differ by the order of their sums: the tiny models' bound (2e-5 at sums of
    # 96 terms, two or three layers) scaled by the square root of the sums' length and of the depth.
    bound32 = ru.TOL["float32"]["atol"] * math.sqrt(QWEN3_8B["hidden_size"] / 96) * math.sqrt(36 / 2)
    assert abs32 <= bound32 * max(1.0, row_scale), (abs32, bound32)
    del out32
    gc.collect()
    torch.cuda.empty_cache()
    out16 = run(torch.bfloat16)
    abs16, rms16 = errors(out16)
    print(f"bfloat16 engine vs plain: worst |diff| {abs16:.3e}, worst relative RMS {rms16:.4f}")
    # bfloat16 rounds every stored activation to 8 bits; the two-layer model of the same sizes is held to a
    # relative RMS error of 0.02 per row, and independent roundings add up with the square root of the depth.
    assert 0.0 < rms16 <= 0.02 * math.sqrt(36 / 2), rms16
    assert rms16 > 10 * rms32                                   # and the float32 path is a float32 path
