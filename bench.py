"""Benchmark of the engine on one B200: decode tokens per second at the Qwen3-8B shape.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Prints ONE JSON line.  A "step" is one decode step of the whole batch through the engine's own step
function (every kernel of the model and the token choice); ``value`` is batch / step time, timed with CUDA
events around K steps.  ``e2e`` is the same quantity through the Python entry point's scheduler loop: every
step copies that step's token ids and index data from pinned host memory to the device and reads the
chosen tokens back.  ``prefill`` is one 2,048-token prompt in one step; ``points`` holds decode at batch 1
and 64; ``roofline`` compares the bytes a decode step must read (every weight once, the live requests'
cache) with the copy bandwidth.  Weights are random (seeded), token ids synthetic (seeded uniform).
Between timed steps nothing is flushed: every step streams the whole model (16 GB at full depth) through
a 126 MB L2, so the inputs are larger than L2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Qwen3-8B shape
QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "max_position_embeddings": 40960, "tie_word_embeddings": False,
    "hidden_act": "silu", "attention_bias": False,
}
# BASELINE.json configs[3] and [4]: the further sizes (`--shape 14b|32b`), each with its own workload
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
SHAPES = {"8b": QWEN3_8B, "14b": QWEN3_14B, "32b": QWEN3_32B}
LONG_CONTEXT = 32768    # 32b: decode at batch 16 with prompts of this many tokens ...
LONG_BATCH = 16
LONG_CHUNK = 2048       # ... prefilled in portions of this many
SERVING_CONTEXT_14B = 16384
CONTEXT = 8192          # the engine's context limit in this run
PROMPT_LEN = 1024       # decode starts from 1,024-token prompts
GEN_LEN = 256
PREFILL_TOKENS = 2048
PAGE_SIZE = 16
SERVING_REQUESTS = 64               # the scheduler load: this many requests ...
SERVING_PROMPT = (128, 4096)        # ... with prompts of uniformly drawn lengths in this range
SERVING_OUTPUT = (128, 512)         # ... and this many generated tokens each
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as handle:
                raw = json.load(handle)
            flat = {}

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)) and k not in flat:
                        flat[k] = float(v)
            walk(raw)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                flat["source"] = "measured"
                return flat
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples: list[list[str]] = []
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        mhz = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        reasons = sorted({name for s in self.samples for name, flag in zip(self.NAMES, s[2:]) if flag == "Active"})
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def model_numbers(cfg: dict, layers: int) -> dict:
    h, nh, nkv, d, i, v = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                           cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = (nh + 2 * nkv) * d * h + h * nh * d + 3 * i * h
    return {"layer_params": per_layer, "head_params": v * h, "layer_norm_params": 2 * h + 2 * d,
            "kv_bytes_per_token": 2 * nkv * d * 2 * layers}


def decode_bytes(cfg, layers, batch, mean_ctx) -> float:
    n = model_numbers(cfg, layers)
    weights = 2.0 * (layers * n["layer_params"] + n["head_params"]) + 4.0 * (layers * n["layer_norm_params"])
    return weights + batch * mean_ctx * n["kv_bytes_per_token"]


def prefill_flops(cfg, layers, tokens) -> dict:
    n = model_numbers(cfg, layers)
    gemm = 2.0 * tokens * layers * n["layer_params"] + 2.0 * n["head_params"]
    attn = 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * layers * tokens * (tokens + 1) / 2
    return {"gemm": gemm, "attention": attn}


def reference_arm(args) -> int:
    """The unmodified reference project (installed under baseline/_ref) on its stock default path.

    Its loader needs the published checkpoint and its extension holds sm_86 code only, but its default generation
    path needs neither: ``ampere_kv.runner.generate_tokens(model, input_ids, cache_kind="contiguous")``
    (ampere_kv/runner.py:301-406; ``--cache contiguous`` is the command line's default, runner.py:667) takes the
    model as an argument and reads weights off it by attribute.  A tree of ``types.SimpleNamespace`` with exactly
    those attributes, holding seeded random bfloat16 tensors of the Qwen3-8B sizes, stands in for the checkpoint.
    The reference without its extension decodes one request at a time, so a "step" of the batch is one token for
    each of the batch's requests in turn.  Nothing of this repository's package is imported here.
    """
    import traceback
    import types
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    cfg = dict(QWEN3_8B)
    cfg["num_hidden_layers"] = args.layers
    steps, warmup, batch = args.steps, max(3, args.warmup), args.batch
    try:
        if not os.path.isdir(os.path.join(ref_root, "ampere_kv")):
            raise RuntimeError("baseline/_ref/ampere_kv is missing (the offline install did not travel)")
        sys.path.insert(0, ref_root)
        sys.dont_write_bytecode = True
        os.environ.setdefault("HF_HUB_OFFLINE", "1")
        import torch
        from ampere_kv import runner as ref           # imports the checkpoint library at module level
        device = torch.device("cuda:0")
        torch.cuda.set_device(device)
        gen = torch.Generator(device=device).manual_seed(0)
        h, nh, nkv, d, inter, vocab = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                                       cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
        ns = types.SimpleNamespace

        def matrix(rows, cols):
            return (torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * 0.02).bfloat16()

        def lin(rows, cols):
            return ns(weight=matrix(rows, cols), bias=None)

        def norm(size):
            w = 1.0 + 0.1 * torch.randn((size,), generator=gen, device=device, dtype=torch.float32)
            return ns(weight=w.bfloat16(), variance_epsilon=cfg["rms_norm_eps"])

        layers = []
        for _ in range(args.layers):
            attn = ns(q_proj=lin(nh * d, h), k_proj=lin(nkv * d, h), v_proj=lin(nkv * d, h), o_proj=lin(h, nh * d),
                      q_norm=norm(d), k_norm=norm(d), head_dim=d, sliding_window=None)
            mlp = ns(gate_proj=lin(inter, h), up_proj=lin(inter, h), down_proj=lin(h, inter))
            layers.append(ns(self_attn=attn, mlp=mlp, input_layernorm=norm(h), post_attention_layernorm=norm(h)))
        exponent = torch.arange(0, d, 2, dtype=torch.int64).float() / d
        model = ns(model=ns(embed_tokens=ns(weight=matrix(vocab, h)), layers=layers, norm=norm(h)),
                   lm_head=lin(vocab, h),
                   config=ns(head_dim=d, num_key_value_heads=nkv, rope_theta=cfg["rope_theta"], hidden_act="silu"),
                   _ampere_inv_freq=(1.0 / (cfg["rope_theta"] ** exponent)).to(device),
                   generation_config=ns(eos_token_id=None))
        host_gen = torch.Generator().manual_seed(1234)
        prompts = [torch.randint(0, vocab, (1, PROMPT_LEN), generator=host_gen).pin_memory() for _ in range(batch)]

        def run(prompt_host, new_tokens, timings=None):
            ids = prompt_host.to(device, non_blocking=True)
            return ref.generate_tokens(model, ids, max_new_tokens=new_tokens, cache_kind="contiguous",
                                       ignore_eos=True, timings=timings)

        def device_ms(prompt_host, new_tokens):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record()
            run(prompt_host, new_tokens)
            stop.record()
            torch.cuda.synchronize()
            return start.elapsed_time(stop)

        run(prompts[0], 4)                       # library handles, kernels loaded
        with ClockSampler() as clocks:
            step_ms = e2e_step_ms = 0.0
            for prompt in prompts:
                # the K timed decode steps of this request: a run of 1 + W + K tokens less a run of 1 + W tokens
                short = min(device_ms(prompt, 1 + warmup) for _ in range(2))
                timings: dict = {}
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                start.record()
                run(prompt, 1 + warmup + steps, timings)
                stop.record()
                torch.cuda.synchronize()
                step_ms += (start.elapsed_time(stop) - short) / steps
                e2e_step_ms += timings["tpot_ms"]        # its own host clock: token ids on the host every step
        clock_summary = clocks.summary()
        # prefill: the time to the first token of a 2,048-token prompt, by the reference's own clock
        long_prompt = torch.randint(0, vocab, (1, PREFILL_TOKENS), generator=host_gen).pin_memory()
        run(long_prompt, 1)
        ttft = []
        for _ in range(3):
            timings = {}
            run(long_prompt, 1, timings)
            ttft.append(timings["ttft_ms"])
        prefill_ms = statistics.median(ttft)
        peaks = load_peaks()
        flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
        line = {
            "impl": "reference",
            "metric": "decode tok/s at batch 8 (Qwen3-8B shape, B200); prefill alongside",
            "value": round(batch / (step_ms / 1000), 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": round(step_ms, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids, seeded random weights)",
            "config": {
                "model": "Qwen3-8B shape", "layers": args.layers, "layers_full": QWEN3_8B["num_hidden_layers"],
                "hidden": h, "heads": nh, "kv_heads": nkv, "head_dim": d, "intermediate": inter, "vocab": vocab,
                "global_batch": batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
                "path": "ampere_kv.runner.generate_tokens, cache_kind=contiguous (its default), SDPA, no extension",
                "batching": "one request at a time (its batched decode needs its sm_86 extension)",
                "timing": "CUDA events: run of 1+W+K tokens less run of 1+W tokens, per request, summed",
                "parallelism": "single GPU", "l2": "inputs larger than L2 (all weights stream every token)",
            },
            "e2e": {"value": round(batch / (e2e_step_ms / 1000), 2), "unit": "tokens/s",
                    "ms_per_step": round(e2e_step_ms, 4), "h2d_bytes_per_step": 8 * batch,
                    "d2h_bytes_per_step": 8 * batch},
            "gpu_launches": 0,
            "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1000), 1), "tokens": PREFILL_TOKENS,
                        "ms": round(prefill_ms, 3),
                        "frac": round(flops["gemm"] / (prefill_ms / 1000) / (peaks["bf16_tflops"] * 1e12), 4)},
            "clocks": clock_summary,
        }
        print(json.dumps(line))
        return 0
    except BaseException as exc:        # the actual error goes on record instead of a guess
        if isinstance(exc, KeyboardInterrupt):
            raise
        last = traceback.format_exception_only(type(exc), exc)[-1].strip()
        where = traceback.extract_tb(exc.__traceback__)[-1]
        print(json.dumps({"impl": "reference", "unavailable":
                          f"{last} (at {os.path.basename(where.filename)}:{where.lineno})"[:400]}))
        return 0


def serving_load(engine, synthetic, num_requests, prompt_range, output_range, seed=7) -> dict:
    """A scheduler load: many requests of mixed lengths, chunked prefill beside decoding, host tokens in and out.
    Two passes; the second is timed (the decode graphs of its batch sizes exist by then).  Throughput by the wall
    clock, and per request the time to its first token and its longest wait between two tokens."""
    import random
    import torch
    rng = random.Random(seed)
    lengths = [(rng.randint(*prompt_range), rng.randint(*output_range)) for _ in range(num_requests)]
    for timed_pass in (False, True):
        scheduler = engine.new_scheduler(record_times=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        requests = [scheduler.submit(f"s{i}", synthetic(n_in), n_out, ignore_eos=True)
                    for i, (n_in, n_out) in enumerate(lengths)]
        while scheduler.has_work():
            scheduler.step()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        assert all(len(r.output_ids) == n_out for r, (_, n_out) in zip(requests, lengths))
    ttft = sorted(r.ttft_ms for r in requests)
    gaps = sorted(r.largest_gap_ms for r in requests if r.largest_gap_ms is not None)
    return {"serving_requests": num_requests,
            "serving_output_tok_s": round(sum(n for _, n in lengths) / wall, 1),
            "serving_total_tok_s": round(sum(a + b for a, b in lengths) / wall, 1),
            "serving_rounds": scheduler.rounds,
            "serving_ttft_ms_median": round(ttft[len(ttft) // 2], 1), "serving_ttft_ms_max": round(ttft[-1], 1),
            "serving_largest_gap_ms_median": round(gaps[len(gaps) // 2], 2),
            "serving_largest_gap_ms_max": round(gaps[-1], 2)}


def insert_point(engine, synthetic, batch, prompt_len=PROMPT_LEN, insert_len=PREFILL_TOKENS) -> dict:
    """``batch`` requests decode; a prompt of ``insert_len`` tokens arrives.  Its time to the first token, the
    longest token-to-token wait of the running requests while it is prefilled, and their usual one."""
    import torch
    scheduler = engine.new_scheduler(record_times=True)
    running = [scheduler.submit(f"i{i}", synthetic(prompt_len), 96, ignore_eos=True) for i in range(batch)]
    while any(len(r.output_ids) < 24 for r in running):
        scheduler.step()
    torch.cuda.synchronize()
    newcomer = scheduler.submit("newcomer", synthetic(insert_len), 4, ignore_eos=True)
    while scheduler.has_work():
        scheduler.step()
    gaps = sorted(b - a for r in running for a, b in zip(r.token_times[8:], r.token_times[9:]))
    return {"insert_prompt_tokens": insert_len, "insert_ttft_ms": round(newcomer.ttft_ms, 2),
            "insert_running_gap_ms_max": round(max(r.largest_gap_ms for r in running), 2),
            "insert_running_gap_ms_median": round(gaps[len(gaps) // 2] * 1000, 3)}


def _shape_setup(args, shape_cfg, *, pool_tokens, max_seqs, max_context):
    import torch
    from ampere_kv_engine_b200.config.engine_config import EngineConfig
    from ampere_kv_engine_b200.engine.engine import Engine
    cfg = dict(shape_cfg)
    cfg["num_hidden_layers"] = args.layers
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    engine = Engine.from_random(cfg, seed=0, device=device, config=EngineConfig(
        dtype="bfloat16", page_size=args.page_size, max_tokens=pool_tokens, max_seqs=max_seqs,
        max_batch_tokens=PREFILL_TOKENS, max_context=max_context))
    gen = torch.Generator().manual_seed(1234)
    vocab = cfg["vocab_size"]
    return cfg, engine, (lambda n: torch.randint(0, vocab, (n,), generator=gen).tolist())


def _shape_config(cfg, args, full_layers, **more) -> dict:
    out = {"layers": args.layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
           "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
           "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "page_size": args.page_size,
           "kv_dtype": "bf16", "parallelism": "single GPU"}
    out.update(more)
    return out


def serving_shape(args) -> int:
    """Qwen3-14B sizes: 64 requests, prompts of 128 to 4,096 tokens, 128 to 512 new tokens each, rounds of at most
    2,048 tokens, 16,384 positions of context.  ``value`` is generated tokens per second of the whole load."""
    pool = SERVING_REQUESTS * (SERVING_PROMPT[1] + SERVING_OUTPUT[1]) // 2 + SERVING_REQUESTS * 64
    cfg, engine, synthetic = _shape_setup(args, QWEN3_14B, pool_tokens=pool, max_seqs=SERVING_REQUESTS + 2,
                                          max_context=SERVING_CONTEXT_14B)
    with ClockSampler() as clocks:
        serving = serving_load(engine, synthetic, SERVING_REQUESTS, SERVING_PROMPT, SERVING_OUTPUT)
    line = {"metric": "generated tok/s of a mixed scheduler load (Qwen3-14B shape, B200)",
            "value": serving["serving_output_tok_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True,
            "dtype": "bf16", "data": "synthetic (seeded uniform token ids, seeded random weights)",
            "config": _shape_config(cfg, args, QWEN3_14B["num_hidden_layers"], model="Qwen3-14B shape",
                                    requests=SERVING_REQUESTS, prompt_tokens="128-4096", new_tokens="128-512",
                                    max_batch_tokens=PREFILL_TOKENS, seq_len=SERVING_CONTEXT_14B),
            "points": serving, "clocks": clocks.summary()}
    print(json.dumps(line))
    return 0


def long_context_shape(args) -> int:
    """Qwen3-32B sizes: 16 requests with 32,768-token prompts, prefilled in portions of 2,048 tokens, then decoded
    together.  At full depth the 16 caches (8.6 GB each) do not fit beside the weights: admission by page budget
    lets as many in as the pool holds and the rest wait; ``value`` is decode tokens per second of the live batch,
    with the bytes it must read over its time as the roofline fraction."""
    import torch
    from ampere_kv_engine_b200.engine.batch import SeqStep
    from ampere_kv_engine_b200.sampling.sampler import SamplingParams
    cfg = dict(QWEN3_32B)
    cfg["num_hidden_layers"] = args.layers
    peaks = load_peaks()
    numbers = model_numbers(cfg, args.layers)
    weight_bytes = 2.0 * (args.layers * numbers["layer_params"] + 2 * numbers["head_params"])
    free_bytes = torch.cuda.mem_get_info(0)[0]
    # every request decodes beside the later ones' prompt portions, so it needs room for those tokens too
    new_tokens = LONG_BATCH * (LONG_CONTEXT // LONG_CHUNK + 1) + args.warmup + args.steps + 8
    per_request = (LONG_CONTEXT + new_tokens + 64) * numbers["kv_bytes_per_token"]
    room = free_bytes - weight_bytes - 12 * 2 ** 30          # activations of a 2,048-token portion, logits, slack
    live = int(max(1, min(LONG_BATCH, room // per_request)))
    cfg, engine, synthetic = _shape_setup(args, QWEN3_32B, pool_tokens=live * (LONG_CONTEXT + new_tokens + 64),
                                          max_seqs=LONG_BATCH + 2, max_context=LONG_CONTEXT + new_tokens)
    runner = engine.runner
    # through the scheduler: all 16 are submitted, the page budget admits `live` of them, the rest wait
    scheduler = engine.new_scheduler(record_times=True)
    requests = [scheduler.submit(f"L{i}", synthetic(LONG_CONTEXT), new_tokens, ignore_eos=True)
                for i in range(LONG_BATCH)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    prefill_rounds = 0
    while scheduler.prefilling or not scheduler.running:
        scheduler.step()
        prefill_rounds += 1
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    admitted = sum(1 for r in requests if r.seq is not None)
    waiting = len(scheduler.waiting)
    for _ in range(args.warmup):
        scheduler.step()
    with ClockSampler() as clocks:
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        t0 = time.perf_counter()
        stats = None
        for _ in range(args.steps):
            _, stats = scheduler.step()
        stop.record()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1000 / args.steps
        ms = start.elapsed_time(stop) / args.steps
    batch = stats.decode_tokens
    assert stats.prefill_tokens == 0 and batch == admitted
    mean_ctx = sum(r.seq.length for r in requests if r.seq is not None) / batch - args.steps / 2
    bytes_step = decode_bytes(cfg, args.layers, batch, mean_ctx)
    achieved = bytes_step / (ms / 1000) / 1e9
    for r in requests:
        scheduler.cancel(r)
    scheduler.step()
    line = {"metric": "decode tok/s at batch 16 with 32,768-token prompts (Qwen3-32B shape, B200)",
            "value": round(batch / (ms / 1000), 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids, seeded random weights)",
            "config": _shape_config(cfg, args, QWEN3_32B["num_hidden_layers"], model="Qwen3-32B shape",
                                    global_batch=LONG_BATCH, live_batch=batch, waiting_for_pages=waiting,
                                    mean_decode_context=round(mean_ctx, 1),
                                    seq_len=LONG_CONTEXT, prefill_chunk=LONG_CHUNK),
            "e2e": {"value": round(batch / (e2e_ms / 1000), 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4)},
            "prefill": {"tokens": admitted * LONG_CONTEXT, "seconds": round(prefill_s, 2), "rounds": prefill_rounds,
                        "value": round(live * LONG_CONTEXT / prefill_s, 1)},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peaks["source"]},
            "clocks": clocks.summary()}
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page (a power of two, 16 or more)")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="8b",
                        help="8b: the headline benchmark; 14b: a mixed scheduler load of 64 requests; 32b: long-context "
                             "decode at batch 16 (each prints its own one line)")
    parser.add_argument("--layers", type=int, default=None,
                        help="run fewer layers of the same sizes (reported in config beside the full count)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--no-points", action="store_true", help="skip the batch-1 and batch-64 decode points")
    args = parser.parse_args()

    if args.layers is None:
        args.layers = SHAPES[args.shape]["num_hidden_layers"]
    if args.impl == "reference":
        if args.shape != "8b":
            print(json.dumps({"impl": "reference", "unavailable": "the reference arm runs the 8b shape only"}))
            return 0
        if args.gpus != 1:
            print(json.dumps({"impl": "reference", "unavailable": "the reference runs on one GPU; --gpus must be 1"}))
            return 0
        return reference_arm(args)
    if args.gpus != 1:
        print(json.dumps({"error": "this engine runs on one GPU; --gpus must be 1", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.shape == "14b":
        return serving_shape(args)
    if args.shape == "32b":
        return long_context_shape(args)

    import torch
    from ampere_kv_engine_b200.engine.batch import SeqStep
    from ampere_kv_engine_b200.engine.engine import Engine
    from ampere_kv_engine_b200.kernels import ops
    from ampere_kv_engine_b200.sampling.sampler import SamplingParams

    cfg = dict(QWEN3_8B)
    cfg["num_hidden_layers"] = args.layers
    peaks = load_peaks()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    max_batch = 64 if not args.no_points else args.batch
    pool_tokens = max(max_batch * (PROMPT_LEN + GEN_LEN + 64),
                      max(args.batch * (CONTEXT + 64), SERVING_REQUESTS * (SERVING_PROMPT[1] + SERVING_OUTPUT[1]) // 2
                          + SERVING_REQUESTS * 64) if not args.no_points else 0,
                      PREFILL_TOKENS + 64)
    from ampere_kv_engine_b200.config.engine_config import EngineConfig
    engine = Engine.from_random(cfg, seed=0, device=device, config=EngineConfig(
        dtype="bfloat16", page_size=args.page_size, max_tokens=pool_tokens, max_seqs=max_batch + 2,
        max_batch_tokens=PREFILL_TOKENS, max_context=CONTEXT))
    runner = engine.runner
    gen = torch.Generator().manual_seed(1234)
    vocab = cfg["vocab_size"]

    def synthetic(n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    def timed(fn, steps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps

    def decode_point(batch, steps, warmup, prompt_len=PROMPT_LEN):
        """ms per decode step of ``batch`` requests that each hold a ``prompt_len``-token prompt."""
        seqs = [runner.open(f"d{batch}-{prompt_len}-{i}") for i in range(batch)]
        if prompt_len <= PREFILL_TOKENS:
            per_step = max(1, PREFILL_TOKENS // prompt_len)
            for i in range(0, batch, per_step):
                runner.step([SeqStep(s, synthetic(prompt_len), []) for s in seqs[i:i + per_step]])
        else:
            for s in seqs:       # long prompts go in portions of the prefill budget
                for start in range(0, prompt_len, PREFILL_TOKENS):
                    runner.step([SeqStep(s, synthetic(min(PREFILL_TOKENS, prompt_len - start)), [])])
        greedy = [SamplingParams()] * batch
        zeros = [0] * batch

        def one():
            logits = runner.step([SeqStep(s, [t], [0]) for s, t in zip(seqs, synthetic(batch))])
            engine.sampler.sample(logits, greedy, zeros)

        for _ in range(warmup):
            one()
        ctx_start = seqs[0].length
        ops.launch_count = 0
        ms = timed(one, steps)
        launches = ops.launch_count
        mean_ctx = ctx_start + (steps + 1) / 2
        runner.raise_on_status()
        for s in seqs:
            runner.close(s)
        return ms, mean_ctx, launches

    with ClockSampler() as clocks:
        ms, mean_ctx, launches = decode_point(args.batch, args.steps, args.warmup)
    clock_summary = clocks.summary()
    value = args.batch / (ms / 1000)
    bytes_step = decode_bytes(cfg, args.layers, args.batch, mean_ctx)
    achieved = bytes_step / (ms / 1000) / 1e9

    # end to end: the scheduler loop of the Python entry point, host tokens in and out every step
    scheduler = engine.new_scheduler()
    slack = args.batch * PROMPT_LEN // PREFILL_TOKENS + 4     # early requests decode while later ones prefill
    requests = [scheduler.submit(f"e{i}", synthetic(PROMPT_LEN), args.warmup + args.steps + slack, ignore_eos=True)
                for i in range(args.batch)]
    while any(not r.output_ids for r in requests):
        scheduler.step()
    for _ in range(args.warmup):
        scheduler.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    stats = None
    for _ in range(args.steps):
        _, stats = scheduler.step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1000 / args.steps
    assert stats.decode_tokens == args.batch and stats.prefill_tokens == 0
    for r in requests:
        scheduler.cancel(r)
    scheduler.step()
    h2d = runner.last_h2d_bytes + 8 * args.batch      # the step's index buffer + temperatures and uniforms
    e2e = {"value": round(args.batch / (e2e_ms / 1000), 2), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * (args.batch + 1)}

    # prefill of 2,048 tokens in one step
    def prefill_once():
        seq = runner.open("prefill")
        logits = runner.step([SeqStep(seq, prompt, [PREFILL_TOKENS - 1])])
        engine.sampler.sample(logits, [SamplingParams()], [0])
        runner.close(seq)

    prompt = synthetic(PREFILL_TOKENS)
    for _ in range(3):
        prefill_once()
    prefill_ms = timed(prefill_once, 5)
    flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1000), 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3),
               "frac": round(flops["gemm"] / (prefill_ms / 1000) / (peaks["bf16_tflops"] * 1e12), 4),
               "frac_of": "matrix-product FLOPs / burst bf16 peak", "gemm_tflop": round(flops["gemm"] / 1e12, 3),
               "attention_tflop": round(flops["attention"] / 1e12, 3),
               "frac_with_attention": round((flops["gemm"] + flops["attention"]) / (prefill_ms / 1000)
                                            / (peaks["bf16_tflops"] * 1e12), 4)}

    points = {}
    if not args.no_points:
        for b in (1, 64):
            p_ms, _, _ = decode_point(b, max(8, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(b / (p_ms / 1000), 2)
        # the same batch at the end of the configuration's 8,192-token context, with its own roofline fraction
        long_steps = max(8, args.steps // 2)
        p_ms, long_ctx, _ = decode_point(args.batch, long_steps, args.warmup, CONTEXT - GEN_LEN)
        points[f"decode_b{args.batch}_ctx{CONTEXT}"] = round(args.batch / (p_ms / 1000), 2)
        points[f"decode_b{args.batch}_ctx{CONTEXT}_hbm_frac"] = round(
            decode_bytes(cfg, args.layers, args.batch, long_ctx) / (p_ms / 1000) / 1e9 / peaks["hbm_gbs"], 4)
        # a scheduler load: many requests of mixed lengths, chunked prefill beside decoding, host tokens in and out
        # (second pass timed: the decode graphs of its batch sizes exist by then); tokens per second of wall clock
        serving = serving_load(engine, synthetic, SERVING_REQUESTS, SERVING_PROMPT, SERVING_OUTPUT)
        points.update(serving)
        # a prompt arrives while the batch decodes: what the newcomer waits for its first token and what the
        # running requests feel meanwhile (the figures of the reference's scheduler benchmark,
        # ampere_kv/bench_scheduler.py:115-125, 242-271)
        points.update(insert_point(engine, synthetic, args.batch))

    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, B200); prefill and batch 1/64 alongside",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded uniform token ids, seeded random weights)",
        "config": {
            "model": "Qwen3-8B shape", "layers": args.layers, "layers_full": QWEN3_8B["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": vocab,
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN, "gen_len": GEN_LEN,
            "mean_decode_context": round(mean_ctx, 1), "page_size": args.page_size, "kv_dtype": "bf16",
            "parallelism": "single GPU", "l2": "inputs larger than L2 (all weights stream every step)",
        },
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "peaks": peaks["source"]},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
