"""Command line and single-request entry point, in the manner of the reference's ``ampere_kv.runner``.

    python -m ampere_kv_engine_b200.runner --model DIR --mode generate --cache paged

The reference's options keep their names and meanings where they still have one
(ampere_kv/runner.py:661-672): ``--mode`` (``check``: run the request through the float32 path as
well and compare every step, the stand-in for the reference's comparison with the checkpoint
library's own forward; ``generate``; ``benchmark``: timed repeats after one warm-up),
``--repeats``, ``--cache`` (only ``paged`` exists here), ``--kv-dtype`` (``bf16`` or ``fp32``;
the reference's ``int8`` cache is outside this engine), ``--decode-kernel`` (the reference
picks between its two decode kernels; here ``auto`` is the only choice).  The reference reads a
line of text and a tokenizer turns it into ids (runner.py:687, :22-28); this engine takes token
ids: from ``--prompt-ids`` (a JSON file or a comma-separated list), ``--prompt-len`` (that many
seeded uniform ids) or, like the reference, from one line of standard input.  Instead of a
model folder, ``--random-config FILE --random-seed S`` builds the model of a config.json with
seeded random weights (the reference has no such mode: it runs one published checkpoint).

``generate_tokens`` is the single-request Python entry point with the reference's name and
keyword meanings (runner.py:301-406).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

MAX_NEW_TOKENS = 32      # the reference's default limit (ampere_kv/runner.py:17)
PAGED_BLOCK_SIZE = 16    # the reference's page size (ampere_kv/runner.py:19)


def generate_tokens(engine, input_ids, *, max_new_tokens: int = MAX_NEW_TOKENS, ignore_eos: bool = False,
                    temperature: float = 0.0, seed: int = 0, timings: dict | None = None) -> list[int]:
    """New token ids for one request.  ``timings`` (a dict) receives ttft_ms, tpot_ms, total_ms and
    output_tokens_per_s measured on the host clock, as the reference's does (runner.py:385-405)."""
    import torch
    from .sampling.sampler import SamplingParams

    ids = input_ids.reshape(-1).tolist() if hasattr(input_ids, "reshape") else list(input_ids)
    scheduler = engine.new_scheduler()
    if timings is not None:
        torch.cuda.synchronize(engine.device)
    started = time.perf_counter()
    request = scheduler.submit("single", ids, max_new_tokens, sampling=SamplingParams(temperature, seed, 0),
                               ignore_eos=ignore_eos)
    first_ready = None
    while scheduler.has_work():
        scheduler.step()
        if first_ready is None and request.output_ids:
            first_ready = time.perf_counter()
    done = time.perf_counter()
    if timings is not None:
        n = len(request.output_ids)
        timings.update(ttft_ms=(first_ready - started) * 1000,
                       tpot_ms=(done - first_ready) * 1000 / (n - 1) if n > 1 else None,
                       total_ms=(done - started) * 1000, output_tokens_per_s=n / (done - started))
    return list(request.output_ids)


def _read_prompt(arg: str | None) -> list[int]:
    if arg is None:
        text = input("token ids (separated by spaces or commas): ")
    elif os.path.isfile(arg):
        with open(arg, "r", encoding="utf-8") as handle:
            text = handle.read()
    else:
        text = arg
    text = text.strip()
    if not text:
        raise ValueError("the prompt must not be empty")
    if text.startswith("["):
        return [int(t) for t in json.loads(text)]
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description="Qwen3 generation on one B200: generate, check against the float32 "
                                                 "path, or time repeats")
    parser.add_argument("--model", default=None, help="folder with config.json and model.safetensors")
    parser.add_argument("--random-config", default=None,
                        help="a config.json to build with seeded random weights instead of --model")
    parser.add_argument("--random-seed", type=int, default=0, help="seed of the random weights")
    parser.add_argument("--mode", choices=("check", "generate", "benchmark"), default="check",
                        help="check: compare every step with the float32 path; generate; benchmark: timed repeats")
    parser.add_argument("--repeats", type=int, default=3, help="timed runs of benchmark mode (one warm-up before)")
    parser.add_argument("--cache", choices=("paged",), default="paged", help="only the paged cache exists")
    parser.add_argument("--kv-dtype", choices=("bf16", "fp32"), default=None,
                        help="cache dtype; follows --dtype (the cache is read as it is stored)")
    parser.add_argument("--decode-kernel", choices=("auto",), default="auto", help="attention kernel choice")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--prompt-ids", default=None, help="JSON file, or comma-separated token ids")
    parser.add_argument("--prompt-len", type=int, default=None,
                        help="use this many seeded uniform token ids as the prompt (seed: --seed)")
    parser.add_argument("--max-new-tokens", type=int, default=MAX_NEW_TOKENS)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--seed", type=int, default=0, help="sampling seed")
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--page-size", type=int, default=PAGED_BLOCK_SIZE)
    parser.add_argument("--max-batch-tokens", type=int, default=2048)
    parser.add_argument("--max-context", type=int, default=None,
                        help="longest prompt + new tokens accepted (default: the model's max_position_embeddings)")
    parser.add_argument("--num-pages", type=int, default=None,
                        help="pages of the cache pool (default: enough for the prompt and the new tokens)")
    args = parser.parse_args(argv)
    if args.repeats < 1:
        parser.error("--repeats must be positive")
    if (args.model is None) == (args.random_config is None):
        parser.error("give --model DIR or --random-config FILE")
    if args.prompt_len is not None and (args.prompt_ids is not None or args.prompt_len < 1):
        parser.error("--prompt-len is a positive count and goes without --prompt-ids")
    from .config.engine_config import EngineConfig, EngineConfigError
    try:
        base_options = EngineConfig(dtype=args.dtype, kv_dtype=args.kv_dtype, page_size=args.page_size, max_seqs=4,
                                    max_batch_tokens=args.max_batch_tokens, num_pages=args.num_pages,
                                    max_context=args.max_context)
    except EngineConfigError as exc:
        parser.error(str(exc))
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("generation needs a CUDA device")
    from .engine.engine import Engine

    if args.random_config is not None:
        with open(args.random_config, "r", encoding="utf-8") as handle:
            raw_config = json.load(handle)

        def build(dtype, **options):
            return Engine.from_random(raw_config, args.random_seed, config=base_options.replace(
                dtype=dtype, kv_dtype=None, **options))
        vocab = int(raw_config["vocab_size"])
    else:
        from .models.registry import load_config

        def build(dtype, **options):
            return Engine.from_pretrained(args.model, config=base_options.replace(dtype=dtype, kv_dtype=None, **options))
        vocab = int(load_config(args.model)[1].vocab_size)
    if args.prompt_len is not None:
        generator = torch.Generator().manual_seed(args.seed)
        prompt = torch.randint(0, vocab, (args.prompt_len,), generator=generator).tolist()
    else:
        prompt = _read_prompt(args.prompt_ids)
    tokens = len(prompt) + args.max_new_tokens
    options = dict(max_tokens=tokens + 64)
    engine = build(args.dtype, **options)
    print(f"model={args.model or args.random_config} mode={args.mode} cache={args.cache} dtype={args.dtype} prompt_tokens={len(prompt)}")
    if args.mode == "benchmark":
        generate_tokens(engine, prompt, max_new_tokens=args.max_new_tokens, ignore_eos=True)
        totals, ttfts, tpots = [], [], []
        for _ in range(args.repeats):
            t: dict = {}
            ids = generate_tokens(engine, prompt, max_new_tokens=args.max_new_tokens, ignore_eos=True, timings=t)
            totals.append(t["total_ms"]); ttfts.append(t["ttft_ms"]); tpots.append(t["tpot_ms"] or 0.0)
        print(f"generated_token_ids = {json.dumps(ids)}")
        print(f"ttft_ms={statistics.median(ttfts):.3f} tpot_ms={statistics.median(tpots):.3f} "
              f"total_ms={statistics.median(totals):.3f} "
              f"output_tokens_per_s={len(ids) / (statistics.median(totals) / 1000):.2f}")
        return 0
    ids = generate_tokens(engine, prompt, max_new_tokens=args.max_new_tokens, ignore_eos=args.ignore_eos,
                          temperature=args.temperature, seed=args.seed)
    print(f"generated_token_ids = {json.dumps(ids)}")
    eos = set(engine.eos_token_ids)
    reason = "EOS" if ids and ids[-1] in eos and not args.ignore_eos else "token limit"
    print(f"stop_reason={reason} generated={len(ids)} decode_steps={len(ids) - 1}")
    if args.mode == "check":
        if args.dtype == "float32":
            print("check: the run itself is the float32 path; nothing to compare")
            return 0
        reference = build("float32", **options)
        from .engine.batch import SeqStep
        seq_a, seq_b = engine.runner.open("check"), reference.runner.open("check")
        feed, worst, agree = list(prompt), 0.0, 0
        for step, token in enumerate(ids):
            la = engine.runner.step([SeqStep(seq_a, feed, [len(feed) - 1])])[0]
            lb = reference.runner.step([SeqStep(seq_b, feed, [len(feed) - 1])])[0]
            worst = max(worst, float((la - lb).abs().max()))
            agree += int(la.argmax() == lb.argmax())
            feed = [token]
        engine.runner.close(seq_a)
        reference.runner.close(seq_b)
        print(f"check: {agree}/{len(ids)} steps pick the same token as the float32 path; "
              f"largest logit difference {worst:.4e}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
