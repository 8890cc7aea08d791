"""Trace replay: feed given token ids through a model step by step and write the logits.

It samples nothing and owns no forward pass, cache or loader: it builds the same model,
:class:`~ampere_kv_engine_b200.engine.step.ModelRunner` (step function, cache manager,
kernels) that generation uses and calls its step function directly.  The reference's nearest
relatives are its checks that feed a prompt whole versus in chunks, and a mixed batch versus
separate ones (ampere_kv/check_chunked.py:69-111, ampere_kv/check_mixed.py:58-117).

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry continues its request where it stopped; ``want`` names places among the entry's
tokens whose logits are written (in entry order, then ``want`` order) to ``<out>/<step>.f32``
as little-endian float32 [wanted, vocab].  Requests named in ``end`` give back what they hold
after the step.  After every step a line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch


class Replayer:
    """Feeds trace steps to an engine's own step function and hands back the logits.  It owns nothing but the map
    from request ids to their cache holds."""

    def __init__(self, engine):
        self.engine = engine
        self.runner = engine.runner
        self.live: dict[str, object] = {}

    def step(self, record: dict):
        """Run one trace step; float32 logits [wanted, vocab] on the device, or None when nothing was wanted."""
        from .engine.batch import SeqStep
        entries = []
        for item in record.get("entries", []):
            rid = str(item["id"])
            if rid not in self.live:
                self.live[rid] = self.runner.open(rid)
            entries.append(SeqStep(self.live[rid], [int(t) for t in item["tokens"]],
                                   [int(w) for w in item.get("want", [])]))
        logits = None
        if entries:
            logits = self.runner.step(entries)
            if logits is not None:
                logits = logits.to(torch.float32)
        for rid in record.get("end", []):
            rid = str(rid)
            if rid in self.live:
                self.runner.close(self.live.pop(rid))
        return logits


def pool_pages(max_tokens: int, page_size: int) -> int:
    """Pages for ``max_tokens`` tokens rounded up to a multiple of 64 (or of the page size, if that is larger)."""
    round_to = max(64, page_size)
    return (max_tokens + round_to - 1) // round_to * round_to // page_size


def main(argv=None, stdin=None, stdout=None) -> int:
    stdin = sys.stdin if stdin is None else stdin
    stdout = sys.stdout if stdout is None else stdout
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16",
                        help="bfloat16: the kernels and precisions of serving; float32: everything in true 32-bit")
    parser.add_argument("--out", required=True, help="folder the <step>.f32 files are written to")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    parser.add_argument("--page-size", type=int, default=16, help="tokens per cache page (default 16)")
    parser.add_argument("--max-seqs", type=int, default=8,
                        help="most requests live at a time (default 8; the trace format promises four)")
    parser.add_argument("--no-graphs", action="store_true",
                        help="run decode-only steps as they come instead of replaying them as CUDA graphs")
    parser.add_argument("--device", default="cuda")
    args = parser.parse_args(argv)
    if args.max_tokens <= 0 or args.max_seqs <= 0:
        parser.error("--max-tokens and --max-seqs must be positive")
    if 64 % args.page_size and args.page_size % 64:
        parser.error("--page-size must divide 64 or be a multiple of it")

    from .config.engine_config import EngineConfig
    from .engine.engine import Engine

    os.makedirs(args.out, exist_ok=True)
    engine = Engine.from_pretrained(args.model, device=args.device, config=EngineConfig(
        dtype=args.dtype, page_size=args.page_size, num_pages=pool_pages(args.max_tokens, args.page_size),
        max_seqs=args.max_seqs, cuda_graphs=not args.no_graphs))
    replayer = Replayer(engine)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        logits = replayer.step(record)
        if logits is not None:
            host = logits.cpu().numpy().astype("<f4", copy=False)
            with open(os.path.join(args.out, f"{step}.f32"), "wb") as handle:
                handle.write(np.ascontiguousarray(host).tobytes())
        engine.runner.raise_on_status()
        print(f"done {step}", file=stdout, flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
