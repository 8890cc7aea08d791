"""Builds replay traces (whole / last tokens one by one / changing portions / mixed with page
reuse), runs them through the engine's trace replay and compares every written logit row with
the plain implementation."""

from __future__ import annotations

import io
import json
import os
import random
import subprocess
import sys
import tempfile

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# float32: the two implementations differ by summation order only
TOL = {"float32": dict(atol=2e-5, rtol=1e-4), "bfloat16": dict(atol=2e-2, rtol=2e-2)}


def make_requests(vocab: int, lengths, seed: int) -> dict[str, list[int]]:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


class Trace:
    def __init__(self):
        self.steps: list[dict] = []
        self.expect: dict[int, list[tuple[str, int]]] = {}   # step -> [(request, position)]

    def add(self, entries: list[tuple[str, list[int], int, list[int]]], end=()):
        """entries: (request id, tokens, position of the first token, wanted places)."""
        step = len(self.steps)
        self.steps.append({"step": step,
                           "entries": [{"id": rid, "tokens": toks, "want": want} for rid, toks, _, want in entries],
                           "end": list(end)})
        rows = [(rid, start + w) for rid, _, start, want in entries for w in want]
        if rows:
            self.expect[step] = rows

    def extend(self, other: "Trace", prefix: str) -> tuple[int, int]:
        """Append another trace with its request ids prefixed; returns the [first, last) steps it occupies."""
        first = len(self.steps)
        for s in other.steps:
            step = len(self.steps)
            self.steps.append({"step": step,
                               "entries": [dict(e, id=prefix + e["id"]) for e in s["entries"]],
                               "end": [prefix + r for r in s["end"]]})
            if s["step"] in other.expect:
                self.expect[step] = [(prefix + rid, pos) for rid, pos in other.expect[s["step"]]]
        return first, len(self.steps)

    def lines(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def trace_whole(requests) -> Trace:
    t = Trace()
    for rid, toks in requests.items():
        t.add([(rid, toks, 0, list(range(len(toks))))], end=[rid])
    return t


def trace_last_decoded(requests, last: int = 32) -> Trace:
    t = Trace()
    for rid, toks in requests.items():
        head = max(1, len(toks) - last)
        t.add([(rid, toks[:head], 0, list(range(head)))])
        for p in range(head, len(toks)):
            t.add([(rid, toks[p:p + 1], p, [0])], end=[rid] if p == len(toks) - 1 else [])
        if head == len(toks):
            t.add([], end=[rid])
    return t


def trace_portions(requests, sizes=(24, 7, 2, 13, 2, 5, 2, 31, 3, 2, 64)) -> Trace:
    t = Trace()
    for rid, toks in requests.items():
        p, k = 0, 0
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            if len(toks) - p - n == 1:      # never leave a lone token for a "portion" step: portions go down to two
                n += 1
            t.add([(rid, toks[p:p + n], p, list(range(n)))], end=[rid] if p + n == len(toks) else [])
            p += n
            k += 1
    return t


def trace_mixed(requests, max_tokens: int, seed: int, max_live: int = 4, decode_tail: int = 6) -> Trace:
    """Up to ``max_live`` requests at a time: prompt portions of some beside single tokens of others; a request
    that is done is ended and the next one starts in pages that were just given back.  The sum over live
    requests of their lengths rounded up to 64 never exceeds ``max_tokens``."""
    rng = random.Random(seed)
    t = Trace()
    pending = list(requests.items())
    live: dict[str, int] = {}     # request -> tokens fed so far
    rounded = lambda n: (n + 63) // 64 * 64
    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending[0]
            if sum(rounded(len(requests[r])) for r in live) + rounded(len(toks)) > max_tokens:
                break
            pending.pop(0)
            live[rid] = 0
        assert live, "max_tokens is too small for the next request"
        chosen = [r for r in live if rng.random() < 0.75] or [rng.choice(list(live))]
        entries, ended = [], []
        for rid in chosen:
            toks, p = requests[rid], live[rid]
            remaining = len(toks) - p
            if remaining <= decode_tail:
                n = 1                                   # the tail goes one token at a time (decoding)
            else:
                n = min(rng.choice((2, 3, 5, 8, 16, 24, 40)), remaining - decode_tail)
                if n == 1:
                    n = 2 if remaining - decode_tail >= 2 else 1
            entries.append((rid, toks[p:p + n], p, list(range(n))))
            live[rid] = p + n
            if live[rid] == len(toks):
                ended.append(rid)
        t.add(entries, end=ended)
        for rid in ended:
            del live[rid]
    return t


def run_subprocess(model_dir: str, dtype: str, trace: Trace, max_tokens: int, page_size: int | None = None,
                   timeout: int = 900, max_seqs: int | None = None) -> dict[int, np.ndarray]:
    out = tempfile.mkdtemp(prefix="replay_out_")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out, "--max-tokens", str(max_tokens)]
    if page_size is not None:
        cmd += ["--page-size", str(page_size)]
    if max_seqs is not None:
        cmd += ["--max-seqs", str(max_seqs)]
    proc = subprocess.run(cmd, input=trace.lines(), text=True, capture_output=True, timeout=timeout)
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert [int(d.split()[1]) for d in done] == list(range(len(trace.steps))), "a 'done <step>' line is missing"
    return read_outputs(out, trace)


def run_inprocess(model_dir: str, dtype: str, trace: Trace, max_tokens: int, page_size: int | None = None
                  ) -> dict[int, np.ndarray]:
    from ampere_kv_engine_b200 import replay
    out = tempfile.mkdtemp(prefix="replay_out_")
    argv = ["--model", model_dir, "--dtype", dtype, "--out", out, "--max-tokens", str(max_tokens), "--device", "cpu"]
    if page_size is not None:
        argv += ["--page-size", str(page_size)]
    sink = io.StringIO()
    assert replay.main(argv, stdin=io.StringIO(trace.lines()), stdout=sink) == 0
    assert len(sink.getvalue().splitlines()) == len(trace.steps)
    return read_outputs(out, trace)


def run_on_device(model_dir: str, dtype: str, trace: Trace, max_tokens: int, page_size: int = 16, max_seqs: int = 8,
                  cuda_graphs: bool = True):
    """The replay program's own loop (``Replayer``) in this process on the GPU, so that a test can also look at
    the runner afterwards (captured graphs, replays, the page pool).  Returns (outputs, engine)."""
    from ampere_kv_engine_b200.config.engine_config import EngineConfig
    from ampere_kv_engine_b200.engine.engine import Engine
    from ampere_kv_engine_b200.replay import Replayer, pool_pages
    engine = Engine.from_pretrained(model_dir, device="cuda", config=EngineConfig(
        dtype=dtype, page_size=page_size, num_pages=pool_pages(max_tokens, page_size), max_seqs=max_seqs,
        cuda_graphs=cuda_graphs))
    return replay_on(engine, trace), engine


def replay_on(engine, trace: Trace) -> dict[int, np.ndarray]:
    from ampere_kv_engine_b200.replay import Replayer
    replayer = Replayer(engine)
    outputs = {}
    for record in trace.steps:
        logits = replayer.step(record)
        assert (logits is not None) == (record["step"] in trace.expect)
        if logits is not None:
            outputs[record["step"]] = logits.cpu().numpy().reshape(-1)
        engine.runner.raise_on_status()
    assert not replayer.live, "the trace left requests open"
    return outputs


def read_outputs(out_dir: str, trace: Trace) -> dict[int, np.ndarray]:
    result = {}
    for step in trace.expect:
        path = os.path.join(out_dir, f"{step}.f32")
        assert os.path.isfile(path), f"step {step} wanted logits but {path} was not written"
        result[step] = np.fromfile(path, dtype="<f4")
    extra = [f for f in os.listdir(out_dir) if f.endswith(".f32") and int(f[:-4]) not in trace.expect]
    assert not extra, f"logit files for steps that wanted nothing: {extra}"
    return result


def compare(trace: Trace, outputs: dict[int, np.ndarray], plain_logits: dict[str, torch.Tensor], dtype: str) -> float:
    """Assert every written row equals the plain implementation's; returns the largest absolute difference."""
    tol = TOL[dtype]
    worst = 0.0
    for step, rows in trace.expect.items():
        vocab = next(iter(plain_logits.values())).shape[1]
        got = torch.from_numpy(outputs[step].copy()).view(-1, vocab)
        assert got.shape[0] == len(rows), f"step {step}: {got.shape[0]} rows written, {len(rows)} wanted"
        want = torch.stack([plain_logits[rid][pos] for rid, pos in rows])
        diff = (got - want).abs()
        bound = tol["atol"] + tol["rtol"] * want.abs()
        if not bool((diff <= bound).all()):
            bad = int((diff - bound).max(dim=1).values.argmax())
            rid, pos = rows[bad]
            raise AssertionError(f"step {step}: request {rid} position {pos} differs from the plain implementation "
                                 f"by {float(diff[bad].max()):.3e} (first wrong row of the step: "
                                 f"{[r for r, ok in zip(rows, (diff <= bound).all(dim=1).tolist()) if not ok][0]})")
        worst = max(worst, float(diff.max()))
    return worst


def compare_rows_to_scale(trace: Trace, outputs: dict[int, np.ndarray], plain_logits: dict[str, torch.Tensor],
                          rms_bound: float = 0.02, peak_bound: float = 0.1) -> tuple[float, float]:
    """bfloat16 rows against the plain implementation, measured against each row's own scale (its root mean
    square): the row's relative RMS error and its worst element.  The bounds are the ones the two-layer model of
    the benchmark's sizes is held to.  Used where a test looks at hundreds of rows of thousands of logits: the
    largest of that many rounding errors sits at the edge of a fixed absolute bound whatever the kernels do, while
    a row that is wrong as a whole (a wrong page, a wrong split, a wrong position) fails either measure by far."""
    worst_rms = worst_peak = 0.0
    for step, rows in trace.expect.items():
        vocab = next(iter(plain_logits.values())).shape[1]
        got = torch.from_numpy(outputs[step].copy()).view(-1, vocab)
        assert got.shape[0] == len(rows), f"step {step}: {got.shape[0]} rows written, {len(rows)} wanted"
        want = torch.stack([plain_logits[rid][pos] for rid, pos in rows])
        scale = want.square().mean(dim=1).sqrt()
        rms = (got - want).square().mean(dim=1).sqrt() / scale
        peak = (got - want).abs().max(dim=1).values / scale
        bad = ((rms > rms_bound) | (peak > peak_bound) | ~torch.isfinite(rms)).nonzero().flatten().tolist()
        if bad:
            rid, pos = rows[bad[0]]
            raise AssertionError(f"step {step}: request {rid} position {pos} differs from the plain implementation: "
                                 f"relative RMS error {float(rms[bad[0]]):.4f} (bound {rms_bound}), worst element "
                                 f"{float(peak[bad[0]]):.4f} of the row's scale (bound {peak_bound})")
        worst_rms, worst_peak = max(worst_rms, float(rms.max())), max(worst_peak, float(peak.max()))
    return worst_rms, worst_peak


def check(trace: Trace, outputs, plain_logits, dtype: str, many_rows: bool = False):
    """float32: element by element.  bfloat16: element by element, or against each row's scale where the test
    looks at very many rows (see :func:`compare_rows_to_scale`)."""
    if dtype == "bfloat16" and many_rows:
        return compare_rows_to_scale(trace, outputs, plain_logits)
    return compare(trace, outputs, plain_logits, dtype)
