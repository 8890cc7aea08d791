"""bin/trace_run on the GPU, as a user runs it (a subprocess fed JSON lines), in float32 and in bfloat16,
for both tiny configurations and a small one with the benchmark model's head shape: each request alone and whole; most of it in one step and the last 32 tokens
one by one; in portions of changing size down to two tokens; and mixed, up to four live requests with so
few pages that they are used again.  Every written row is compared with the plain implementation."""

import functools

import pytest

import replay_util as ru
import tiny
from models_util import model_folder, plain_logits

pytestmark = pytest.mark.gpu

LENGTHS = {"A": (5, 17, 33, 130), "B": (1, 31, 64, 130), "C": (3, 40, 64, 130)}
MODES = ("whole", "last32", "portions", "mixed")
MAX_TOKENS = 64 * 6


@functools.lru_cache(maxsize=None)
def _run(name: str, dtype: str):
    raw, page = tiny.CONFIGS[name]
    folder = model_folder(name)
    requests = ru.make_requests(raw["vocab_size"], LENGTHS[name] + (70, 45), seed=11)
    plain = plain_logits(folder, raw, requests, dtype)
    combined = ru.Trace()
    spans, expected = {}, {}
    for mode in MODES:
        sub = {"whole": ru.trace_whole, "last32": ru.trace_last_decoded, "portions": ru.trace_portions,
               "mixed": lambda r: ru.trace_mixed(r, MAX_TOKENS, seed=5)}[mode](requests)
        spans[mode] = combined.extend(sub, mode + ":")
        expected.update({f"{mode}:{rid}": logits for rid, logits in plain.items()})
    outputs = ru.run_subprocess(folder, dtype, combined, MAX_TOKENS, page_size=page)
    return combined, spans, outputs, expected


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("mode", MODES)
def test_replay_matches_plain(name, dtype, mode):
    combined, spans, outputs, expected = _run(name, dtype)
    first, last = spans[mode]
    part = ru.Trace()
    part.expect = {s: rows for s, rows in combined.expect.items() if first <= s < last}
    assert part.expect
    ru.compare(part, outputs, expected, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_default_page_size_long_decode_and_first_tokens(dtype):
    """With the replay program's own default page size: a sequence fed one token at a time from its very
    first token (the first tokens of a sequence), on through 200 positions (long decoding)."""
    raw, _ = tiny.CONFIGS["A"]
    folder = model_folder("A")
    requests = ru.make_requests(raw["vocab_size"], (200,), seed=23)
    trace = ru.trace_last_decoded(requests, last=200)
    outputs = ru.run_subprocess(folder, dtype, trace, 256)
    ru.compare(trace, outputs, plain_logits(folder, raw, requests, dtype), dtype)
