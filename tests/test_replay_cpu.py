"""The engine's host side (batch layout, cache manager, step function, replay program) driven on the
CPU through a stand-in for the kernels, against the plain implementation, in all four ways of cutting."""

import pytest

import replay_util as ru
import tiny
from models_util import model_folder, plain_logits

LENGTHS = {"A": (5, 17, 33, 130), "B": (1, 31, 64, 130)}


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("mode", ["whole", "last32", "portions", "mixed"])
def test_replay_matches_plain(fake_ext, name, mode):
    raw, page = tiny.CONFIGS[name]
    folder = model_folder(name)
    requests = ru.make_requests(raw["vocab_size"], LENGTHS[name] + ((70, 45) if mode == "mixed" else ()), seed=11)
    expected = plain_logits(folder, raw, requests, "float32")
    max_tokens = 64 * 6
    trace = {"whole": ru.trace_whole, "last32": ru.trace_last_decoded, "portions": ru.trace_portions,
             "mixed": lambda r: ru.trace_mixed(r, max_tokens, seed=5)}[mode](requests)
    outputs = ru.run_inprocess(folder, "float32", trace, max_tokens, page_size=page)
    ru.compare(trace, outputs, expected, "float32")


def test_mixed_trace_reuses_pages(fake_ext):
    """The mixed scenario is only worth its name if pages really are handed on to later requests."""
    raw, page = tiny.CONFIGS["A"]
    requests = ru.make_requests(raw["vocab_size"], LENGTHS["A"] + (70, 45), seed=11)
    trace = ru.trace_mixed(requests, 64 * 6, seed=5)
    assert max(len(s["entries"]) for s in trace.steps) >= 3
    assert any(len(e["tokens"]) == 1 for s in trace.steps for e in s["entries"]) and \
        any(len(e["tokens"]) > 1 and len(s["entries"]) > 1 for s in trace.steps for e in s["entries"])
    total_rounded = sum((len(t) + 63) // 64 * 64 for t in requests.values())
    assert total_rounded > 64 * 6, "all requests fit at once: nothing would be reused"
