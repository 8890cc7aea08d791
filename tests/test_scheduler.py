"""The scheduler's decisions, with a stub in place of the model: admission in arrival order against the page
budget, prompts cut into portions under the token budget beside decoded tokens, finishing and freeing,
cancel and deadline at round starts, and what happens when pages run out (wait / preempt and recompute /
give up)."""

import pytest
import torch

from ampere_kv_engine_b200.cache.manager import CacheManager
from ampere_kv_engine_b200.engine.scheduler import (FINISHED, PREFILLING, RUNNING, WAITING, Scheduler)
from ampere_kv_engine_b200.parts.base import CacheSpec

VOCAB = 101


class StubExecutor:
    """Does what the real step does to the cache (reserve, commit) and 'predicts' a token that depends on
    every token the request has been fed so far, so a recomputed request must come out the same."""

    def __init__(self, pages=16, page=16, seqs=8, specs=None):
        specs = specs or [CacheSpec("full", 2, 16)]
        self.manager = CacheManager(specs, [None] * len(specs), page_size=page, num_pages=pages, max_seqs=seqs,
                                    dtype=torch.float32, device="cpu", allocate_storage=False)
        self.vocab_size = VOCAB
        self.fed: dict[object, list[int]] = {}
        self.batches: list[list[tuple[object, int, int, bool]]] = []

    def execute(self, entries, wanted):
        tokens = []
        record = []
        for e in entries:
            self.manager.reserve(e.seq, len(e.tokens))
        for e in entries:
            history = self.fed.setdefault(e.seq.request_id, [])
            if e.seq.length == 0:
                history.clear()
            assert len(history) == e.seq.length, "a step must continue where the cache stops"
            history.extend(e.tokens)
            record.append((e.seq.request_id, e.seq.length, len(e.tokens), bool(e.want)))
            self.manager.commit(e.seq, len(e.tokens))
            if e.want:
                tokens.append(predict(history))
        self.batches.append(record)
        self.manager.check_invariants()
        return tokens


def predict(history):
    return (sum((i + 1) * t for i, t in enumerate(history)) * 31 + len(history)) % VOCAB


def expected_output(prompt, n):
    ids, out = list(prompt), []
    for _ in range(n):
        out.append(predict(ids))
        ids.append(out[-1])
    return out


def drive(s, limit=500):
    finished = []
    for _ in range(limit):
        if not s.has_work():
            return finished
        done, _ = s.step(now=0.0)
        finished += done
    raise AssertionError("the scheduler did not finish")


def prompt(n, salt=0):
    return [(7 * i + salt) % VOCAB for i in range(n)]


def test_prompt_is_cut_under_the_token_budget_and_mixed_with_decoding():
    ex = StubExecutor(pages=64)
    s = Scheduler(ex, max_batch_tokens=24)
    a = s.submit("a", prompt(10), 5)
    s.step(now=0.0)
    assert a.status == RUNNING and len(a.output_ids) == 1
    b = s.submit("b", prompt(60, 3), 3)
    s.step(now=0.0)
    # a's single token comes first, b's portion fills the rest of the 24-token budget, no logits for a mid-prompt portion
    assert ex.batches[-1] == [("a", 10, 1, True), ("b", 0, 23, False)]
    assert b.status == PREFILLING and b.output_ids == []
    s.step(now=0.0)
    assert ex.batches[-1] == [("a", 11, 1, True), ("b", 23, 23, False)]
    s.step(now=0.0)
    assert ex.batches[-1] == [("a", 12, 1, True), ("b", 46, 14, True)]
    assert b.status == RUNNING and len(b.output_ids) == 1
    done = drive(s)
    assert {r.request_id for r in done} == {"a", "b"} and all(r.status == FINISHED for r in done)
    assert a.output_ids == expected_output(prompt(10), 5) and b.output_ids == expected_output(prompt(60, 3), 3)
    assert a.stop_reason == b.stop_reason == "length"
    # the last chosen token is never fed: a held 10 + 5 - 1 positions at the end
    assert len(ex.fed["a"]) == 14
    assert ex.manager.free_pages() == [64] and s.reserved == [0]


def test_admission_is_fifo_against_the_page_budget():
    ex = StubExecutor(pages=8)                       # 128 positions
    s = Scheduler(ex, max_batch_tokens=512)
    big = s.submit("big", prompt(70), 10)            # budget (80 + 16) // 16 = 6 pages
    small = s.submit("small", prompt(20, 1), 4)      # budget 2 pages
    late = s.submit("late", prompt(5, 2), 4)         # budget 1 page: would fit, but must not overtake
    s.step(now=0.0)
    assert (big.status, small.status, late.status) == (RUNNING, RUNNING, WAITING)
    assert s.reserved == [8]
    done = drive(s)
    assert [r.request_id for r in done] == ["small", "late", "big"] or [r.request_id for r in done][0] == "small"
    assert late.output_ids == expected_output(prompt(5, 2), 4)
    assert ex.manager.free_pages() == [8]
    with pytest.raises(ValueError, match="pages"):
        s.submit("huge", prompt(200), 10)


def test_submit_validates():
    s = Scheduler(StubExecutor(), max_context=64)
    with pytest.raises(ValueError, match="at least one token"):
        s.submit("x", [], 3)
    with pytest.raises(ValueError, match="positive"):
        s.submit("x", [1], 0)
    with pytest.raises(ValueError, match="vocabulary"):
        s.submit("x", [1, VOCAB], 3)
    with pytest.raises(ValueError, match="maximum context"):
        s.submit("x", prompt(60), 10)


def test_eos_stops_unless_ignored():
    ex = StubExecutor()
    out = expected_output(prompt(6), 8)
    s = Scheduler(ex, eos_token_ids=(out[2],))
    a = s.submit("a", prompt(6), 8)
    b = s.submit("b", prompt(6), 8, ignore_eos=True)
    drive(s)
    assert a.output_ids == out[:out.index(out[2]) + 1] and a.stop_reason == "eos"
    assert b.output_ids == out and b.stop_reason == "length"


def test_cancel_and_deadline_are_seen_at_round_start_only():
    ex = StubExecutor(pages=8)
    s = Scheduler(ex, max_batch_tokens=8)
    running = s.submit("run", prompt(4), 50)
    chunked = s.submit("pre", prompt(30, 1), 5, deadline=10.0)
    queued = s.submit("wait", prompt(40, 2), 5)       # no budget left for it: stays waiting
    s.step(now=0.0)
    assert (running.status, chunked.status, queued.status) == (RUNNING, PREFILLING, WAITING)
    s.cancel(running)
    s.cancel(queued)
    assert running.status == RUNNING                   # nothing happens until the next round starts
    done, _ = s.step(now=5.0)
    assert {r.request_id for r in done} == {"run", "wait"}
    assert running.stop_reason == queued.stop_reason == "cancelled" and queued.output_ids == []
    assert all(r[0] == "pre" for r in ex.batches[-1])  # the cancelled request ran no more
    done, _ = s.step(now=10.0)                         # a deadline in the past, never a sleep
    assert [r.request_id for r in done] == ["pre"] and chunked.stop_reason == "deadline"
    assert ex.manager.free_pages() == [8] and s.reserved == [0] and not s.has_work()
    s.cancel(running)                                  # cancelling a finished request changes nothing
    assert running.stop_reason == "cancelled"


def test_optimistic_admission_preempts_the_newest_and_recomputes():
    ex = StubExecutor(pages=6)                         # 96 positions
    s = Scheduler(ex, max_batch_tokens=64, admission="optimistic")
    first = s.submit("first", prompt(40), 30)          # grows to 69 positions = 5 pages
    second = s.submit("second", prompt(30, 1), 30)     # grows to 59 positions = 4 pages: both cannot finish together
    finished = drive(s)
    assert s.preemptions >= 1 and second.preemptions >= 1 and first.preemptions == 0
    assert first.output_ids == expected_output(prompt(40), 30)
    assert second.output_ids == expected_output(prompt(30, 1), 30)      # recomputed, same tokens
    assert [r.request_id for r in finished] == ["first", "second"]
    assert ex.manager.free_pages() == [6]
    # under the budget policy the same load never preempts: the second request waits instead
    ex2 = StubExecutor(pages=6)
    s2 = Scheduler(ex2, max_batch_tokens=64)
    a = s2.submit("first", prompt(40), 30)
    b = s2.submit("second", prompt(30, 1), 30)
    s2.step(now=0.0)
    assert b.status == WAITING
    drive(s2)
    assert s2.preemptions == 0 and b.output_ids == second.output_ids


def test_a_lone_request_that_cannot_be_backed_gives_up():
    ex = StubExecutor(pages=2)
    s = Scheduler(ex, max_batch_tokens=64, admission="optimistic")
    with pytest.raises(ValueError, match="needs up to 3 pages"):
        s.submit("r", prompt(20), 12)                  # can never fit: refused at once
    ex3 = StubExecutor(pages=3)
    s3 = Scheduler(ex3, max_batch_tokens=64, admission="optimistic")
    hog = ex3.manager.open("someone else")             # a page the scheduler does not own
    ex3.manager.reserve(hog, 16)
    r = s3.submit("r", prompt(20), 20)
    done = drive(s3)
    assert done == [r] and r.stop_reason == "out of pages" and len(r.output_ids) > 0
    assert ex3.manager.free_pages() == [2]


def test_window_groups_need_fewer_pages():
    specs = [CacheSpec("full", 2, 16), CacheSpec("window", 2, 16, window=32)]
    ex = StubExecutor(pages=40, specs=specs)
    s = Scheduler(ex, max_batch_tokens=16)
    r = s.submit("r", prompt(300), 20)
    assert r.budget[0] == (320 + 16) // 16 and r.budget[1] < 10
    peak = 0
    while s.has_work():
        s.step(now=0.0)
        if r.seq is not None:
            peak = max(peak, len(r.seq.held_pages(1)))
            assert len(r.seq.held_pages(1)) <= r.budget[1]
    assert 3 <= peak <= r.budget[1] and r.output_ids == expected_output(prompt(300), 20)


def test_stats_report_what_ran():
    ex = StubExecutor(pages=32)
    s = Scheduler(ex, max_batch_tokens=20)
    s.submit("a", prompt(8), 3)
    _, st = s.step(now=0.0)
    assert (st.prefill_tokens, st.decode_tokens, st.num_seqs) == (8, 0, 1)
    s.submit("b", prompt(50, 1), 3)
    _, st = s.step(now=0.0)
    assert (st.prefill_tokens, st.decode_tokens, st.num_seqs, st.batch_tokens) == (19, 1, 2, 20)
    assert st.free_pages == ex.manager.free_pages()


class AheadExecutor(StubExecutor):
    """The stub with ``launch`` / ``collect``: a round's tokens become readable only at ``collect``, and an entry
    with a ``source`` takes its token from the previous round's choices, as the device does."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.sampled: list[int] = []
        self.launched = self.collected = 0

    def launch(self, entries, wanted, steps):
        assert self.launched - self.collected <= 1, "at most one round may be unread when the next is queued"
        assert len(steps) == len(wanted)
        resolved = []
        for e in entries:
            if e.source is not None:
                assert e.tokens == [0] and e.want == [0]
                e = type(e)(e.seq, [self.sampled[e.source]], e.want)
            resolved.append(e)
        tokens = StubExecutor.execute(self, resolved, wanted)
        self.sampled = list(tokens)
        self.launched += 1
        return list(tokens)

    def collect(self, handle):
        self.collected += 1
        return handle


def test_lookahead_gives_the_same_tokens_and_frees_everything():
    prompts = [prompt(10), prompt(33, 3), prompt(5, 9), prompt(47, 1)]
    limits = [5, 1, 12, 2]
    outs = {}
    for ahead in (False, True):
        ex = AheadExecutor(pages=64)
        s = Scheduler(ex, max_batch_tokens=24, lookahead=ahead)
        assert s.lookahead is ahead
        reqs = [s.submit(i, p, n) for i, (p, n) in enumerate(zip(prompts, limits))]
        done = drive(s)
        assert sorted(r.request_id for r in done) == [0, 1, 2, 3]
        assert all(r.status == FINISHED and r.stop_reason == "length" for r in reqs)
        outs[ahead] = [r.output_ids for r in reqs]
        assert ex.manager.free_pages() == [64] and ex.launched == ex.collected
        assert s.dropped_tokens == 0           # a token limit is known a round early: nothing speculative
    assert outs[True] == outs[False] == [expected_output(p, n) for p, n in zip(prompts, limits)]


def test_lookahead_drops_the_token_computed_past_an_eos():
    p = prompt(10)
    chain = expected_output(p, 6)
    eos = chain[3]
    assert eos not in chain[:3]
    ex = AheadExecutor(pages=64)
    s = Scheduler(ex, eos_token_ids=[eos], lookahead=True)
    a = s.submit("a", p, 10)
    b = s.submit("b", prompt(12, 5), 10, ignore_eos=True)
    drive(s)
    assert a.output_ids == chain[:4] and a.stop_reason == "eos"
    assert len(b.output_ids) == 10 and b.output_ids == expected_output(prompt(12, 5), 10)
    assert s.dropped_tokens == 1               # the round queued before the EOS was read
    assert ex.manager.free_pages() == [64]
    # the stub saw one token more of "a" than it kept: the speculative one
    assert len(ex.fed["a"]) == len(p) + 4


def test_lookahead_reads_the_round_in_flight_before_it_preempts():
    ex = AheadExecutor(pages=6, page=16)
    s = Scheduler(ex, admission="optimistic", max_batch_tokens=64, lookahead=True)
    a = s.submit("a", prompt(40), 30)
    b = s.submit("b", prompt(40, 2), 30)
    drive(s)
    assert s.preemptions >= 1
    assert a.output_ids == expected_output(prompt(40), 30)
    assert b.output_ids == expected_output(prompt(40, 2), 30)
    assert ex.manager.free_pages() == [6]


def test_lookahead_cancel_and_empty_rounds():
    ex = AheadExecutor(pages=64)
    s = Scheduler(ex, lookahead=True)
    a = s.submit("a", prompt(8), 50, ignore_eos=True)
    for _ in range(5):
        s.step(now=0.0)
    s.cancel(a)
    done = drive(s)
    assert [r.request_id for r in done] == ["a"] and a.stop_reason == "cancelled"
    assert not s.has_work() and ex.manager.free_pages() == [64] and ex.launched == ex.collected
    assert a.output_ids == expected_output(prompt(8), len(a.output_ids))


@pytest.mark.parametrize("seed", range(24))
def test_random_arrivals_cancels_and_pools_end_right(seed):
    """Random prompts, limits, arrival rounds, cancellations, deadlines and end-of-sequence tokens, under both
    admission rules, round by round and queued ahead, with full and windowed cache groups and pools from roomy to
    barely enough: every request ends exactly once, with the tokens it would get alone (cut at its end-of-sequence
    token, or a prefix of them if it was cancelled or timed out), and every page and slot comes back."""
    import random
    rng = random.Random(seed)
    specs = [CacheSpec("full", 2, 16)] + ([CacheSpec("window", 2, 16, window=rng.choice((8, 24)))] if seed % 3 == 0 else [])
    page = rng.choice((4, 16))
    count = rng.randint(3, 9)
    prompts = [prompt(rng.randint(1, 70), salt=rng.randint(0, 50)) for _ in range(count)]
    limits = [rng.randint(1, 30) for _ in range(count)]
    arrive = sorted(rng.randint(0, 25) for _ in range(count))
    biggest = max((len(p) + n + page) // page + 1 for p, n in zip(prompts, limits))
    pages = biggest + rng.choice((0, 2, biggest, 4 * biggest))
    admission = rng.choice(("budget", "optimistic"))
    ahead = bool(seed % 2)
    eos = rng.randrange(VOCAB) if rng.random() < 0.5 else None
    ex = AheadExecutor(pages=pages, page=page, seqs=rng.choice((2, 4, 8)), specs=specs)
    s = Scheduler(ex, max_batch_tokens=rng.choice((8, 24, 64)), admission=admission, lookahead=ahead,
                  eos_token_ids=(eos,) if eos is not None else ())
    cancel_at = {i: arrive[i] + rng.randint(0, 20) for i in range(count) if rng.random() < 0.25}
    deadline = {i: float(arrive[i] + rng.randint(1, 30)) for i in range(count) if rng.random() < 0.15}
    requests, ended = {}, []
    for round_no in range(3000):
        for i in range(count):
            if arrive[i] == round_no and i not in requests:
                requests[i] = s.submit(i, prompts[i], limits[i], deadline=deadline.get(i))
            if cancel_at.get(i) == round_no and i in requests:
                s.cancel(requests[i])
        if len(requests) == count and not s.has_work():
            break
        done, stats = s.step(now=float(round_no))
        ended += done
        assert stats.batch_tokens <= s.max_batch_tokens
    else:
        raise AssertionError("the scheduler did not finish")
    assert sorted(r.request_id for r in ended) == list(range(count)), "every request ends exactly once"
    for i, r in requests.items():
        full = expected_output(prompts[i], limits[i])
        if eos is not None and eos in full:
            full = full[:full.index(eos) + 1]
        assert r.status == FINISHED and r.stop_reason
        if r.stop_reason in ("length", "eos"):
            assert r.output_ids == full, (i, r.stop_reason)
            if r.stop_reason == "eos":
                assert full[-1] == eos
            else:
                assert len(full) == limits[i]
        else:
            assert r.stop_reason in ("cancelled", "deadline", "out of pages"), r.stop_reason
            assert r.output_ids == full[:len(r.output_ids)]
            if r.stop_reason == "out of pages":
                assert admission == "optimistic"
    ex.manager.check_invariants()
    assert ex.manager.free_pages() == [pages] * len(specs) and s.reserved == [0] * len(specs)
    assert ex.launched == ex.collected


def test_kernel_status_becomes_an_error_and_is_cleared(fake_ext):
    """A kernel that met an impossible index, or whose bounded wait gave up, leaves a code in the status word; the
    step's owner turns it into one Python error at its sync point and clears the word."""
    from ampere_kv_engine_b200.config.engine_config import EngineConfig
    from ampere_kv_engine_b200.engine.engine import Engine
    from ampere_kv_engine_b200.engine.step import KernelStatusError
    from models_util import model_folder
    engine = Engine.from_pretrained(model_folder("A"), device="cpu", config=EngineConfig(dtype="float32", num_pages=16))
    runner = engine.runner
    runner.raise_on_status()                         # nothing reported: nothing raised
    for code, text in ((5, "bounded wait"), (1, "block-table"), (3, "token id"), (77, "unknown")):
        runner.status.fill_(code)
        with pytest.raises(KernelStatusError, match=text):
            runner.raise_on_status()
        assert int(runner.status.item()) == 0
    # through the executor: a code left by the step surfaces when its tokens are collected
    scheduler = engine.new_scheduler(lookahead=False)
    scheduler.submit("r", [1, 2, 3], 4, ignore_eos=True)
    scheduler.step()
    runner.status.fill_(5)
    with pytest.raises(KernelStatusError, match="bounded wait"):
        scheduler.step()
    assert int(runner.status.item()) == 0


def test_recorded_times_give_ttft_and_the_largest_gap():
    """With ``record_times`` every request keeps its submit time and the arrival of each token: the time to the
    first token and the longest wait between two tokens (what a running request feels when a prompt arrives)."""
    import time as clock
    ex = StubExecutor()
    real_execute = ex.execute

    def execute(entries, wanted):
        if len(ex.batches) == 3:           # one slow round in the middle of the decoding
            clock.sleep(0.03)
        return real_execute(entries, wanted)
    ex.execute = execute
    s = Scheduler(ex, max_batch_tokens=64, record_times=True)
    a = s.submit("a", list(range(1, 9)), 6, ignore_eos=True)
    while s.has_work():
        s.step()
    assert len(a.token_times) == 6 and a.submitted_at is not None
    assert a.ttft_ms is not None and a.ttft_ms >= 0
    assert a.largest_gap_ms >= 25                      # the slow round shows as the largest gap
    plain = Scheduler(StubExecutor(), max_batch_tokens=64)
    b = plain.submit("b", [1, 2, 3], 2, ignore_eos=True)
    while plain.has_work():
        plain.step()
    assert b.token_times == [] and b.ttft_ms is None and b.largest_gap_ms is None
