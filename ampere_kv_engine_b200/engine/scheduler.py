"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

States and rules follow the reference's scheduler (ampere_kv/scheduler.py:11, 73-110, 196-281):
``waiting -> prefilling -> running -> finished``; FIFO admission against a page *budget* (the
pages a request can ever hold, reserved at admission, so decoding can never run out:
scheduler.py:85-93, 196-204); stop on the token limit or on EOS (scheduler.py:104-110);
cancel and deadline seen only at the start of a round (scheduler.py:95-102, 206-227); one
place where a request's pages go back (scheduler.py:229-240).  The last chosen token is never
fed, so a finished request holds ``prompt + outputs - 1`` positions (ampere_kv/runner.py:367-369).

What differs: several requests may be prefilling; every round is one mixed batch (all running
requests' single tokens first, then prompt portions in arrival order until ``max_batch_tokens``
is used up); and what happens when pages run out is a policy:

``admission="budget"`` (default): as the reference; pages cannot run out after admission.
``admission="optimistic"``: a request is admitted when the pages for its *next portion* are
free.  If a later round cannot back its tokens, the most recently admitted live request is
preempted: its pages are given back and it returns to the head of the waiting queue, to be
prefilled again over ``prompt + outputs so far`` (recomputation; its outputs are kept).
A request alone in the engine that still cannot be backed is finished with reason
``"out of pages"``.

The scheduler is host logic only.  It talks to an *executor* with three members:
``manager`` (the :class:`CacheManager`), ``execute(entries, requests) -> list[int]`` (run the
batch, choose a token for every entry that wants one, in order) and ``vocab_size``.

An executor that also has ``launch(entries, requests, steps) -> handle`` and
``collect(handle) -> list[int]`` is driven one round ahead: round k + 1 is laid out and queued
on the device before round k's tokens are read, so the host's work hides behind the device's.
A request whose newest token is still on the device contributes an entry with a ``source``
(the row of that token among round k's choices) instead of a token id.  What the host cannot
know a round early is an EOS: a request that turns out to have ended in round k has one
speculative token computed in round k + 1, which is dropped (its pages go back as always; the
device runs rounds in order, so nobody else sees those pages before round k + 1 is through).
A request that ends by its token limit is not scheduled speculatively.  When pages run short
the round in flight is read first, so preemption decides with everything known.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field

from ..cache.manager import SequenceCache
from ..sampling.sampler import SamplingParams
from .batch import SeqStep

WAITING, PREFILLING, RUNNING, FINISHED = "waiting", "prefilling", "running", "finished"


class Request:
    def __init__(self, request_id, prompt: list[int], max_new_tokens: int, sampling: SamplingParams,
                 ignore_eos: bool = False, deadline: float | None = None):
        self.request_id = request_id
        self.prompt = list(prompt)
        self.max_new_tokens = max_new_tokens
        self.sampling = sampling
        self.ignore_eos = ignore_eos
        self.deadline = deadline            # absolute time.monotonic() value, or None
        self.status = WAITING
        self.output_ids: list[int] = []
        self.stop_reason = ""
        self.seq: SequenceCache | None = None
        self.budget: list[int] = []         # pages per group reserved at admission (budget policy)
        self.preemptions = 0
        self.admit_order = -1
        self.inflight_row: int | None = None    # row of this request's newest token in the round not yet read
        #: host clock (time.perf_counter) at submit and at every token's arrival on the host; kept only when the
        #: scheduler records times
        self.submitted_at: float | None = None
        self.token_times: list[float] = []

    @property
    def ttft_ms(self) -> float | None:
        """Submit to first token on the host, as the reference's request timings count it (ampere_kv/runner.py:385-405)."""
        if self.submitted_at is None or not self.token_times:
            return None
        return (self.token_times[0] - self.submitted_at) * 1000

    @property
    def largest_gap_ms(self) -> float | None:
        """The longest wait between two consecutive tokens of this request: what a running request feels when a
        prompt arrives beside it (the reference's scheduler benchmark reports the same,
        ampere_kv/bench_scheduler.py:242-271)."""
        if len(self.token_times) < 2:
            return None
        return max(b - a for a, b in zip(self.token_times, self.token_times[1:])) * 1000

    @property
    def tokens(self) -> list[int]:
        """Everything that must be in the cache before the next token can be chosen."""
        return self.prompt + self.output_ids

    @property
    def computed(self) -> int:
        return self.seq.length if self.seq is not None else 0


@dataclass
class StepStats:
    prefill_tokens: int = 0
    decode_tokens: int = 0
    num_seqs: int = 0
    preempted: int = 0
    free_pages: list[int] = field(default_factory=list)

    @property
    def batch_tokens(self) -> int:
        return self.prefill_tokens + self.decode_tokens


class Scheduler:
    def __init__(self, executor, *, max_batch_tokens: int = 2048, max_seqs: int = 256,
                 eos_token_ids=(), admission: str = "budget", max_context: int | None = None,
                 lookahead: bool | None = None, record_times: bool = False, nvtx: bool = False):
        if max_batch_tokens < 1 or max_seqs < 1:
            raise ValueError("max_batch_tokens and max_seqs must be positive")
        if admission not in ("budget", "optimistic"):
            raise ValueError("admission must be 'budget' or 'optimistic'")
        self.executor = executor
        self.manager = executor.manager
        self.max_batch_tokens = max_batch_tokens
        self.max_seqs = min(max_seqs, self.manager.max_seqs)
        self.eos_ids = set(eos_token_ids)
        self.admission = admission
        self.max_context = max_context
        self.waiting: list[Request] = []
        self.prefilling: list[Request] = []
        self.running: list[Request] = []
        self.reserved = [0] * len(self.manager.groups)
        self._admitted = 0
        self.preemptions = 0
        can_look_ahead = hasattr(executor, "launch") and hasattr(executor, "collect")
        #: queue each round before the previous round's tokens are read (None: whenever the executor can)
        self.lookahead = can_look_ahead if lookahead is None else bool(lookahead) and can_look_ahead
        self._inflight = None       # (handle, wanted requests) of the queued round whose tokens are not read yet
        self.dropped_tokens = 0     # speculative tokens of requests that had already ended
        #: keep the host time of every submit and every token (``Request.ttft_ms`` / ``largest_gap_ms``)
        self.record_times = bool(record_times)
        #: wrap every round in an NVTX range that names what it holds, as the reference's profiling run does
        #: (ampere_kv/bench_external.py:82-126); needs a CUDA build of torch, costs a few microseconds a round
        self.nvtx = bool(nvtx)
        self.rounds = 0

    # ------------------------------------------------------------------ public

    def submit(self, request_id, prompt, max_new_tokens: int, *, sampling: SamplingParams | None = None,
               ignore_eos: bool = False, deadline: float | None = None) -> Request:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("the prompt must hold at least one token")
        if max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be positive")
        vocab = self.executor.vocab_size
        bad = [t for t in prompt if not 0 <= t < vocab]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside the vocabulary of {vocab}")
        total = len(prompt) + max_new_tokens
        if self.max_context is not None and total > self.max_context:
            raise ValueError(f"prompt ({len(prompt)}) + max_new_tokens ({max_new_tokens}) exceeds the "
                             f"maximum context of {self.max_context}")
        request = Request(request_id, prompt, max_new_tokens, sampling or SamplingParams(), ignore_eos, deadline)
        request.budget = self._budget(total)
        if self.record_times:
            request.submitted_at = time.perf_counter()
        for need, group in zip(request.budget, self.manager.groups):
            if need > group.pool.count:
                raise ValueError(f"the request needs up to {need} pages of cache group {group.index}, "
                                 f"the pool holds {group.pool.count}")
        self.waiting.append(request)
        return request

    def cancel(self, request: Request) -> None:
        """Mark for removal; pages go back at the start of the next round."""
        if request.status != FINISHED:
            request.stop_reason = request.stop_reason or "cancelled"

    def has_work(self) -> bool:
        return bool(self.waiting or self.prefilling or self.running or self._inflight is not None)

    def step(self, now: float | None = None) -> tuple[list[Request], StepStats]:
        """One round.  Returns the requests that finished in it (each exactly once) and what ran."""
        self.rounds += 1
        if not self.nvtx:
            return self._round(now)
        import torch
        torch.cuda.nvtx.range_push(f"round {self.rounds}: running={len(self.running)} prefilling={len(self.prefilling)} "
                                   f"waiting={len(self.waiting)}")
        try:
            return self._round(now)
        finally:
            torch.cuda.nvtx.range_pop()

    def _round(self, now: float | None = None) -> tuple[list[Request], StepStats]:
        now = time.monotonic() if now is None else now
        finished = self._stop_round(now)
        self._admit()
        stats = StepStats()
        entries, owners = self._build_batch(stats, finished)
        if self.lookahead:
            launched = None
            if entries:
                wanted = [r for r, e in zip(owners, entries) if e.want]
                steps = [len(r.output_ids) + (r.inflight_row is not None) for r in wanted]
                launched = (self.executor.launch(entries, wanted, steps), wanted)
                for request in owners:      # the whole prompt is in the cache (or on its way): it decodes from now on
                    if request.status == PREFILLING and request.computed >= len(request.tokens):
                        self.prefilling.remove(request)
                        request.status = RUNNING
                        self.running.append(request)
            self._collect(finished)         # the round before, now that this one is queued behind it
            if launched is not None:
                self._inflight = launched
                for row, request in enumerate(launched[1]):
                    request.inflight_row = row
            stats.free_pages = self.manager.free_pages()
            return finished, stats
        if entries:
            wanted = [r for r, e in zip(owners, entries) if e.want]
            tokens = self.executor.execute(entries, wanted)
            if len(tokens) != len(wanted):
                raise RuntimeError("the executor returned a token count that does not match the batch")
            for request, token in zip(wanted, tokens):
                self._commit(request, int(token))
            for request in list(self.prefilling):
                if request.output_ids and request.computed >= len(request.tokens) - 1:
                    self.prefilling.remove(request)
                    if not request.stop_reason:
                        request.status = RUNNING
                        self.running.append(request)
            for request in [r for r in owners if r.stop_reason and r.status != FINISHED]:
                self._retire(request)
                finished.append(request)
        stats.free_pages = self.manager.free_pages()
        return finished, stats

    # ------------------------------------------------------------------ internals

    def _budget(self, total_tokens: int) -> list[int]:
        """Pages per group a request may hold: the final length is total - 1 (the last token is not fed),
        one spare page keeps the reference's conservative formula (ampere_kv/scheduler.py:85)."""
        page = self.manager.page_size
        conservative = (total_tokens + page) // page
        bounds = self.manager.pages_for_tokens(total_tokens, self.max_batch_tokens)
        return [min(conservative, b + 1) if g.window is not None else conservative
                for g, b in zip(self.manager.groups, bounds)]

    def _live(self) -> list[Request]:
        return self.prefilling + self.running

    def _admit(self) -> None:
        while self.waiting and len(self._live()) < self.max_seqs:
            request = self.waiting[0]
            if self.admission == "budget":
                if any(r + b > g.pool.count for r, b, g in zip(self.reserved, request.budget, self.manager.groups)):
                    return
            else:
                first = min(len(request.tokens), self.max_batch_tokens)
                need = self.manager.pages_to_start(first)
                if any(n > g.pool.num_free for n, g in zip(need, self.manager.groups)):
                    return
            self.waiting.pop(0)
            request.seq = self.manager.open(request.request_id)
            request.status = PREFILLING
            request.admit_order = self._admitted
            self._admitted += 1
            if self.admission == "budget":
                self.reserved = [r + b for r, b in zip(self.reserved, request.budget)]
            self.prefilling.append(request)

    def _collect(self, finished: list[Request]) -> None:
        """Read the tokens of the round in flight, if any, and do what ``step`` does after a round."""
        if self._inflight is None:
            return
        handle, wanted = self._inflight
        self._inflight = None
        tokens = self.executor.collect(handle)
        if len(tokens) != len(wanted):
            raise RuntimeError("the executor returned a token count that does not match the batch")
        for request, token in zip(wanted, tokens):
            request.inflight_row = None
            if request.status == FINISHED or request.stop_reason:
                self.dropped_tokens += 1        # it had ended before this round ran
                continue
            self._commit(request, int(token))
        for request in wanted:
            if request.stop_reason and request.status != FINISHED:
                self._retire(request)
                finished.append(request)

    def _plan(self) -> list[tuple[Request, int, int]]:
        """(request, first token index, count) for this round under the token budget."""
        plan = []
        budget = self.max_batch_tokens
        for request in self.running:
            if budget <= 0:
                break
            if request.inflight_row is not None and len(request.output_ids) + 1 >= request.max_new_tokens:
                continue        # the token in flight is its last
            plan.append((request, request.computed, 1))
            budget -= 1
        for request in self.prefilling:
            if budget <= 0:
                break
            remaining = len(request.tokens) - request.computed
            count = min(remaining, budget)
            plan.append((request, request.computed, count))
            budget -= count
        return plan

    def _build_batch(self, stats: StepStats, finished: list[Request]):
        while True:
            plan = self._plan()
            if not plan:
                return [], []
            # do the pages suffice?  (always, under budget admission)
            need = [0] * len(self.manager.groups)
            for request, _, count in plan:
                for gi, n in enumerate(self.manager.pages_needed(request.seq, count)):
                    need[gi] += n
            if all(n <= g.pool.num_free for n, g in zip(need, self.manager.groups)):
                break
            if self._inflight is not None:
                self._collect(finished)     # decide with everything known: requests may just have ended
                continue
            live = self._live()
            victim = max(live, key=lambda r: r.admit_order)
            if len(live) == 1:
                victim.stop_reason = "out of pages"
                self._retire(victim)
                finished.append(victim)
            else:
                self._preempt(victim)
                stats.preempted += 1
        entries, owners = [], []
        for request, start, count in plan:
            if request.inflight_row is not None:
                # its next token is the one the round in flight chooses
                entries.append(SeqStep(request.seq, [0], [0], source=request.inflight_row))
            else:
                tokens = request.tokens[start:start + count]
                last = start + count == len(request.tokens)
                entries.append(SeqStep(request.seq, tokens, [count - 1] if last else []))
            owners.append(request)
            if request.status == RUNNING:
                stats.decode_tokens += count
            else:
                stats.prefill_tokens += count
        stats.num_seqs = len(entries)
        return entries, owners

    def _preempt(self, request: Request) -> None:
        """Give the request's pages back and queue it again at the head; its outputs are kept."""
        self._release(request)
        request.status = WAITING
        request.preemptions += 1
        self.preemptions += 1
        self.waiting.insert(0, request)

    def _commit(self, request: Request, token: int) -> None:
        request.output_ids.append(token)
        if self.record_times:
            request.token_times.append(time.perf_counter())
        if len(request.output_ids) >= request.max_new_tokens:
            request.stop_reason = "length"
        elif token in self.eos_ids and not request.ignore_eos:
            request.stop_reason = "eos"

    def _stop_round(self, now: float) -> list[Request]:
        stopped = []
        for queue in (self.waiting, self.prefilling, self.running):
            for request in list(queue):
                expired = request.deadline is not None and request.deadline <= now
                if request.stop_reason or expired:
                    request.stop_reason = request.stop_reason or "deadline"
                    self._retire(request)
                    stopped.append(request)
        return stopped

    def _release(self, request: Request) -> None:
        if request in self.prefilling:
            self.prefilling.remove(request)
        if request in self.running:
            self.running.remove(request)
        if request in self.waiting:
            self.waiting.remove(request)
        if request.seq is not None:
            self.manager.close(request.seq)
            request.seq = None
            if self.admission == "budget":
                self.reserved = [r - b for r, b in zip(self.reserved, request.budget)]

    def _retire(self, request: Request) -> None:
        """The one place a finished request's pages and slot go back."""
        self._release(request)
        request.status = FINISHED
