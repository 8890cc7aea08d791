"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

One function replaces the reference's three (``model_forward``, ``model_forward_batched``,
``model_forward_mixed``: ampere_kv/runner.py:219-290).  A step reserves pages for the new
tokens, lays the batch out, runs the model's schedule over exactly these tokens (earlier ones
are only read from the cache) and, when it succeeded, commits the new lengths.  Pages that a
failed step reserved are given back; the reference offers no such rollback
(runner.py:112 docstring).
"""

from __future__ import annotations

import torch

from ..cache.manager import CacheManager, SequenceCache
from ..kernels import ops
from .batch import BatchLayout, SeqStep, build_context, fill_host, make_context, validate_entries

_STATUS_TEXT = {
    1: "a block-table entry pointed outside the page pool",
    2: "a cache slot was outside the page pool",
    3: "a token id was outside the vocabulary",
    4: "a wanted row was outside the batch",
    5: "a bounded wait inside a kernel gave up",
}


class KernelStatusError(RuntimeError):
    """A kernel met an impossible index, skipped the access and reported it."""


_SEQ_BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)
_WIDTH_STEP = 64            # block-table widths of captured decode steps are multiples of this many pages


class _CapturedDecode:
    """A decode step of a fixed layout, captured once and replayed: pinned host buffer, device buffer,
    the context of views into it, the graph and its output logits."""

    RING = 4

    def __init__(self, layout, dev, ctx, graph, logits, launches):
        self.layout, self.dev, self.ctx, self.graph, self.logits = layout, dev, ctx, graph, logits
        self.launches = launches      # kernels of this package inside the graph
        # The host may run several steps ahead of the device, so the staging buffer of one step must not be
        # rewritten before its copy has run: a small ring of pinned buffers, each guarded by an event.
        self.pinned = [torch.empty(layout.total, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self.copied = [None] * self.RING
        self.turn = 0

    def stage(self):
        """The next free pinned buffer (waits for its last copy to have run)."""
        self.turn = (self.turn + 1) % self.RING
        if self.copied[self.turn] is not None:
            self.copied[self.turn].synchronize()
        return self.pinned[self.turn]

    def upload(self, pinned):
        self.dev.copy_(pinned, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self.copied[self.turn] = event


class ModelRunner:
    def __init__(self, model, *, page_size: int = 16, num_pages: int, max_seqs: int = 256,
                 kv_dtype: torch.dtype | None = None, cuda_graphs: bool = True):
        if not model.loaded:
            raise ValueError("the model has no weights yet")
        self.model = model
        self.device = model.device
        kv_dtype = kv_dtype or model.dtype
        if kv_dtype != model.dtype:
            raise ValueError(f"the cache dtype ({kv_dtype}) must equal the compute dtype ({model.dtype}): "
                             f"cache pages are read by the attention kernels as they are")
        self.manager = CacheManager(model.cache_specs(), model.cache_of(), page_size=page_size, num_pages=num_pages,
                                    max_seqs=max_seqs, dtype=kv_dtype, device=self.device)
        self.views = self.manager.layer_views()
        self.q_tile = model.q_tile() if hasattr(model, "q_tile") else ops.ATTENTION_Q_TILE
        # the kernels' status word and, behind it, the tokens the last step chose (kept on the device: an entry with
        # a ``source`` reads its token here): one buffer, so that one copy brings both to the host
        self.outcome = torch.zeros(1 + max(1, max_seqs), dtype=torch.int32, device=self.device)
        self.status = self.outcome[:1]
        self.sampled = self.outcome[1:]
        self.steps_run = 0
        self.last_h2d_bytes = 0
        #: decode-only steps are replayed as CUDA graphs (one per batch-size and table-width bucket)
        self.cuda_graphs = bool(cuda_graphs) and self.device.type == "cuda" and model.graph_safe
        self._captured: dict[tuple, _CapturedDecode] = {}
        # captured steps share one memory pool: they never run at the same time and each one's logits are
        # consumed before the next step starts
        self._graph_pool = torch.cuda.graph_pool_handle() if self.cuda_graphs else None
        self.graph_replays = 0

    # ------------------------------------------------------------------ requests

    def open(self, request_id) -> SequenceCache:
        return self.manager.open(request_id)

    def close(self, seq: SequenceCache) -> None:
        self.manager.close(seq)

    # ------------------------------------------------------------------ the step

    def step(self, entries: list[SeqStep]) -> torch.Tensor | None:
        """Run one batch.  Returns float32 logits [wanted places in entry order, vocab], or None."""
        vocab = self.model.spec.vocab_size
        for e in entries:
            for t in e.tokens:
                if not 0 <= t < vocab:
                    raise ValueError(f"request {e.seq.request_id!r}: token id {t} is outside the vocabulary "
                                     f"of {vocab}")
        reserved: list[SeqStep] = []
        try:
            for e in entries:
                self.manager.reserve(e.seq, len(e.tokens))
                reserved.append(e)
            validate_entries(entries)
            if self.cuda_graphs and all(len(e.tokens) == 1 for e in entries) and len(entries) <= _SEQ_BUCKETS[-1]:
                logits = self._decode_step_captured(entries)
            else:
                ctx = build_context(self.manager, entries, self.device, status=self.status, sampled=self.sampled,
                                    q_tile=self.q_tile)
                self.last_h2d_bytes = ctx.h2d_bytes
                logits = self.model.forward(ctx, self.views)
        except BaseException:
            for e in reserved:
                self.manager.release_unused(e.seq)
            raise
        for e in entries:
            self.manager.commit(e.seq, len(e.tokens))
        self.steps_run += 1
        return logits

    # ------------------------------------------------------------------ captured decode steps

    def _decode_layout(self, entries: list[SeqStep]) -> BatchLayout:
        n = len(entries)
        bucket = next(b for b in _SEQ_BUCKETS if b >= n)
        widths = []
        for g in self.manager.groups:
            widest = max(len(self.manager.table_row(e.seq, g.index)) for e in entries)
            widths.append((max(1, widest) + _WIDTH_STEP - 1) // _WIDTH_STEP * _WIDTH_STEP)
        # every row's logits are computed; rows that are not wanted are dropped afterwards
        return BatchLayout(bucket, bucket, bucket, bucket, tuple(widths))

    def _decode_step_captured(self, entries: list[SeqStep]) -> torch.Tensor | None:
        layout = self._decode_layout(entries)
        captured = self._captured.get(layout.key())
        full = [SeqStep(e.seq, e.tokens, [0], e.source) for e in entries]
        if captured is None:
            captured = self._capture(layout, full)
        else:
            pinned = captured.stage()
            fill_host(self.manager, full, layout, pinned.numpy(), 1)
            captured.upload(pinned)
            captured.graph.replay()
            ops.launch_count += captured.launches
            self.graph_replays += 1
        self.last_h2d_bytes = int(layout.total * 4)
        wanted = [i for i, e in enumerate(entries) if e.want]
        if not wanted:
            return None
        if len(wanted) == len(entries):
            return captured.logits[:len(entries)]
        return captured.logits[torch.tensor(wanted, device=self.device)]

    def _capture(self, layout: BatchLayout, entries: list[SeqStep]) -> _CapturedDecode:
        pinned = torch.empty(layout.total, dtype=torch.int32).pin_memory()
        dev = torch.empty(layout.total, dtype=torch.int32, device=self.device)
        q_lens, ctx_lens = fill_host(self.manager, entries, layout, pinned.numpy(), 1)
        dev.copy_(pinned, non_blocking=False)
        # the split count of the attention kernels is fixed at capture: size it for the middle of the contexts that
        # this bucket of table widths serves (any count is right for any context; it only decides the speed)
        max_context = max(1, (max(layout.widths) - _WIDTH_STEP // 2) * self.manager.page_size)
        # and for the mix of lengths this batch has (the next batches of the bucket are mostly this one, grown)
        live = [c for c in ctx_lens if c > 0] or [max_context]
        mean_context = max(1, max_context * sum(live) // (len(live) * max(live)))
        ctx = make_context(layout, dev, tile_rows=1, max_context=max_context, status=self.status,
                           q_lens=q_lens, ctx_lens=ctx_lens, state_slots=[e.seq.state_slot for e in entries],
                           h2d_bytes=int(layout.total * 4), sampled=self.sampled,
                           decode_contexts=(max_context, mean_context))
        # one eager run first (library handles and workspaces come into being outside the capture); it writes the
        # same cache slots the captured run writes again
        self.model.forward(ctx, self.views)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self.model.forward(ctx, self.views)
        launches = ops.launch_count - before
        graph.replay()
        captured = _CapturedDecode(layout, dev, ctx, graph, logits, launches)
        self._captured[layout.key()] = captured
        return captured

    def raise_on_status(self) -> None:
        """Read the kernels' status word (synchronises) and raise if a kernel reported a bad index."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise KernelStatusError(f"kernel status {code}: {_STATUS_TEXT.get(code, 'unknown')}")
