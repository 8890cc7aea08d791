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

from ..cache.block_pool import OutOfPages
from ..cache.manager import CacheManager, SequenceCache
from ..kernels import ops
from .batch import SeqStep, StepContext, build_context

_STATUS_TEXT = {
    1: "a block-table entry pointed outside the page pool",
    2: "a cache slot was outside the page pool",
    3: "a token id was outside the vocabulary",
    4: "a wanted row was outside the batch",
    5: "a bounded wait inside a kernel gave up",
}


class KernelStatusError(RuntimeError):
    """A kernel met an impossible index, skipped the access and reported it."""


class ModelRunner:
    def __init__(self, model, *, page_size: int = 16, num_pages: int, max_seqs: int = 256,
                 kv_dtype: torch.dtype | None = None):
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
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self.last_h2d_bytes = 0

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
            ctx = build_context(self.manager, entries, self.device, status=self.status)
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

    def raise_on_status(self) -> None:
        """Read the kernels' status word (synchronises) and raise if a kernel reported a bad index."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise KernelStatusError(f"kernel status {code}: {_STATUS_TEXT.get(code, 'unknown')}")
