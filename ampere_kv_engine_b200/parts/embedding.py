"""Token embedding and output head.

Embedding: a row gather without scaling (ampere_kv/runner.py:282) into the float32 residual
stream.  Head: ``logits = x W^T`` on the rows that were asked for, float32 out
(runner.py:297); a tied head reads the embedding matrix.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import ParamSpec, Part


class TokenEmbedding(Part):
    """params: ``vocab_size``."""

    graph_safe = True


    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.vocab_size = int(spec.params["vocab_size"])
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        return ops.embedding(token_ids, self.weight, status=getattr(ctx, "status", None),
                             sampled=getattr(ctx, "sampled", None))


class LinearHead(Part):
    """params: ``vocab_size``, ``tied`` (read the embedding's matrix instead of one's own)."""

    graph_safe = True


    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.vocab_size = int(spec.params["vocab_size"])
        self.tied = bool(spec.params.get("tied", False))
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        # a tied checkpoint may still carry the head's tensor; it is then ignored
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size), optional=self.tied)}

    def load(self, tensors):
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, embedding: TokenEmbedding) -> None:
        if self.tied:
            self.weight = embedding.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, out_dtype=torch.float32)
