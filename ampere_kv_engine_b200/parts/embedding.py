"""Token embedding and output head.

Embedding: a row gather without scaling (ampere_kv/runner.py:282) into the float32 residual
stream.  Head: ``logits = x W^T`` on the rows that were asked for, float32 out
(runner.py:297); a tied head reads the embedding matrix.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Embedding, Head, ParamSpec, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Embedding):
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


@register_head("linear_head")
class LinearHead(Head):
    """params: ``vocab_size``, ``tied`` (read the embedding's matrix instead of one's own).  A tied checkpoint may
    still carry the head's tensor: it is accepted if it equals the embedding's and refused if it differs."""

    graph_safe = True


    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.vocab_size = int(spec.params["vocab_size"])
        self.tied = bool(spec.params.get("tied", False))
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab_size, self.hidden_size), optional=self.tied)}

    def load(self, tensors):
        if not self.tied:
            self.weight = tensors["weight"].contiguous()
        else:
            self._stored = tensors.get("weight")

    def tie(self, embedding) -> None:
        if not self.tied:
            return
        if getattr(embedding, "weight", None) is None or tuple(embedding.weight.shape) != (self.vocab_size,
                                                                                           self.hidden_size):
            raise ValueError("a tied head needs an embedding with a [vocab, hidden] matrix named 'weight'")
        stored = getattr(self, "_stored", None)
        if stored is not None and not torch.equal(stored, embedding.weight):
            from ..weights.loader import WeightError
            name = f"{self.spec.prefix}.weight" if self.spec.prefix else "weight"
            raise WeightError(f"the checkpoint ties the head to the embedding but carries a different {name} "
                              f"(largest difference {float((stored.float() - embedding.weight.float()).abs().max()):.3g})")
        self._stored = None
        self.weight = embedding.weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, out_dtype=torch.float32)
