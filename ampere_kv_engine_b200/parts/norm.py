"""RMSNorm fused with the residual sum.

Formula of the reference (ampere_kv/runner.py:48-57): float32 mean of squares over the last
dim, ``x * rsqrt(ms + eps)``, times a plain weight (not ``1 + w``).  The reference rounds to
the activation dtype before the weight multiply; here the product is formed in float32 and
rounded once.  The residual sums of runner.py:167 and :179 are folded into the same kernel and
kept in float32.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, ParamSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """params: ``size`` (defaults to the hidden size), ``eps``."""

    graph_safe = True


    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.size = int(spec.params.get("size", self.hidden_size))
        self.eps = float(spec.params["eps"])
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), kind="vector", init="norm")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    takes_summed = True
    takes_pending = True

    def forward(self, hidden, delta, ctx, rows=None, lazy=False):
        status = getattr(ctx, "status", None)
        if isinstance(delta, ops.PendingPhases):
            if lazy and rows is None and self.size == hidden.shape[1] and self.weight.data_ptr() % 16 == 0:
                return ops.StreamNorm(delta, self.weight, self.eps, self.dtype)
            return None
        if isinstance(delta, ops.Summed):
            if lazy and rows is None and self.size == hidden.shape[1]:
                return ops.LazyNorm(delta, self.weight, self.eps, self.dtype, status)
            delta = None      # hidden holds the sum already
        return ops.add_rmsnorm(hidden, delta, self.weight, self.eps, self.dtype, rows=rows, status=status)
