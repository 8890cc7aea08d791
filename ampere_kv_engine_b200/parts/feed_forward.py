"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))``.

The reference's form (ampere_kv/runner.py:172-177) with SiLU.  gate and up are stored as one
matrix (gate rows first), so one product feeds the activation kernel; each output element
keeps its own row's accumulation order.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, ParamSpec, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """params: ``intermediate_size``, ``activation`` (only ``"silu"``)."""

    graph_safe = True


    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.intermediate_size = int(spec.params["intermediate_size"])
        activation = spec.params.get("activation", "silu")
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} is not supported (only 'silu')")
        self.gate_up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None

    def param_specs(self):
        i, h = self.intermediate_size, self.hidden_size
        return {
            "gate_proj.weight": ParamSpec((i, h)),
            "up_proj.weight": ParamSpec((i, h)),
            "down_proj.weight": ParamSpec((h, i)),
        }

    def load(self, tensors):
        self.gate_up = torch.cat((tensors["gate_proj.weight"], tensors["up_proj.weight"]), dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def forward(self, x, ctx):
        status = getattr(ctx, "status", None)
        gate_up = ops.linear(x, self.gate_up, partial_ok=True, status=status)
        return ops.linear(ops.silu_mul(gate_up, self.dtype), self.down, partial_ok=True, status=status)
