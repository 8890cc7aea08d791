"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))``.

The reference's form (ampere_kv/runner.py:172-177) with SiLU.  gate and up are stored as one
matrix, so one product feeds the activation; each output element keeps its own row's
accumulation order.  Where the intermediate size allows it the rows alternate in runs of 64
gate rows and the 64 up rows of the same outputs: a 128-row tile of the decode GEMM then holds
both and applies the activation itself, and the prompt path's activation kernel reads the same
layout.  Otherwise all gate rows come first.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, ParamSpec, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """params: ``intermediate_size``, ``activation`` (only ``"silu"``)."""

    graph_safe = True
    takes_lazy_norm = True
    adds_residual = True
    takes_stream_norm = True

    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.intermediate_size = int(spec.params["intermediate_size"])
        activation = spec.params.get("activation", "silu")
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} is not supported (only 'silu')")
        self.gate_up: torch.Tensor | None = None
        self.run = ops.GATE_UP_RUN if self.intermediate_size % ops.GATE_UP_RUN == 0 else 0
        self.down: torch.Tensor | None = None

    def param_specs(self):
        i, h = self.intermediate_size, self.hidden_size
        return {
            "gate_proj.weight": ParamSpec((i, h)),
            "up_proj.weight": ParamSpec((i, h)),
            "down_proj.weight": ParamSpec((h, i)),
        }

    def load(self, tensors):
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if self.run:
            self.gate_up = ops.interleave_gate_up(gate, up, self.run).contiguous()
        else:
            self.gate_up = torch.cat((gate, up), dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def forward(self, x, ctx, residual=None):
        status = getattr(ctx, "status", None)
        if isinstance(x, ops.StreamNorm):
            # a few decoded tokens: both products go behind the output projection that is still queued; whoever
            # comes next (the next layer's q/k/v projection, or the final norm) launches them
            if (residual is x.hidden and self.run == ops.GATE_UP_RUN and self.gate_up.shape[0] % 128 == 0
                    and ops.stream_takes(x.shape[0], self.gate_up, self.down)):
                act = torch.empty((x.shape[0], self.intermediate_size), dtype=torch.bfloat16,
                                  device=self.gate_up.device)
                x.pending.add(x.normed_phase(self.gate_up, epilogue="gated", out=act))
                x.pending.add(dict(w=self.down, x=act, epilogue="residual"))
                return x.pending
            x = x.materialize()
        act = ops.gated_linear(x, self.gate_up, self.run, status=status)
        if residual is not None:
            summed = ops.linear_into_residual(act, self.down, residual, status=status)
            if summed is not None:
                return summed
        return ops.linear(act, self.down, partial_ok=True, status=status)
