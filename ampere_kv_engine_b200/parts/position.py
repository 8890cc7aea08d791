"""Position encodings.

``rope``: rotate-half rotary embedding over the first ``rotary_dim`` dims of every head
(the whole head for Qwen3).  ``inv_freq[j] = 1 / theta^(2j / rotary_dim)`` is computed once
in float32 on the host from an int64 ``arange`` exactly as the reference does
(ampere_kv/runner.py:41-44); angles ``position * inv_freq`` and their cos/sin are float32
in the kernel (runner.py:86-93).  ``none``: positions do not enter the mixer.
"""

from __future__ import annotations

import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope")
class RotaryEmbedding(PositionEncoding):
    """params: ``theta``, ``rotary_dim``."""

    graph_safe = True


    def __init__(self, spec, **kw):
        super().__init__(spec, **kw)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rope: rotary_dim must be a positive even number, got {self.rotary_dim}")
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.int64).float() / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(self.device)

    def fused_rotary(self):
        return self.inv_freq, self.rotary_dim


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    graph_safe = True
    def fused_rotary(self):
        return None, 0
