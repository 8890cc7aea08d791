"""Arrangements of a layer's parts around the residual stream.

``prenorm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))`` (ampere_kv/runner.py:117-121
and 156-179).  The residual stream is float32; each branch output is handed to the next norm
as a pending ``delta`` so that the sum and the norm are one kernel.
"""

from __future__ import annotations

from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def forward(self, hidden, delta, ctx, cache):
        x = self.mixer_norm.forward(hidden, delta, ctx)
        attn = self.mixer.forward(x, ctx, cache)
        x = self.feed_forward_norm.forward(hidden, attn, ctx)
        return hidden, self.feed_forward.forward(x, ctx)
