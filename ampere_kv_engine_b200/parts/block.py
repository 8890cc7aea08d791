"""Arrangements of a layer's parts around the residual stream.

``prenorm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))`` (ampere_kv/runner.py:117-121
and 156-179).  The residual stream is float32; each branch output is handed to the next norm
as a pending ``delta`` so that the sum and the norm are one kernel.  On decode steps the branch's
last product may add to the stream itself and the next product apply the norm (``Summed``,
``LazyNorm``): then no kernel stands between the two products.
"""

from __future__ import annotations

from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    """roles: ``mixer_norm``, ``mixer``, ``feed_forward_norm``, ``feed_forward``."""

    def __init__(self, layer, **kw):
        super().__init__(layer, **kw)
        self.mixer_norm = self.build_role("mixer_norm")
        self.mixer = self.build_role("mixer")
        self.feed_forward_norm = self.build_role("feed_forward_norm")
        self.feed_forward = self.build_role("feed_forward")

    def forward(self, hidden, delta, ctx, cache):
        x = self.run_norm(self.mixer_norm, hidden, delta, ctx, consumer=self.mixer)
        attn = self.run_branch(self.mixer, hidden, x, ctx, cache)
        x = self.run_norm(self.feed_forward_norm, hidden, attn, ctx, consumer=self.feed_forward)
        return hidden, self.run_branch(self.feed_forward, hidden, x, ctx)
