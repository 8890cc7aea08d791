"""A decoder assembled from a :class:`ModelSpec`: embedding, layers run in the schedule's order,
final norm and head on the rows whose logits are wanted.

This is the one forward pass of the package (the reference has three, one per batch shape:
ampere_kv/runner.py:219-290).  It runs exactly the tokens of the step's batch, reads earlier
tokens only through the cache, and returns float32 logits for ``ctx.logit_rows``
(the reference returns the last position only, runner.py:293-297).
"""

from __future__ import annotations

import torch

from ..config.spec import ModelSpec
from ..kernels import ops
from ..parts import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (register the built-in kinds)
from ..parts.base import BLOCKS, EMBEDDINGS, HEADS, NORMS, Block, CacheSpec, ParamSpec, build_part


class DecoderModel:
    def __init__(self, spec: ModelSpec, *, dtype: torch.dtype, device: torch.device | str):
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        kw = dict(hidden_size=spec.hidden_size, dtype=dtype, device=self.device)
        self.embedding = build_part(EMBEDDINGS, spec.embedding, **kw)
        self.blocks = [BLOCKS.get(layer.block)(layer, **kw) for layer in spec.layers]
        self.final_norm = build_part(NORMS, spec.final_norm, **kw)
        self.head = build_part(HEADS, spec.head, **kw)
        self.loaded = False

    # ------------------------------------------------------------------ tensors

    def _parts(self):
        """Every part, a part's own children after it."""
        def walk(part):
            yield part
            for child in part.children():
                yield from walk(child)
        yield from walk(self.embedding)
        for blk in self.blocks:
            for part in blk.parts():
                yield from walk(part)
        yield from walk(self.final_norm)
        yield from walk(self.head)

    def param_specs(self) -> dict[str, ParamSpec]:
        """Every tensor of the checkpoint by its full name."""
        out: dict[str, ParamSpec] = {}
        for part in self._parts():
            for local, ps in part.param_specs().items():
                name = f"{part.spec.prefix}.{local}" if part.spec.prefix else local
                if name in out and out[name] != ps:
                    raise ValueError(f"tensor {name} is declared twice with different shapes")
                out[name] = ps
        return out

    def load_tensors(self, tensors: dict[str, torch.Tensor]) -> None:
        """``tensors``: full name -> tensor, already validated, cast and on the device."""
        for part in self._parts():
            local = {}
            for name in part.param_specs():
                full = f"{part.spec.prefix}.{name}" if part.spec.prefix else name
                if full in tensors:
                    local[name] = tensors[full]
            part.load(local)
        self.head.tie(self.embedding)
        self.loaded = True

    @property
    def graph_safe(self) -> bool:
        """Every part only enqueues device work that depends on the batch layout alone."""
        return all(getattr(part, "graph_safe", False) for part in self._parts())

    # ------------------------------------------------------------------ cache needs

    def cache_specs(self) -> list[CacheSpec]:
        """One per schedule position."""
        return [self.blocks[e.layer].cache_spec() for e in self.spec.schedule]

    def q_tile(self) -> int:
        """Query tokens per attention tile of the batch layout: what every mixer with a preference asks for, if they
        agree."""
        wishes = {m.preferred_q_tile() for blk in self.blocks for m in [getattr(blk, "mixer", None)]
                  if m is not None and m.preferred_q_tile() is not None}
        return wishes.pop() if len(wishes) == 1 else ops.ATTENTION_Q_TILE

    def cache_of(self) -> list[int | None]:
        return [e.cache_of for e in self.spec.schedule]

    # ------------------------------------------------------------------ forward

    @torch.no_grad()
    def forward(self, ctx, cache_views) -> torch.Tensor | None:
        """Run the step's tokens through the schedule; logits [wanted, vocab] float32, or None if none wanted."""
        ops.stream_begin_step(self.device)
        hidden = self.embedding.forward(ctx.token_ids, ctx)
        delta = None
        for pos, entry in enumerate(self.spec.schedule):
            hidden, delta = self.blocks[entry.layer].forward(hidden, delta, ctx, cache_views[pos])
        if ctx.num_logit_rows == 0:
            return None
        normed = Block.run_norm(self.final_norm, hidden, delta, ctx, rows=ctx.logit_rows)
        return self.head.forward(normed)
