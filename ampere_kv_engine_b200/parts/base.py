"""Interfaces and registries of the parts a model is put together from.

A part is built from a :class:`~ampere_kv_engine_b200.config.spec.PartSpec` (its kind and
its sizes and constants), declares the tensors it wants by local name, receives them, and
computes on the flat token batch of one step.  Parts never look at a model configuration
and do not know which architecture uses them; the reference, by contrast, wires one model's
attribute paths into every function (ampere_kv/runner.py:60-77, 102-179).

Kinds are looked up in seven registries (mixers, feed-forwards, norms, position encodings,
blocks, embeddings, heads).  Registering a new kind is one decorator call and needs no change
here.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import torch

from ..config.spec import LayerSpec, PartSpec
from ..kernels import ops


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part wants from the checkpoint.

    ``kind``: ``"matrix"`` and ``"bias"`` (kept in the compute dtype), ``"vector"`` (norm
    weights: always float32 on the device, an exact widening of what is stored; a tensor
    stored in 32-bit stays 32-bit) or ``"table"`` (integer tables, int32).  ``init`` names the random draw of the random-weights mode.
    """

    shape: tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"        # "normal": N(0, 0.02); "norm": 1 + N(0, 0.1); "zeros"
    optional: bool = False


@dataclass(frozen=True)
class CacheTensor:
    """One thing a token leaves in a paged cache: ``heads`` rows of ``width`` elements."""

    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer needs the cache manager to keep for each request.

    ``kind``: ``"none"``, ``"full"`` (every position is kept) or ``"window"`` (only the last
    ``window`` positions are ever read, pages behind it are given back).  What a position stores
    is a tuple of named tensors (``tensors``); when none is given it is what attention stores:
    ``k`` and ``v``, each ``num_kv_heads`` rows of ``head_dim``.  A mixer that keeps one
    compressed tensor per token, or keys and values of different widths, names them itself.
    ``state_shape`` asks for a fixed-size float32 state per request (``()`` = none).
    Mixers whose specs are equal share a cache group: one page pool, one block table per
    request.
    """

    kind: str = "none"
    num_kv_heads: int = 0
    head_dim: int = 0
    window: int | None = None
    state_shape: tuple[int, ...] = ()
    tensors: tuple[CacheTensor, ...] | None = None

    def stored(self) -> tuple[CacheTensor, ...]:
        if self.kind == "none":
            return ()
        if self.tensors is not None:
            return tuple(self.tensors)
        return (CacheTensor("k", self.num_kv_heads, self.head_dim), CacheTensor("v", self.num_kv_heads, self.head_dim))

    def group_key(self) -> tuple:
        return (self.kind, self.stored(), self.window)


class Part:
    """Common life cycle: build from a spec, declare tensors, load them."""

    #: True when ``forward`` only enqueues device work whose shapes depend on the batch layout alone (no host
    #: loops over sequences, no host reads), so a decode step through it can be replayed as a CUDA graph.
    graph_safe = False

    def __init__(self, spec: PartSpec, *, hidden_size: int, dtype: torch.dtype, device: torch.device):
        self.spec = spec
        self.hidden_size = hidden_size
        self.dtype = dtype
        self.device = device

    def param_specs(self) -> dict[str, ParamSpec]:
        """Tensors wanted, by name relative to ``spec.prefix``."""
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receive the tensors of :meth:`param_specs` (already on the device, cast per kind)."""

    def children(self) -> tuple["Part", ...]:
        """Parts this part built for itself (a mixer's position encoding): the model asks them for tensors and for
        ``graph_safe`` as it asks the part itself."""
        return ()


class Norm(Part):
    def forward(self, hidden: torch.Tensor, delta: torch.Tensor | None, ctx, rows: torch.Tensor | None = None
                ) -> torch.Tensor:
        """Add ``delta`` into the float32 residual stream ``hidden`` (in place) and return the
        normalised activations in the compute dtype.  With ``rows`` only those rows are
        normalised and ``hidden`` is not changed.  ``delta`` is a branch output [tokens, hidden]
        in the compute dtype, or a 3-D float32 stack [parts, tokens, hidden] of partial sums
        (a split-K product) that are to be added together."""
        raise NotImplementedError

    #: True when ``forward`` takes an ``ops.PendingPhases`` as ``delta`` with ``lazy=True`` and answers with an
    #: ``ops.StreamNorm`` (or None if it cannot): the chained-product kernel then applies the norm
    takes_pending = False

    #: True when ``forward`` also takes a ``Summed`` as ``delta`` (the branch's product kernel has already added
    #: its result to ``hidden`` and left the sums of squares) and a keyword ``lazy``: with ``lazy=True`` it may
    #: return a ``LazyNorm`` for a consumer with ``takes_lazy_norm``.  A norm without it is handed ``delta=None``
    #: in that case, which means the same thing.
    takes_summed = False


class PositionEncoding(Part):
    """How positions enter a mixer.  ``fused_rotary()`` returns ``(inv_freq, rotary_dim)`` when
    the fused q/k kernel can apply the encoding itself (a rotate-half rotation, or nothing:
    ``(None, 0)``), else None; then :meth:`apply` is called on dense q and k
    ([tokens, heads * head_dim]) before k is written to the cache."""

    def fused_rotary(self) -> tuple[torch.Tensor, int] | None:
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        return q, k


class Mixer(Part):
    #: ``forward`` accepts a ``LazyNorm`` as ``x`` (it hands it to ``ops.linear`` / ``ops.project_qkv``, which let
    #: the small-batch product kernel apply the norm).
    takes_lazy_norm = False
    #: ``forward`` accepts a keyword ``residual`` (the float32 residual stream): it may then add its output there
    #: itself and return a ``Summed`` instead of the output, or queue the product that adds it and return the
    #: ``PendingPhases``.
    adds_residual = False
    #: ``forward`` accepts an ``ops.StreamNorm`` as ``x``: it queues its first product behind the products that are
    #: pending there and launches them together
    takes_stream_norm = False

    def cache_spec(self) -> CacheSpec:
        return CacheSpec()

    def preferred_q_tile(self) -> int | None:
        """Query tokens per attention tile this mixer's kernels like best (None: no preference).  The batch layout
        cuts prompt portions into tiles of one size for the whole model: the one all mixers agree on, else the
        default."""
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        """x: [tokens, hidden] in the compute dtype; ``ctx`` is the step's batch
        (:class:`~ampere_kv_engine_b200.engine.batch.StepContext`); ``cache`` is this schedule
        position's :class:`~ampere_kv_engine_b200.cache.manager.LayerCacheView`."""
        raise NotImplementedError


class FeedForward(Part):
    takes_lazy_norm = False     # as for Mixer
    adds_residual = False
    takes_stream_norm = False

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Embedding(Part):
    """Token ids to the float32 residual stream."""

    def forward(self, token_ids: torch.Tensor, ctx) -> torch.Tensor:
        """[tokens] int32 -> [tokens, hidden] float32.  ``ctx.sampled`` may stand for ids the host has not read."""
        raise NotImplementedError


class Head(Part):
    """Normalised activations of the wanted rows to float32 logits."""

    def tie(self, embedding: Embedding) -> None:
        """Called once all tensors are loaded: a head that shares the embedding's matrix takes it here."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """Arrangement of one layer's parts around the residual stream.

    A block kind is built from the layer's spec and builds its own parts from the roles it knows
    (:meth:`build_role`), so how many norms or branches a layer has is the block's business.  The model needs three
    things of it: :meth:`parts` (whose tensors to load), :meth:`cache_spec` (what the layer keeps per request: one
    cache view per schedule position) and :meth:`forward`.
    """

    #: registry of each role this base class knows; a block kind with other roles extends it
    ROLE_REGISTRIES: dict[str, "Registry"] = {}

    def __init__(self, layer: LayerSpec, *, hidden_size: int, dtype: torch.dtype, device: torch.device):
        self.layer = layer
        self.hidden_size, self.dtype, self.device = hidden_size, dtype, device
        self._built: list[Part] = []

    def build_role(self, role: str, registry: "Registry | None" = None) -> Part:
        """Build the part the layer spec names for ``role`` and remember it."""
        registry = registry or self.ROLE_REGISTRIES.get(role)
        if registry is None:
            raise ValueError(f"block kind {self.layer.block!r}: no registry is known for role {role!r}")
        part = build_part(registry, self.layer.role(role), hidden_size=self.hidden_size, dtype=self.dtype,
                          device=self.device)
        self._built.append(part)
        return part

    def parts(self) -> list[Part]:
        return list(self._built)

    def cache_spec(self) -> CacheSpec:
        """What this layer keeps per request: its mixer's needs (a layer without a mixer keeps nothing)."""
        mixer = getattr(self, "mixer", None)
        return mixer.cache_spec() if mixer is not None else CacheSpec()

    def forward(self, hidden: torch.Tensor, delta: torch.Tensor | None, ctx, cache
                ) -> tuple[torch.Tensor, torch.Tensor | None]:
        """Takes the residual stream and a not-yet-added branch output; returns the same pair.  The branch output
        may be a ``Summed``: already added by the kernel that made it."""
        raise NotImplementedError

    @staticmethod
    def run_norm(norm: Norm, hidden, delta, ctx, consumer=None, rows=None):
        """``norm`` over ``hidden`` (+ ``delta``), lazily if ``delta`` is a ``Summed`` and both the norm and the
        consumer of its result know how."""
        if isinstance(delta, ops.PendingPhases):
            # products still queued for the chained-product kernel: a norm that knows how hands its consumer the
            # not-yet-computed norm (the consumer queues its own product behind them); otherwise they run now
            if rows is None and getattr(norm, "takes_pending", False) and getattr(consumer, "takes_stream_norm", False):
                lazy = norm.forward(hidden, delta, ctx, rows=None, lazy=True)
                if lazy is not None:
                    return lazy
            delta.launch()
            return norm.forward(hidden, None, ctx, rows=rows)
        if isinstance(delta, ops.Summed):
            if not norm.takes_summed:
                return norm.forward(hidden, None, ctx, rows=rows)
            return norm.forward(hidden, delta, ctx, rows=rows, lazy=bool(getattr(consumer, "takes_lazy_norm", False)))
        return norm.forward(hidden, delta, ctx, rows=rows)

    @staticmethod
    def run_branch(part, hidden, *args):
        """``part.forward(*args)``, with the residual stream offered to a part that can add to it itself."""
        if part.adds_residual:
            return part.forward(*args, residual=hidden)
        return part.forward(*args)


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: dict[str, Callable[..., Any]] = {}

    def register(self, kind: str):
        def wrap(cls):
            if kind in self._kinds and self._kinds[kind] is not cls:
                raise ValueError(f"{self.what} kind {kind!r} is already registered")
            self._kinds[kind] = cls
            return cls
        return wrap

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str):
        if kind not in self._kinds:
            raise KeyError(f"unknown {self.what} kind {kind!r}; registered: {sorted(self._kinds)}")
        return self._kinds[kind]

    def kinds(self) -> list[str]:
        return sorted(self._kinds)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
Block.ROLE_REGISTRIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "mixer_norm": NORMS,
                         "feed_forward_norm": NORMS}

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_block = BLOCKS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register


def build_part(registry: Registry, spec: PartSpec, *, hidden_size: int, dtype: torch.dtype,
               device: torch.device):
    return registry.get(spec.kind)(spec, hidden_size=hidden_size, dtype=dtype, device=device)
