"""What a model is made of, as data.

An architecture turns its typed configuration into a :class:`ModelSpec`: for every layer
which mixer, feed-forward, norm and block arrangement it uses (each a :class:`PartSpec`:
a registered kind plus its sizes and constants), the checkpoint-name prefixes of its
tensors, and the order in which layers run.  Nothing below this file knows which model
the parts belong to.

The reference hard-wires one arrangement (ampere_kv/runner.py:102-179: pre-norm,
attention, residual, pre-norm, SiLU-gated MLP, residual) and one order (runner.py:284).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class PartSpec:
    """A registered part kind and the parameters it is built with."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    #: checkpoint-name prefix of this part's tensors ("" for parts without tensors)
    prefix: str = ""

    def with_prefix(self, prefix: str) -> "PartSpec":
        return PartSpec(self.kind, dict(self.params), prefix)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: how its parts are arranged (``block``, a registered block kind) and which parts they are.

    The block kind decides which roles it has and builds each from the spec under that role's name.  The four
    roles of a two-branch layer (a mixer and a feed-forward, a norm before each) have fields of their own;
    a block with other roles (more norms, one norm shared by parallel branches, no feed-forward at all) finds
    them in ``parts``, and its own constants in ``params``.
    """

    block: str
    mixer: PartSpec | None = None
    feed_forward: PartSpec | None = None
    mixer_norm: PartSpec | None = None
    feed_forward_norm: PartSpec | None = None
    parts: dict[str, PartSpec] = field(default_factory=dict)
    params: dict[str, Any] = field(default_factory=dict)

    def roles(self) -> dict[str, PartSpec]:
        """Every part of the layer by role name."""
        out = {name: getattr(self, name) for name in ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")
               if getattr(self, name) is not None}
        for name, spec in self.parts.items():
            if name in out:
                raise ValueError(f"layer spec: role {name!r} is given twice")
            out[name] = spec
        return out

    def role(self, name: str) -> PartSpec:
        roles = self.roles()
        if name not in roles:
            raise ValueError(f"layer spec: block kind {self.block!r} needs a part in role {name!r}; "
                             f"the layer has {sorted(roles)}")
        return roles[name]


@dataclass(frozen=True)
class ScheduleEntry:
    """One position in the run order.

    ``layer`` indexes :attr:`ModelSpec.layers` (a layer may appear more than once: its
    weights are shared, each appearance has a cache of its own unless ``cache_of`` says
    otherwise).  ``cache_of`` names an earlier position of the schedule whose cache this
    position reads instead of writing one of its own.
    """

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    max_position: int
    eos_token_ids: tuple[int, ...] = ()

    def validate(self) -> None:
        if not self.schedule:
            raise ValueError("model spec: the schedule is empty")
        for pos, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"model spec: schedule position {pos} names layer {entry.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < pos:
                    raise ValueError(f"model spec: schedule position {pos} reads the cache of position "
                                     f"{entry.cache_of}, which is not an earlier position")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ValueError(f"model spec: schedule position {pos} reads the cache of position "
                                     f"{entry.cache_of}, which itself borrows a cache")
