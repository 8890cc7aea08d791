"""The cache manager: paged keys/values per group of layers, and per-request state slots.

What the reference keeps per layer and per request (one pool and one block table for each of
36 layers, advanced in lock-step: ampere_kv/paged_cache.py:10-27, ampere_kv/scheduler.py:63-64,
:202) is kept once per *group* here.  A group is the set of schedule positions whose mixers
ask for the same kind of cache (:class:`CacheSpec`): all positions, or only a window of them.
Every group has its own page pool, one block table per request, and for every tensor its
mixers store per token (attention: ``k`` and ``v``; another mixer may name one compressed
tensor, or keys and values of different widths) a storage
``[positions in group, pages, heads, page_size, width]``; a page id means the same page for
every position and every tensor of the group.

Pages come back in two ways: all of a request's pages when it is closed, and, in a window
group, every page that lies wholly behind the window of the next query, as soon as the
request's length has moved past it.  Returned pages are reused first (LIFO).

Beside the pages each request holds one state slot: an index into fixed-size float32 state
tensors ``[max_seqs, *state_shape]`` of the positions whose mixers ask for state.  The dense
attention model asks for none; the slot is still taken and returned with the request.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..parts.base import CacheSpec
from .block_pool import IdPool, OutOfPages


@dataclass
class LayerCacheView:
    """What one schedule position's mixer sees of the cache."""

    position: int
    group: int | None          # index into CacheManager.groups / StepContext.groups
    k_cache: torch.Tensor | None    # tensors["k"] / tensors["v"] of an attention cache, else None
    v_cache: torch.Tensor | None
    page_size: int
    writes: bool               # False: the pages belong to an earlier position, only read them
    state: torch.Tensor | None  # [max_seqs, *state_shape] float32, or None
    #: every tensor the position's cache spec names: name -> [pages, heads, page_size, width]
    tensors: dict[str, torch.Tensor] = field(default_factory=dict)


@dataclass
class CacheGroup:
    index: int
    spec: CacheSpec
    positions: list[int]
    page_size: int
    pool: IdPool
    #: tensor name -> [positions, pages, heads, page_size, width], or None when storage is not allocated
    storage: dict[str, torch.Tensor] | None = None

    @property
    def window(self) -> int | None:
        return self.spec.window if self.spec.kind == "window" else None

    def bytes_per_page(self, element_size: int) -> int:
        per_token = sum(t.heads * t.width for t in self.spec.stored())
        return len(self.positions) * per_token * self.page_size * element_size


class SequenceCache:
    """One request's hold on the cache: per group a logical-to-physical page list, and a state slot."""

    def __init__(self, request_id, num_groups: int, state_slot: int):
        self.request_id = request_id
        self.length = 0                      # tokens whose keys/values are in the cache
        self.pages: list[list[int]] = [[] for _ in range(num_groups)]   # -1 where given back
        self.first_live: list[int] = [0] * num_groups
        self.state_slot = state_slot
        self.closed = False

    def held_pages(self, group: int) -> list[int]:
        return [p for p in self.pages[group] if p >= 0]


class CacheManager:
    def __init__(self, cache_specs: list[CacheSpec], cache_of: list[int | None], *, page_size: int,
                 num_pages: int | list[int], max_seqs: int, dtype: torch.dtype = torch.bfloat16,
                 device: torch.device | str = "cpu", allocate_storage: bool = True):
        """``cache_specs[i]`` / ``cache_of[i]`` describe schedule position i.  ``num_pages`` is the
        pool size of every group (or one size per group, in order of first appearance)."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_seqs = max_seqs
        self.dtype = dtype
        self.device = torch.device(device)
        self.groups: list[CacheGroup] = []
        self._position_group: list[int | None] = []
        self._position_slot: list[int | None] = []
        by_key: dict[tuple, CacheGroup] = {}
        for pos, spec in enumerate(cache_specs):
            if cache_of[pos] is not None:
                owner = cache_of[pos]
                if cache_specs[owner].group_key() != spec.group_key():
                    raise ValueError(f"schedule position {pos} reads the cache of position {owner}, "
                                     f"whose cache has another shape or kind")
                self._position_group.append(self._position_group[owner])
                self._position_slot.append(self._position_slot[owner])
                continue
            if spec.kind == "none":
                self._position_group.append(None)
                self._position_slot.append(None)
                continue
            if spec.kind not in ("full", "window"):
                raise ValueError(f"schedule position {pos}: unknown cache kind {spec.kind!r}")
            if spec.kind == "window" and (spec.window is None or spec.window <= 0):
                raise ValueError(f"schedule position {pos}: a window cache needs a positive window")
            stored = spec.stored()
            if not stored or any(t.heads <= 0 or t.width <= 0 for t in stored) or \
                    len({t.name for t in stored}) != len(stored):
                raise ValueError(f"schedule position {pos}: a paged cache stores at least one tensor per token, "
                                 f"each with a name of its own and positive sizes; got {stored}")
            key = spec.group_key()
            if key not in by_key:
                count = num_pages if isinstance(num_pages, int) else num_pages[len(self.groups)]
                group = CacheGroup(len(self.groups), spec, [], page_size, IdPool(count, "page"))
                by_key[key] = group
                self.groups.append(group)
            group = by_key[key]
            self._position_group.append(group.index)
            self._position_slot.append(len(group.positions))
            group.positions.append(pos)
        self.slots = IdPool(max_seqs, "state slot")
        self.state: list[torch.Tensor | None] = []
        for pos, spec in enumerate(cache_specs):
            if spec.state_shape and allocate_storage:
                self.state.append(torch.zeros((max_seqs, *spec.state_shape), dtype=torch.float32, device=self.device))
            else:
                self.state.append(None)
        self._state_shapes = [tuple(spec.state_shape) for spec in cache_specs]
        if allocate_storage:
            for group in self.groups:
                group.storage = {
                    t.name: torch.empty((len(group.positions), group.pool.count, t.heads, page_size, t.width),
                                        dtype=dtype, device=self.device)
                    for t in group.spec.stored()}
        self._cache_of = list(cache_of)
        self.sequences: dict[object, SequenceCache] = {}

    # ------------------------------------------------------------------ views

    def layer_view(self, position: int) -> LayerCacheView:
        g = self._position_group[position]
        state = self.state[position]
        if g is None:
            return LayerCacheView(position, None, None, None, self.page_size, False, state)
        group = self.groups[g]
        slot = self._position_slot[position]
        tensors = {}
        if group.storage is not None:
            tensors = {name: whole[slot] for name, whole in group.storage.items()}
        return LayerCacheView(position, g, tensors.get("k"), tensors.get("v"), self.page_size,
                              self._cache_of[position] is None, state, tensors)

    def layer_views(self) -> list[LayerCacheView]:
        return [self.layer_view(i) for i in range(len(self._position_group))]

    # ------------------------------------------------------------------ requests

    def open(self, request_id) -> SequenceCache:
        if request_id in self.sequences:
            raise ValueError(f"request {request_id!r} already holds a cache")
        slot = self.slots.allocate()
        for state in self.state:
            if state is not None:
                state[slot].zero_()
        seq = SequenceCache(request_id, len(self.groups), slot)
        self.sequences[request_id] = seq
        return seq

    def _pages_wanted(self, seq: SequenceCache, group: CacheGroup, new_length: int) -> int:
        """Pages to allocate so that positions [first live page, new_length) are backed."""
        have = len(seq.pages[group.index])
        need = (new_length + self.page_size - 1) // self.page_size
        return max(0, need - have)

    def pages_needed(self, seq: SequenceCache, num_tokens: int) -> list[int]:
        return [self._pages_wanted(seq, g, seq.length + num_tokens) for g in self.groups]

    def can_reserve(self, seq: SequenceCache, num_tokens: int) -> bool:
        return all(n <= g.pool.num_free for n, g in zip(self.pages_needed(seq, num_tokens), self.groups))

    def reserve(self, seq: SequenceCache, num_tokens: int) -> None:
        """Back positions [length, length + num_tokens) with pages in every group, all or nothing."""
        if seq.closed:
            raise ValueError(f"request {seq.request_id!r} is closed")
        needs = self.pages_needed(seq, num_tokens)
        for n, g in zip(needs, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(f"group {g.index} ({g.spec.kind}): {n} pages wanted for request "
                                 f"{seq.request_id!r}, {g.pool.num_free} free of {g.pool.count}")
        for n, g in zip(needs, self.groups):
            seq.pages[g.index].extend(g.pool.allocate_many(n))

    def commit(self, seq: SequenceCache, num_tokens: int) -> None:
        """The step wrote ``num_tokens`` more positions.  Pages wholly behind every window are given back."""
        seq.length += num_tokens
        for g in self.groups:
            if g.window is None:
                continue
            # the next query is at position >= length and sees keys > position - window
            first_needed_key = seq.length - g.window + 1
            releasable = max(0, first_needed_key) // self.page_size
            pages = seq.pages[g.index]
            for logical in range(seq.first_live[g.index], min(releasable, len(pages))):
                if pages[logical] >= 0:
                    g.pool.free(pages[logical])
                    pages[logical] = -1
            seq.first_live[g.index] = max(seq.first_live[g.index], min(releasable, len(pages)))

    def release_unused(self, seq: SequenceCache) -> None:
        """Give back pages that were reserved beyond the committed length (a step that did not run)."""
        keep = (seq.length + self.page_size - 1) // self.page_size
        for g in self.groups:
            pages = seq.pages[g.index]
            while len(pages) > keep:
                page = pages.pop()
                if page >= 0:
                    g.pool.free(page)

    def close(self, seq: SequenceCache) -> None:
        """Give back everything the request holds.  Closing twice is an error."""
        if seq.closed:
            raise ValueError(f"request {seq.request_id!r} was closed before")
        for g in self.groups:
            for page in seq.pages[g.index]:
                if page >= 0:
                    g.pool.free(page)
            seq.pages[g.index] = []
        self.slots.free(seq.state_slot)
        seq.closed = True
        seq.length = 0
        del self.sequences[seq.request_id]

    # ------------------------------------------------------------------ for the batch builder

    def slot_of(self, seq: SequenceCache, group: int, position: int) -> int:
        page = seq.pages[group][position // self.page_size]
        if page < 0:
            raise ValueError(f"request {seq.request_id!r}: position {position} lies in a page that was given back")
        return page * self.page_size + position % self.page_size

    def table_row(self, seq: SequenceCache, group: int) -> list[int]:
        return seq.pages[group]

    # ------------------------------------------------------------------ accounting

    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.groups]

    def pages_to_start(self, num_tokens: int) -> list[int]:
        """Pages per group that a request without a cache yet needs for its first ``num_tokens`` positions."""
        return [(num_tokens + g.page_size - 1) // g.page_size for g in self.groups]

    def pages_for_tokens(self, num_tokens: int, chunk: int = 0) -> list[int]:
        """Upper bound of pages per group a request of ``num_tokens`` positions holds at any time,
        when it is fed at most ``chunk`` tokens a step (0 = any)."""
        out = []
        full = (num_tokens + self.page_size - 1) // self.page_size
        for g in self.groups:
            if g.window is None or chunk <= 0:
                out.append(full)
            else:
                span = g.window + chunk + self.page_size  # window behind, the step's tokens, a partial page
                out.append(min(full, (span + self.page_size - 1) // self.page_size + 1))
        return out

    def check_invariants(self) -> None:
        """Every page is free or held by exactly one live request; raises AssertionError otherwise."""
        for g in self.groups:
            owners: dict[int, object] = {}
            for seq in self.sequences.values():
                for page in seq.held_pages(g.index):
                    assert 0 <= page < g.pool.count, f"group {g.index}: page {page} out of range"
                    assert page not in owners, (f"group {g.index}: page {page} held by {owners[page]!r} "
                                                f"and {seq.request_id!r}")
                    assert g.pool.is_held(page), f"group {g.index}: page {page} in a table but free in the pool"
                    owners[page] = seq.request_id
            assert len(owners) == g.pool.num_held, (f"group {g.index}: {g.pool.num_held} pages taken from the pool, "
                                                    f"{len(owners)} found in block tables (a page was lost)")
        slots = [seq.state_slot for seq in self.sequences.values()]
        assert len(set(slots)) == len(slots), "a state slot is held twice"
        assert len(slots) == self.slots.num_held, "a state slot was lost"
