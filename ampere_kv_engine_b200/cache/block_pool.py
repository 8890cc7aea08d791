"""Id pools: cache pages and per-request state slots.

Same contract as the reference's allocator (ampere_kv/block_pool.py:4-35): a LIFO free
stack that first hands out 0, 1, 2, ... and reuses returned ids first; returning an id that
is not held is an error; an empty pool raises instead of growing.  Only ids are managed
here, never tensors.
"""

from __future__ import annotations


class OutOfPages(RuntimeError):
    """The pool has fewer free ids than were asked for; nothing was taken."""


class IdPool:
    def __init__(self, count: int, what: str = "page"):
        if count < 0:
            raise ValueError(f"{what} pool: count must not be negative")
        self.what = what
        self.count = count
        self._free = list(range(count - 1, -1, -1))
        self._held = [False] * count

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.count - len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages(f"{self.what} pool is empty ({self.count} in all)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def allocate_many(self, n: int) -> list[int]:
        """All or nothing."""
        if n > len(self._free):
            raise OutOfPages(f"{self.what} pool: {n} wanted, {len(self._free)} free of {self.count}")
        return [self.allocate() for _ in range(n)]

    def free(self, i: int) -> None:
        if not isinstance(i, int) or not 0 <= i < self.count:
            raise ValueError(f"{self.what} pool: id {i!r} is outside [0, {self.count})")
        if not self._held[i]:
            raise ValueError(f"{self.what} pool: id {i} is not held (freed twice, or never allocated)")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return self._held[i]
