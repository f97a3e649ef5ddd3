"""Host-side bookkeeping of the cache: which slots and which pages are held by whom.

A *slot* is a live sequence's row (of the block tables, of the length table, of
the per-sequence state).  A *page* holds ``page_size`` consecutive positions of
one sequence for every layer of one group.  Both allocators refuse to give out
what is held and to take back what is free, so that a slot or page is never
lost, held twice or freed twice.
"""
from __future__ import annotations

from typing import List


class CacheFull(RuntimeError):
    """The cache cannot hold what was asked; nothing was taken."""


class FreeList:
    """Ids 0..n-1, handed out lowest-first, checked on both ways."""

    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free: List[int] = list(range(self.n - 1, -1, -1))   # pop() gives the lowest id
        self._held = [False] * self.n

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.n - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def take(self, count: int) -> List[int]:
        if count < 0:
            raise ValueError(f"cannot take {count} {self.what}s")
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}(s) wanted, {len(self._free)} of {self.n} free")
        out = [self._free.pop() for _ in range(count)]
        for i in out:
            assert not self._held[i], f"{self.what} {i} was on the free list while held"
            self._held[i] = True
        return out

    def give(self, ids) -> None:
        ids = list(ids)
        for i in ids:
            if not (0 <= i < self.n):
                raise ValueError(f"{self.what} {i} does not exist (0..{self.n - 1})")
            if not self._held[i]:
                raise ValueError(f"{self.what} {i} is given back but is not held")
        if len(set(ids)) != len(ids):
            raise ValueError(f"a {self.what} is given back twice in one call: {ids}")
        for i in ids:
            self._held[i] = False
        # keep lowest-first order of hand-out
        self._free.extend(ids)
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Every id is either free once or held, never both, never neither."""
        free = set(self._free)
        assert len(free) == len(self._free), f"a {self.what} is on the free list twice"
        for i in range(self.n):
            assert self._held[i] != (i in free), f"{self.what} {i} is lost or doubled"
