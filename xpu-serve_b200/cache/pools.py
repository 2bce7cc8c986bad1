"""Host-side accounting of slots and pages: nothing is lost, held twice or freed twice.

A slot is one sequence's place in the cache; a page is storage for `page_size`
positions of keys and values. Both pools hand out the lowest free index first, so a
finished batch's slots and pages are the first to be used again.
"""
from __future__ import annotations

import heapq
from typing import Iterable, List


class CacheError(RuntimeError):
    """The cache was asked for something it cannot do; nothing was changed."""


class CacheFull(CacheError):
    """Not enough free slots or pages; nothing was changed."""


class IndexPool:
    """`count` indices, each either free or held."""

    def __init__(self, count: int, what: str):
        if count < 0:
            raise ValueError(f"a pool of {count} {what}s")
        self.count = count
        self.what = what
        self._free: List[int] = list(range(count))
        heapq.heapify(self._free)
        self._held = [False] * count

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.count - len(self._free)

    def is_held(self, index: int) -> bool:
        return 0 <= index < self.count and self._held[index]

    def take(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError(f"cannot take {n} {self.what}s")
        if n > len(self._free):
            raise CacheFull(f"{n} {self.what}s wanted, {len(self._free)} of {self.count} free")
        out = [heapq.heappop(self._free) for _ in range(n)]
        for i in out:
            self._held[i] = True
        return out

    def give_back(self, indices: Iterable[int]) -> None:
        indices = list(indices)
        seen = set()
        for i in indices:                       # check everything before changing anything
            if not 0 <= i < self.count:
                raise CacheError(f"{self.what} {i} does not exist (0..{self.count - 1})")
            if not self._held[i] or i in seen:
                raise CacheError(f"{self.what} {i} is freed twice or was never held")
            seen.add(i)
        for i in indices:
            self._held[i] = False
            heapq.heappush(self._free, i)

    def check(self) -> None:
        """Every index is free exactly once or held, never both."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise CacheError(f"a {self.what} is in the free list twice")
        for i in range(self.count):
            if self._held[i] == (i in set(free)):
                raise CacheError(f"{self.what} {i} is {'held and free' if self._held[i] else 'lost'}")
