"""Host-side bookkeeping of the cache: which pages and which sequence slots are in use.

Pure Python, no device memory: the invariants (no page lost, held twice or freed twice; no
slot given out twice) are checked here and tested without a GPU.
"""
from __future__ import annotations

import heapq
from typing import Dict, List


class CacheFull(RuntimeError):
    """More tokens were asked for than the cache was sized for."""


class CacheError(RuntimeError):
    """Misuse of the cache: a page or slot freed twice, an unknown slot, and the like."""


class IdPool:
    """Integer ids 0 .. capacity-1, handed out lowest first and taken back."""

    def __init__(self, capacity: int, what: str):
        if capacity < 0:
            raise ValueError(f"{what} capacity must be >= 0, got {capacity}")
        self.capacity = capacity
        self.what = what
        self._free: List[int] = list(range(capacity))
        heapq.heapify(self._free)
        self._held = [False] * capacity

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.capacity - len(self._free)

    def take(self, n: int = 1) -> List[int]:
        if n < 0:
            raise ValueError("cannot take a negative number of ids")
        if n > len(self._free):
            raise CacheFull(f"{n} more {self.what}(s) needed but only {len(self._free)} of {self.capacity} are free")
        out = [heapq.heappop(self._free) for _ in range(n)]
        for i in out:
            if self._held[i]:
                raise CacheError(f"{self.what} {i} was in the free list while held")  # never expected
            self._held[i] = True
        return out

    def give_back(self, ids) -> None:
        ids = list(ids)
        for i in ids:
            if not (0 <= i < self.capacity):
                raise CacheError(f"{self.what} {i} is outside 0..{self.capacity - 1}")
            if not self._held[i]:
                raise CacheError(f"{self.what} {i} is freed twice (or was never given out)")
        if len(set(ids)) != len(ids):
            raise CacheError(f"a {self.what} is named twice in one release: {ids}")
        for i in ids:
            self._held[i] = False
            heapq.heappush(self._free, i)

    def check(self) -> None:
        """Every id is either free or held, exactly once."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise CacheError(f"a {self.what} is twice in the free list")
        held = [i for i, h in enumerate(self._held) if h]
        if sorted(free + held) != list(range(self.capacity)):
            raise CacheError(f"{self.what} ids are lost or duplicated: free={free} held={held}")


class SequenceRecord:
    """What one live sequence holds: its length and, for each storage group, its pages.
    ``pages[g][i]`` holds positions [page_size*i, page_size*(i+1)); -1 marks a page that a
    window group has already released."""
    __slots__ = ("length", "pages")

    def __init__(self, n_groups: int):
        self.length = 0
        self.pages: List[List[int]] = [[] for _ in range(n_groups)]
