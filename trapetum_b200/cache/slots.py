"""Bookkeeping of the cache: which slots and which pages are in use.

Plain Python, no tensors, so it can be tested anywhere.  A *slot* belongs to one
sequence from its first token to its end; a *page* holds the keys and values of
``PAGE_ROWS`` consecutive tokens.  Both come from pools that hand out the lowest
free number first and refuse to free what is not held, so a lost, doubled or
twice-freed slot shows up as an error at once.  The reference has one flat
cache per layer for its single sequence (runtime/src/lib.rs:4475) and nothing
to hand out.
"""
from __future__ import annotations

import heapq
from typing import List


class CacheError(RuntimeError):
    """Misuse of the cache's bookkeeping (double free, unknown slot...)."""


class CacheFull(CacheError):
    """Not enough free slots or pages for what was asked."""


class Pool:
    """Numbers 0..capacity-1, each either free or held."""

    def __init__(self, capacity: int, what: str):
        if capacity < 0:
            raise ValueError(f"{what} pool: capacity {capacity}")
        self.capacity = capacity
        self.what = what
        self._free: List[int] = list(range(capacity))
        heapq.heapify(self._free)
        self._held = set()

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return len(self._held)

    def take(self, n: int = 1) -> List[int]:
        if n > len(self._free):
            raise CacheFull(f"{self.what} pool: {n} asked, {len(self._free)} of {self.capacity} free")
        out = [heapq.heappop(self._free) for _ in range(n)]
        self._held.update(out)
        return out

    def give_back(self, ids) -> None:
        ids = list(ids)
        for i in ids:
            if i not in self._held:
                raise CacheError(f"{self.what} pool: {i} is not held (freed twice, or never taken)")
        if len(set(ids)) != len(ids):
            raise CacheError(f"{self.what} pool: a number is given back twice in one call: {ids}")
        for i in ids:
            self._held.remove(i)
            heapq.heappush(self._free, i)

    def is_held(self, i: int) -> bool:
        return i in self._held

    def check(self) -> None:
        """Every number is either free or held, exactly once."""
        free = sorted(self._free)
        if len(set(free)) != len(free) or set(free) & self._held or len(free) + len(self._held) != self.capacity:
            raise CacheError(f"{self.what} pool is inconsistent: {len(free)} free, {len(self._held)} held, "
                             f"capacity {self.capacity}")
