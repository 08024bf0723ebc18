"""Bookkeeping of pages and slots: plain host code, no device needed."""
from __future__ import annotations

from typing import List


class CacheError(RuntimeError):
    """Misuse or exhaustion of the cache (a slot freed twice, no page left, ...)."""


class FreeList:
    """Ids 0..n-1, each either free or held; lowest free id first, so reuse is immediate."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._held = [False] * n
        self._free: List[int] = list(range(n - 1, -1, -1))     # pop() yields the lowest id

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what} left (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give_back(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (there are {self.n})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is given back but not held (freed twice?)")
        self._held[i] = False
        self._free.append(i)
        if len(self._free) > 1 and self._free[-2] < i:
            self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)
