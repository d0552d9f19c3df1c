"""Host-side bookkeeping: slots of sequences and pages of tokens.

Both are plain free lists with the checks that the tests lean on: nothing is
handed out twice, nothing is freed twice, and everything handed out is either
held or free.
"""
from __future__ import annotations

from typing import Iterable, List

from .spec import CacheFull


class FreeList:
    """Integers 0..n-1; the one most recently given back is handed out first,
    so a batch that follows another one reuses its predecessor's places."""

    what = "item"

    def __init__(self, n: int):
        if n < 0:
            raise ValueError(f"cannot manage {n} {self.what}s")
        self.n = n
        self._free: List[int] = list(range(n - 1, -1, -1))
        self._held = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return len(self._held)

    def held(self):
        return sorted(self._held)

    def acquire(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n} {self.what}s are in use")
        i = self._free.pop()
        self._held.add(i)
        return i

    def acquire_many(self, k: int) -> List[int]:
        if k > len(self._free):
            raise CacheFull(f"{k} {self.what}s wanted, {len(self._free)} of {self.n} free")
        return [self.acquire() for _ in range(k)]

    def release(self, i: int) -> None:
        if i not in self._held:
            state = "already free" if 0 <= i < self.n else "unknown"
            raise ValueError(f"{self.what} {i} is {state}: it cannot be released")
        self._held.remove(i)
        self._free.append(i)

    def release_many(self, items: Iterable[int]) -> None:
        for i in items:
            self.release(i)

    def check(self) -> None:
        """Raises if an item is lost, duplicated, or both held and free."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError(f"a {self.what} is on the free list twice")
        if free & self._held:
            raise AssertionError(f"{self.what}s {sorted(free & self._held)} are held and free")
        if free | self._held != set(range(self.n)):
            raise AssertionError(f"{self.what}s {sorted(set(range(self.n)) - free - self._held)} are lost")


class SlotList(FreeList):
    what = "slot"


class PagePool(FreeList):
    what = "page"
