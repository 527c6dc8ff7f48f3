"""Host-side bookkeeping of the cache: which slots and which pages are free.

Pure Python with no device calls, so its invariants are tested on the CPU: a slot or page is
never handed out twice, never lost, and never freed twice.
"""
from __future__ import annotations

from typing import List


class CacheFull(RuntimeError):
    """No free slot, or not enough free pages, for what was asked."""


class FreeList:
    """Hands out the integers 0..n-1, lowest first; takes them back for reuse."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))   # pop() gives the lowest
        self._held = [False] * n

    def available(self) -> int:
        return len(self._free)

    def held(self) -> int:
        return self.n - len(self._free)

    def take(self, count: int = 1) -> List[int]:
        if count < 0:
            raise ValueError("negative count")
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}s asked for, {len(self._free)} of {self.n} free")
        out = []
        for _ in range(count):
            i = self._free.pop()
            self._held[i] = True
            out.append(i)
        return out

    def give_back(self, items) -> None:
        items = list(items)
        for i in items:
            if not 0 <= i < self.n:
                raise ValueError(f"{self.what} {i} does not exist")
            if not self._held[i]:
                raise ValueError(f"{self.what} {i} is freed twice (or was never held)")
        if len(set(items)) != len(items):
            raise ValueError(f"a {self.what} is named twice in one release")
        for i in items:
            self._held[i] = False
        self._free.extend(items)
        self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]
