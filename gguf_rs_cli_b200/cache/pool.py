"""Host-side bookkeeping of the cache: which sequence slots and which pages are held.

A slot stands for one live sequence; a page holds `PAGE` consecutive positions of
one sequence in one group of layers.  Both are handed out from free lists and
refuse to be lost, held twice or freed twice.  The reference has neither: it keeps
one sequence in buffers sized for the whole context (src/model/llama.rs:64-73,
179-186).
"""
from __future__ import annotations

from typing import List

PAGE = 64          # positions per page; kernels rely on it being a power of two
PAGE_SHIFT = 6


class CacheError(RuntimeError):
    """Misuse of the cache (double free, unknown slot)."""


class CacheFull(CacheError):
    """Not enough free slots or pages; nothing was taken."""


class FreeList:
    """Integers 0..n-1, handed out lowest first so that reuse is early and visible."""

    def __init__(self, n: int, what: str):
        self.n, self.what = int(n), what
        self._free = list(range(self.n - 1, -1, -1))      # pop() gives the lowest
        self._held = [False] * self.n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def take(self, count: int = 1) -> List[int]:
        if count > len(self._free):
            raise CacheFull(f"need {count} {self.what}s, {len(self._free)} of {self.n} are free")
        out = []
        for _ in range(count):
            i = self._free.pop()
            assert not self._held[i], f"{self.what} {i} was on the free list while held"
            self._held[i] = True
            out.append(i)
        return out

    def give_back(self, items) -> None:
        items = list(items)
        for i in items:
            if not (0 <= i < self.n):
                raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
            if not self._held[i]:
                raise CacheError(f"{self.what} {i} is freed twice or was never held")
        if len(set(items)) != len(items):
            raise CacheError(f"{self.what}s {items} name one twice")
        for i in items:
            self._held[i] = False
            self._free.append(i)
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Every item is either free or held, exactly once."""
        assert len(set(self._free)) == len(self._free), f"a {self.what} is on the free list twice"
        for i in range(self.n):
            assert self._held[i] != (i in self._free_set()), f"{self.what} {i} is lost or held while free"

    def _free_set(self):
        return set(self._free)


def pages_for(n_tokens: int) -> int:
    return (int(n_tokens) + PAGE - 1) >> PAGE_SHIFT
