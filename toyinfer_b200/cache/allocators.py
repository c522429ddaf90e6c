"""Host-side bookkeeping of the cache: which slots and which pages are in use.

Pure Python, no device: a slot is a sequence's place in the cache (its row of every
page table and of every fixed-size state); a page holds ``page_size`` consecutive
positions of one sequence.  Both come from free lists, are handed out at most once at
a time and must be given back exactly once; every misuse raises ``CacheError``.
The reference keeps one sequence in one region that the next turn overwrites
(src/transformer.cpp:188-195); it has nothing to allocate.
"""
from __future__ import annotations

from typing import List


PAGE = 64  # positions per page: the one place this number stands


class CacheError(RuntimeError):
    pass


class SlotAllocator:
    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise CacheError(f"the cache needs at least one slot, got {n_slots}")
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots - 1, -1, -1))  # pop() hands out 0 first
        self._live = [False] * n_slots

    @property
    def n_free(self) -> int:
        return len(self._free)

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.n_slots and self._live[slot]

    def allocate(self) -> int:
        if not self._free:
            raise CacheError(f"all {self.n_slots} slots are in use")
        slot = self._free.pop()
        self._live[slot] = True
        return slot

    def release(self, slot: int) -> None:
        if not (0 <= slot < self.n_slots):
            raise CacheError(f"slot {slot} does not exist (0..{self.n_slots - 1})")
        if not self._live[slot]:
            raise CacheError(f"slot {slot} is not in use (released twice?)")
        self._live[slot] = False
        self._free.append(slot)


class PagePool:
    """Pages 1..n_pages of a group (page 0 is the scratch page that padding writes to
    and is never handed out)."""

    def __init__(self, n_pages: int):
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages, 0, -1))
        self._live = [False] * (n_pages + 1)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def allocate(self, n: int) -> List[int]:
        if n > len(self._free):
            raise CacheError(
                f"the cache is full: {n} more pages needed, {len(self._free)} of {self.n_pages} free"
            )
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._live[p] = True
        return out

    def release(self, pages: List[int]) -> None:
        for p in pages:
            if not (1 <= p <= self.n_pages) or not self._live[p]:
                raise CacheError(f"page {p} is not in use (released twice?)")
        for p in pages:
            self._live[p] = False
            self._free.append(p)
