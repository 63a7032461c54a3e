"""Host-side bookkeeping of the cache: which slots and which pages are in use.

Both allocators hand out the lowest free number first and refuse to free what is not held,
so that no slot or page is lost, held twice or freed twice. The reference has one
sequence and therefore no such bookkeeping (its ``pos`` lives in the engine,
src/engine.h:49); its counted heap plays the same role of an exact ledger
(src/util.h:81-89).
"""
from __future__ import annotations

import heapq
from typing import List, Set


class CacheFull(RuntimeError):
    """No free slot, or not enough free pages for the tokens asked for."""


class CacheStateError(RuntimeError):
    """A slot or page was freed twice, or is not known."""


class SlotAllocator:
    def __init__(self, count: int):
        if count <= 0:
            raise ValueError("the cache needs at least one slot")
        self.count = count
        self._free: List[int] = list(range(count))
        heapq.heapify(self._free)
        self._held: Set[int] = set()

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.count} slots are in use")
        slot = heapq.heappop(self._free)
        self._held.add(slot)
        return slot

    def free(self, slot: int) -> None:
        if slot not in self._held:
            raise CacheStateError(f"slot {slot} is not held (freed twice, or never given out)")
        self._held.remove(slot)
        heapq.heappush(self._free, slot)

    def held(self) -> Set[int]:
        return set(self._held)

    @property
    def free_count(self) -> int:
        return len(self._free)


class PageAllocator:
    def __init__(self, count: int):
        if count <= 0:
            raise ValueError("the cache needs at least one page")
        self.count = count
        self._free: List[int] = list(range(count))
        heapq.heapify(self._free)
        self._held: Set[int] = set()

    def alloc(self, n: int) -> List[int]:
        """All or nothing."""
        if n > len(self._free):
            raise CacheFull(f"{n} pages asked for, {len(self._free)} of {self.count} free")
        pages = [heapq.heappop(self._free) for _ in range(n)]
        self._held.update(pages)
        return pages

    def free(self, pages: List[int]) -> None:
        for p in pages:
            if p not in self._held:
                raise CacheStateError(f"page {p} is not held (freed twice, or never given out)")
        for p in pages:
            self._held.remove(p)
            heapq.heappush(self._free, p)

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return len(self._held)
