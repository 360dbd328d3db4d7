"""Host-side bookkeeping of cache pages and state slots.  No tensor lives here.

:class:`PageAllocator` is a LIFO free list over page ids, as the reference's
``PageAllocator`` (src/core/paging/paged_kv_cache.h:47-71) but without reference
counts: pages are never shared here (no fork, no prefix cache).  Running out is
reported, not thrown, by :meth:`try_allocate`, so the scheduler can decide.
"""
from __future__ import annotations

from typing import List, Optional


class OutOfPages(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))  # pop() hands out 0 first
        self._is_free = [True] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def try_allocate(self, n: int) -> Optional[List[int]]:
        """``n`` pages or None; never a part of them."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._is_free[p] = False
        return out

    def allocate(self, n: int) -> List[int]:
        out = self.try_allocate(n)
        if out is None:
            raise OutOfPages(f"asked for {n} pages, {len(self._free)} of {self.num_pages} are free")
        return out

    def free(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page id {p} is outside the pool of {self.num_pages}")
            if self._is_free[p]:
                raise ValueError(f"page {p} freed twice")
        for p in pages:
            self._is_free[p] = True
            self._free.append(p)


class SlotAllocator:
    """Fixed number of per-request slots (index into every fixed-size state tensor)."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError("need at least one slot")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._is_free = [True] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def try_allocate(self) -> Optional[int]:
        if not self._free:
            return None
        s = self._free.pop()
        self._is_free[s] = False
        return s

    def free(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots:
            raise ValueError(f"slot {slot} is outside [0, {self.num_slots})")
        if self._is_free[slot]:
            raise ValueError(f"slot {slot} freed twice")
        self._is_free[slot] = True
        self._free.append(slot)
