"""Page and slot allocators: pure host bookkeeping, no tensors.

``PageAllocator`` is a first-in-first-out free list with a reference count per
page, after the reference's block manager
(crates/prelude-core/src/scheduler/components/cache/block_manager.rs:12-110):
``allocate`` is all-or-nothing, ``free`` drops one reference and a page goes
back to the list when nobody holds it.  ``SlotAllocator`` hands out the
fixed-size per-request state slots
(crates/prelude-core/src/scheduler/components/cache/deltanet_pool.rs:54-175).
Freeing what is not held is an error, never silently ignored.
"""
from __future__ import annotations

from collections import deque
from typing import Deque, Iterable, List


class OutOfPages(RuntimeError):
    """Not enough free pages (or slots) for the request; nothing was taken."""


class CacheAccountingError(RuntimeError):
    """A page or slot was freed that nobody held, or an id is out of range."""


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: Deque[int] = deque(range(num_pages))
        self._refs: List[int] = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def can_allocate(self, n: int) -> bool:
        return n <= len(self._free)

    def allocate(self, n: int) -> List[int]:
        """``n`` pages, each with one reference; raises OutOfPages and takes none if fewer are free."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"need {n} pages, {len(self._free)} of {self.num_pages} are free")
        out = [self._free.popleft() for _ in range(n)]
        for p in out:
            self._refs[p] = 1
        return out

    def incref(self, pages: Iterable[int]) -> None:
        for p in pages:
            self._check_held(p)
            self._refs[p] += 1

    def free(self, pages: Iterable[int]) -> None:
        """Drop one reference to each page; pages nobody holds go back to the list."""
        for p in pages:
            self._check_held(p)
            self._refs[p] -= 1
            if self._refs[p] == 0:
                self._free.append(p)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    def _check_held(self, p: int) -> None:
        if not 0 <= p < self.num_pages:
            raise CacheAccountingError(f"page id {p} outside [0, {self.num_pages})")
        if self._refs[p] <= 0:
            raise CacheAccountingError(f"page {p} is not held by anyone")

    def check(self) -> None:
        """Internal consistency: every page is either free once or held."""
        free = list(self._free)
        if len(set(free)) != len(free):
            raise CacheAccountingError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (self._refs[p] == 0) != (p in set(free)):
                raise CacheAccountingError(f"page {p}: refcount {self._refs[p]} disagrees with the free list")


class SlotAllocator:
    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError(f"a slot pool needs at least one slot, got {num_slots}")
        self.num_slots = num_slots
        self._free: Deque[int] = deque(range(num_slots))
        self._held = [False] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages(f"all {self.num_slots} state slots are in use")
        s = self._free.popleft()
        self._held[s] = True
        return s

    def free(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise CacheAccountingError(f"state slot {slot} is not held")
        self._held[slot] = False
        self._free.append(slot)

    def check(self) -> None:
        free = list(self._free)
        if len(set(free)) != len(free):
            raise CacheAccountingError("a slot is on the free list twice")
        for s in range(self.num_slots):
            if self._held[s] == (s in set(free)):
                raise CacheAccountingError(f"slot {s}: held flag disagrees with the free list")
