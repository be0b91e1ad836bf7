"""A pool of pages with a free list and reference counts.

Semantics of the reference's allocator (src/flexengine/engine/kv_cache/allocator.py:25-105,147-158):
FIFO free list, allocation of several pages is atomic (fails before touching anything),
a page returns to the free list when its last owner lets go, and an invariants check.
"""
from __future__ import annotations

from collections import deque


class CacheExhausted(RuntimeError):
    """Not enough free pages (or state slots) for what was asked."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self.free: deque[int] = deque(range(self.num_pages))
        self.refs = [0] * self.num_pages
        self.shared = 0          # pages with more than one owner (none in the usual case: a fast path asks)

    @property
    def free_pages(self) -> int:
        return len(self.free)

    @property
    def used_pages(self) -> int:
        return self.num_pages - len(self.free)

    def allocate(self, count: int) -> list[int]:
        if count < 0:
            raise ValueError("negative page count")
        if count > len(self.free):
            raise CacheExhausted(f"Need {count} pages; only {len(self.free)} free")
        pages = []
        for _ in range(count):
            page = self.free.popleft()
            assert self.refs[page] == 0, "free list held a page that is in use"
            self.refs[page] = 1
            pages.append(page)
        return pages

    def retain(self, page: int) -> None:
        """Add an owner to a page that is in use."""
        if not (0 <= page < self.num_pages) or self.refs[page] <= 0:
            raise ValueError("cannot retain a page that is not allocated")
        self.refs[page] += 1
        if self.refs[page] == 2:
            self.shared += 1

    def release(self, page: int) -> None:
        """Drop one owner; the page becomes free when none is left."""
        if not (0 <= page < self.num_pages):
            raise ValueError(f"page {page} does not exist")
        if self.refs[page] <= 0:
            raise RuntimeError(f"page {page} released more often than it was held")
        self.refs[page] -= 1
        if self.refs[page] == 1:
            self.shared -= 1
        if self.refs[page] == 0:
            self.free.append(page)

    def assert_invariants(self, owners: dict[int, int]) -> None:
        """``owners``: {page: number of holders the caller knows of}."""
        free = list(self.free)
        if len(free) != len(set(free)):
            raise AssertionError("a page is on the free list twice")
        if set(free) & set(p for p, n in owners.items() if n > 0):
            raise AssertionError("a page is both free and held")
        for page in range(self.num_pages):
            if self.refs[page] != owners.get(page, 0):
                raise AssertionError(f"page {page}: {self.refs[page]} references, {owners.get(page, 0)} holders")
        if len(free) + sum(1 for r in self.refs if r > 0) != self.num_pages:
            raise AssertionError("a page was lost")
