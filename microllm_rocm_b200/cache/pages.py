"""Page bookkeeping, free of any device memory: a pool of fixed-size pages with a LIFO
free list (a page given back is the next one handed out, so tight pools reuse pages at
once), and a pool of slots for per-request state of fixed size.

Both refuse what would corrupt the books: freeing a page that is not held, holding one
twice, running past the pool.  `held` is kept only to be able to refuse.
"""
from __future__ import annotations

from typing import List, Optional, Set


class PageError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))   # pop() hands out 0 first
        self._held: Set[int] = set()
        self.peak_used = 0
        self.total_allocations = 0

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return len(self._held)

    def alloc(self) -> Optional[int]:
        """A free page, or None when the pool is exhausted."""
        if not self._free:
            return None
        page = self._free.pop()
        if page in self._held:
            raise PageError(f"page {page} was on the free list while held")
        self._held.add(page)
        self.total_allocations += 1
        self.peak_used = max(self.peak_used, len(self._held))
        return page

    def free(self, page: int) -> None:
        if page not in self._held:
            raise PageError(f"page {page} is freed but not held (double free?)")
        self._held.remove(page)
        self._free.append(page)

    def check(self) -> None:
        """Every page is either free or held, never both, never neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageError("a page is on the free list twice")
        if free & self._held:
            raise PageError(f"pages both free and held: {sorted(free & self._held)}")
        if len(free) + len(self._held) != self.num_pages:
            lost = set(range(self.num_pages)) - free - self._held
            raise PageError(f"pages lost: {sorted(lost)}")


class SlotPool(PagePool):
    """Slots for fixed-size per-request state; same rules as pages."""
