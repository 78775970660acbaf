"""Free list of cache pages: bookkeeping only, no tensors.

Contract of the reference's ``BlockAllocator`` (pyre/paged_cache.py:40-92): a stack of
free page numbers (the page freed last is handed out first), a reference count per
page in use, ``OutOfPages`` (a MemoryError) when the pool is empty, ValueError on a
double free and on a reference to a page that is not in use.  ``can_allocate`` lets
the scheduler ask before it takes, so running out is a decision and not an exception.
"""

from __future__ import annotations


class OutOfPages(MemoryError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: list[int] = list(range(self.num_pages - 1, -1, -1))  # page 0 goes out first
        self._refs: list[int] = [0] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def can_allocate(self, n: int) -> bool:
        return n <= len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages(f"page pool exhausted: all {self.num_pages} pages are in use")
        page = self._free.pop()
        self._refs[page] = 1
        return page

    def allocate_many(self, n: int) -> list[int]:
        if n > len(self._free):
            raise OutOfPages(f"page pool exhausted: {n} pages wanted, {len(self._free)} of {self.num_pages} free")
        return [self.allocate() for _ in range(n)]

    def incref(self, page: int) -> None:
        if not 0 <= page < self.num_pages or self._refs[page] <= 0:
            raise ValueError(f"page {page} is not in use; cannot take another reference")
        self._refs[page] += 1

    def free(self, page: int) -> bool:
        """Drop one reference; True if the page went back to the pool."""
        if not 0 <= page < self.num_pages or self._refs[page] <= 0:
            raise ValueError(f"double free or free of a page that is not in use: {page}")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)
            return True
        return False

    def ref_count(self, page: int) -> int:
        return self._refs[page]

    def check(self) -> None:
        """Invariants: every page is either free exactly once or referenced, never both."""
        seen = set(self._free)
        if len(seen) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        for p in range(self.num_pages):
            if (self._refs[p] > 0) == (p in seen):
                raise AssertionError(f"page {p}: refs {self._refs[p]}, on free list: {p in seen}")
