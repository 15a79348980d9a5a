"""Page allocator: fixed-size pages handed out from a LIFO free list.

After the reference's block allocator (src/runtime/serving/PagedKvBlockAllocator.cpp:11-60):
ids are first handed out in ascending order, a freed id is the next one reused, exhaustion
is reported by a sentinel and never by an exception.  Unlike it there is no refcount or
hash slot (no prefix sharing); instead the allocator knows which ids are out, so freeing a
page twice or freeing a page that was never given is an error at once.
"""
from __future__ import annotations

from typing import List, Optional

INVALID_PAGE = -1


class PageAllocatorError(RuntimeError):
    pass


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))  # pop() gives 0, 1, 2, ...
        self._out = [False] * num_pages
        self.total_allocs = 0
        self.reuses = 0                      # allocations that handed out a page used before
        self._ever_used = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            return INVALID_PAGE
        p = self._free.pop()
        self._out[p] = True
        self.total_allocs += 1
        if self._ever_used[p]:
            self.reuses += 1
        self._ever_used[p] = True
        return p

    def alloc_many(self, n: int) -> Optional[List[int]]:
        """n pages or none at all."""
        if n > len(self._free):
            return None
        return [self.alloc() for _ in range(n)]

    def free(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise PageAllocatorError(f"page {page} is outside the pool of {self.num_pages}")
        if not self._out[page]:
            raise PageAllocatorError(f"page {page} freed twice or never allocated")
        self._out[page] = False
        self._free.append(page)

    def is_allocated(self, page: int) -> bool:
        return 0 <= page < self.num_pages and self._out[page]

    def check(self) -> None:
        """Every page is either free exactly once or out: none lost, none held twice."""
        seen = [0] * self.num_pages
        for p in self._free:
            seen[p] += 1
        for p in range(self.num_pages):
            if seen[p] > 1:
                raise PageAllocatorError(f"page {p} is on the free list {seen[p]} times")
            if seen[p] == 1 and self._out[p]:
                raise PageAllocatorError(f"page {p} is both free and allocated")
            if seen[p] == 0 and not self._out[p]:
                raise PageAllocatorError(f"page {p} is lost: neither free nor allocated")
