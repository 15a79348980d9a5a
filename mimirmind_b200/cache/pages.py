"""Page allocator: fixed-size pages handed out from a LIFO free list (C++: ``csrc/host/runtime.cpp``).

After the reference's block allocator (src/runtime/serving/PagedKvBlockAllocator.cpp:11-60):
ids are first handed out in ascending order, a freed id is the next one reused, exhaustion
is reported by a sentinel and never by an exception.  Unlike it there is no refcount or
hash slot (no prefix sharing); instead the allocator knows which ids are out, so freeing a
page twice or freeing a page that was never given is an error at once.
"""
from __future__ import annotations

from typing import List, Optional

from . import host

INVALID_PAGE = -1


class PageAllocatorError(RuntimeError):
    pass


class PageAllocator:
    """Thin handle on the C++ allocator.  ``_borrowed``: the object belongs to a cache manager."""

    def __init__(self, num_pages: int, _borrowed=None, _owner=None):
        self._lib = host.load()
        if _borrowed is not None:
            self._h, self._owned, self._owner = _borrowed, False, _owner    # keeps the owner alive
            return
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self._h, self._owned, self._owner = self._lib.mmh_alloc_create(num_pages), True, None

    def __del__(self):
        if getattr(self, "_owned", False) and self._h:
            self._lib.mmh_alloc_destroy(self._h)
            self._h = None

    @property
    def num_pages(self) -> int:
        return int(self._lib.mmh_alloc_stat(self._h, 0))

    @property
    def num_free(self) -> int:
        return int(self._lib.mmh_alloc_stat(self._h, 1))

    @property
    def num_used(self) -> int:
        return int(self._lib.mmh_alloc_stat(self._h, 2))

    @property
    def total_allocs(self) -> int:
        return int(self._lib.mmh_alloc_stat(self._h, 3))

    @property
    def reuses(self) -> int:
        """Allocations that handed out a page used before."""
        return int(self._lib.mmh_alloc_stat(self._h, 4))

    def alloc(self) -> int:
        return self._lib.mmh_alloc_alloc(self._h)

    def alloc_many(self, n: int) -> Optional[List[int]]:
        """n pages or none at all."""
        if n > self.num_free:
            return None
        return [self.alloc() for _ in range(n)]

    def free(self, page: int) -> None:
        if self._lib.mmh_alloc_free(self._h, int(page)) != 0:
            raise PageAllocatorError(host.last_error())

    def is_allocated(self, page: int) -> bool:
        return bool(self._lib.mmh_alloc_is_allocated(self._h, int(page)))

    def check(self) -> None:
        """Every page is either free exactly once or out: none lost, none held twice."""
        if self._lib.mmh_alloc_check(self._h) != 0:
            raise PageAllocatorError(host.last_error())
