"""Cache manager: per-request block tables over page pools, and slots for fixed-size state.

Layers whose mixers keep keys and values are sorted into *groups* by what they need (head
geometry, and whether they look at every earlier token or at a window).  Each group has
its own page pool and each request one block table per group, shared by the group's
layers.  A request also owns one *state slot*: an index into per-layer arrays of
fixed-size state (the reference's ``SsmState [layers, nSeq, elems]`` slab, zeroed when a
sequence starts, src/runtime/SsmState.hpp:39-86), even when no layer has such state.

Protocol per step, after the reference's commit rule (rows written during the forward
count only after ``commit``, src/runtime/KvCache.hpp:90-103):
  ``reserve(request, new_len)``  pages for positions [len, new_len) in every group, all or
                                 nothing (src/runtime/serving/PagedKvSequence.cpp:41-74)
  ... the step writes K/V at [len, new_len) ...
  ``commit(request, new_len)``   the tokens count; a windowed group gives back the pages
                                 that no later query can reach
  ``release(request)``           everything goes back (src/runtime/serving/PagedKvSequence.cpp:76-87)

Pure host logic, in C++ (``csrc/host/runtime.cpp``); this module is its Python face and maps the caller's request
ids (any hashable) to the integers the library uses.  Block tables index by absolute position
(``table[pos // page_size]``); an entry of -1 is a page never needed or already given back.
"""
from __future__ import annotations

import ctypes
import itertools
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from . import host
from .pages import PageAllocator


class CacheError(RuntimeError):
    pass


@dataclass(frozen=True)
class GroupSpec:
    """One cache group: which schedule entries it serves and what they keep per token."""

    name: str
    entries: Tuple[int, ...]
    num_kv_heads: int
    head_dim: int
    window: int = 0
    # what an entry keeps per token: (name, shape per token, dtype name or None for the run's dtype); empty means
    # keys and values of (num_kv_heads, head_dim)
    arrays: Tuple[Tuple[str, Tuple[int, ...], Optional[str]], ...] = ()

    def token_arrays(self) -> Tuple[Tuple[str, Tuple[int, ...], Optional[str]], ...]:
        return self.arrays or (("k", (self.num_kv_heads, self.head_dim), None), ("v", (self.num_kv_heads, self.head_dim), None))


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], page_size: int, pages_per_group, max_requests: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self._lib = host.load()
        self.page_size = page_size
        self.groups: Dict[str, GroupSpec] = {g.name: g for g in groups}
        self._index: Dict[str, int] = {g.name: i for i, g in enumerate(groups)}
        if isinstance(pages_per_group, int):
            pages_per_group = {g.name: pages_per_group for g in groups}
        pages = [int(pages_per_group[g.name]) for g in groups]
        if any(n < 0 for n in pages) or max_requests < 0:
            raise ValueError("page and request counts must be >= 0")
        self._h = self._lib.mmh_cache_create(len(pages), host.int_array(pages), host.int_array([int(g.window) for g in groups]),
                                             page_size, max_requests)
        if not self._h:
            raise CacheError("the cache manager could not be created")
        self.max_requests = max_requests
        self.allocators: Dict[str, PageAllocator] = {
            g.name: PageAllocator(0, _borrowed=self._lib.mmh_cache_allocator(self._h, i), _owner=self) for i, g in enumerate(groups)}
        self._slots = PageAllocator(0, _borrowed=self._lib.mmh_cache_allocator(self._h, -1), _owner=self)
        self._ids: Dict[Hashable, int] = {}          # the caller's request id -> the library's
        self._next_id = itertools.count(1)
        self._need = (ctypes.c_int * max(1, len(pages)))()

    def __del__(self):
        if getattr(self, "_h", None):
            # handles on the allocators only borrow; nothing else outlives this object
            self._lib.mmh_cache_destroy(self._h)
            self._h = None

    # ---- request ids --------------------------------------------------------
    def handle(self, rid: Hashable) -> int:
        """The library's id of a live request."""
        try:
            return self._ids[rid]
        except KeyError:
            raise CacheError(f"unknown request {rid!r}") from None

    def _call(self, rc: int, rid: Hashable) -> int:
        if rc == -2:
            raise CacheError(f"request {rid!r}: {host.last_error()}")
        return rc

    # ---- requests ----------------------------------------------------------
    def has(self, rid: Hashable) -> bool:
        return rid in self._ids

    def add_request(self, rid: Hashable) -> Optional[int]:
        """Registers a request and gives it a state slot; None when every slot is taken."""
        if rid in self._ids:
            raise CacheError(f"request {rid!r} already exists")
        h = next(self._next_id)
        slot = self._call(self._lib.mmh_cache_add(self._h, h), rid)
        if slot < 0:
            return None
        self._ids[rid] = h
        return slot

    def adopt(self, rid: Hashable, handle: int) -> None:
        """Records a request that the scheduler's C++ side registered under ``handle``."""
        self._ids[rid] = handle

    def forget(self, rid: Hashable) -> None:
        """Drops the id of a request that the scheduler's C++ side released."""
        self._ids.pop(rid, None)

    def new_handle(self) -> int:
        return next(self._next_id)

    def length(self, rid: Hashable) -> int:
        return self._call(self._lib.mmh_cache_request(self._h, self.handle(rid), 0), rid)

    def slot(self, rid: Hashable) -> int:
        return self._call(self._lib.mmh_cache_request(self._h, self.handle(rid), 1), rid)

    def mark_started(self, rid: Hashable) -> bool:
        """True the first time it is called for a request (its state slot must be zeroed then)."""
        return bool(self._call(self._lib.mmh_cache_request(self._h, self.handle(rid), 3), rid))

    def live_requests(self) -> List[Hashable]:
        return list(self._ids)

    # ---- pages ---------------------------------------------------------------
    def pages_needed(self, rid: Hashable, new_len: int) -> Dict[str, int]:
        """New pages each group must find to hold positions up to new_len."""
        self._call(self._lib.mmh_cache_pages_needed(self._h, self.handle(rid), int(new_len), self._need), rid)
        return {name: int(self._need[i]) for name, i in self._index.items()}

    def can_reserve(self, rid: Hashable, new_len: int) -> bool:
        need = self.pages_needed(rid, new_len)
        return all(self.allocators[g].num_free >= n for g, n in need.items())

    def reserve(self, rid: Hashable, new_len: int) -> bool:
        """Pages for positions [length, new_len) in every group; False (and no change) if any group
        cannot supply them."""
        return bool(self._call(self._lib.mmh_cache_reserve(self._h, self.handle(rid), int(new_len)), rid))

    def commit(self, rid: Hashable, new_len: int) -> None:
        self._call(self._lib.mmh_cache_commit(self._h, self.handle(rid), int(new_len)), rid)

    def release(self, rid: Hashable) -> None:
        h = self.handle(rid)
        del self._ids[rid]
        self._call(self._lib.mmh_cache_release(self._h, h), rid)

    def table(self, rid: Hashable, group: str) -> List[int]:
        h, g = self.handle(rid), self._index[group]
        n = self._call(self._lib.mmh_cache_table(self._h, h, g, None, 0), rid)
        buf = (ctypes.c_int * max(1, n))()
        self._call(self._lib.mmh_cache_table(self._h, h, g, buf, n), rid)
        return list(buf[:n])

    def fill_tables(self, group: str, rids: Sequence[Hashable], width: int, out_ptr: int) -> None:
        """Writes the block tables of ``rids`` as int32 rows of ``width`` entries (-1 beyond a table's end) at
        ``out_ptr``: one call for a whole batch."""
        ids = host.long_array([self.handle(r) for r in rids])
        if self._lib.mmh_cache_tables(self._h, self._index[group], len(rids), ids, int(width), ctypes.c_void_p(out_ptr)) != 0:
            raise CacheError(host.last_error())

    # ---- accounting --------------------------------------------------------------
    def free_pages(self, group: Optional[str] = None) -> int:
        if group is not None:
            return self.allocators[group].num_free
        return min((a.num_free for a in self.allocators.values()), default=0)

    def total_pages(self, group: Optional[str] = None) -> int:
        if group is not None:
            return self.allocators[group].num_pages
        return min((a.num_pages for a in self.allocators.values()), default=0)

    def reuses(self) -> int:
        return sum(a.reuses for a in self.allocators.values())

    def check(self) -> None:
        """Invariants: every allocated page is in exactly one table; allocators are consistent."""
        if self._lib.mmh_cache_check(self._h) != 0:
            raise CacheError(host.last_error())
        live = (ctypes.c_longlong * max(1, len(self._ids)))()
        n = self._lib.mmh_cache_live(self._h, live, len(self._ids))
        if n != len(self._ids) or set(live[:n]) != set(self._ids.values()):
            raise CacheError("the request ids of the Python face and of the library differ")
