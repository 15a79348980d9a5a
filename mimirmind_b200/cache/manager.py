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

Pure host logic: no tensors here.  Block tables index by absolute position
(``table[pos // page_size]``); an entry of -1 is a page never needed or already given back.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from .pages import INVALID_PAGE, PageAllocator


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


@dataclass
class _Request:
    length: int = 0                       # committed tokens
    reserved: int = 0                     # tokens with pages
    slot: int = -1
    tables: Dict[str, List[int]] = field(default_factory=dict)
    started: bool = False                 # state slot already zeroed by the runner


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], page_size: int, pages_per_group, max_requests: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.groups: Dict[str, GroupSpec] = {g.name: g for g in groups}
        if isinstance(pages_per_group, int):
            pages_per_group = {g.name: pages_per_group for g in groups}
        self.allocators: Dict[str, PageAllocator] = {g.name: PageAllocator(pages_per_group[g.name]) for g in groups}
        self.max_requests = max_requests
        self._slots = PageAllocator(max_requests)
        self._requests: Dict[Hashable, _Request] = {}

    # ---- requests ----------------------------------------------------------
    def has(self, rid: Hashable) -> bool:
        return rid in self._requests

    def add_request(self, rid: Hashable) -> Optional[int]:
        """Registers a request and gives it a state slot; None when every slot is taken."""
        if rid in self._requests:
            raise CacheError(f"request {rid!r} already exists")
        slot = self._slots.alloc()
        if slot == INVALID_PAGE:
            return None
        self._requests[rid] = _Request(slot=slot, tables={name: [] for name in self.groups})
        return slot

    def _req(self, rid: Hashable) -> _Request:
        try:
            return self._requests[rid]
        except KeyError:
            raise CacheError(f"unknown request {rid!r}") from None

    def length(self, rid: Hashable) -> int:
        return self._req(rid).length

    def slot(self, rid: Hashable) -> int:
        return self._req(rid).slot

    def mark_started(self, rid: Hashable) -> bool:
        """True the first time it is called for a request (its state slot must be zeroed then)."""
        r = self._req(rid)
        first = not r.started
        r.started = True
        return first

    def live_requests(self) -> List[Hashable]:
        return list(self._requests)

    # ---- pages ---------------------------------------------------------------
    def _blocks_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    def pages_needed(self, rid: Hashable, new_len: int) -> Dict[str, int]:
        """New pages each group must find to hold positions up to new_len."""
        r = self._req(rid)
        need = {}
        for name in self.groups:
            table = r.tables[name]
            first = r.length // self.page_size
            last = self._blocks_for(new_len)
            n = 0
            for b in range(first, last):
                if b >= len(table) or table[b] == INVALID_PAGE:
                    n += 1
            need[name] = n
        return need

    def can_reserve(self, rid: Hashable, new_len: int) -> bool:
        need = self.pages_needed(rid, new_len)
        return all(self.allocators[g].num_free >= n for g, n in need.items())

    def reserve(self, rid: Hashable, new_len: int) -> bool:
        """Pages for positions [length, new_len) in every group; False (and no change) if any group
        cannot supply them."""
        r = self._req(rid)
        if new_len < r.length:
            raise CacheError(f"request {rid!r}: cannot reserve {new_len} below its length {r.length}")
        if not self.can_reserve(rid, new_len):
            return False
        first = r.length // self.page_size
        last = self._blocks_for(new_len)
        for name in self.groups:
            table = r.tables[name]
            while len(table) < last:
                table.append(INVALID_PAGE)
            for b in range(first, last):
                if table[b] == INVALID_PAGE:
                    p = self.allocators[name].alloc()
                    assert p != INVALID_PAGE
                    table[b] = p
        r.reserved = max(r.reserved, new_len)
        return True

    def commit(self, rid: Hashable, new_len: int) -> None:
        r = self._req(rid)
        if new_len < r.length or new_len > r.reserved:
            raise CacheError(f"request {rid!r}: commit to {new_len} outside [{r.length}, {r.reserved}]")
        r.length = new_len
        # the next query sits at position new_len and sees keys >= new_len + 1 - W
        for name, g in self.groups.items():
            if g.window <= 0:
                continue
            dead_before = new_len + 1 - g.window       # positions below this are never read again
            if dead_before <= 0:
                continue
            table = r.tables[name]
            for b in range(min(dead_before // self.page_size, len(table))):
                if table[b] != INVALID_PAGE:
                    self.allocators[name].free(table[b])
                    table[b] = INVALID_PAGE

    def release(self, rid: Hashable) -> None:
        r = self._requests.pop(rid, None)
        if r is None:
            raise CacheError(f"unknown request {rid!r}")
        for name, table in r.tables.items():
            for p in table:
                if p != INVALID_PAGE:
                    self.allocators[name].free(p)
        self._slots.free(r.slot)

    def table(self, rid: Hashable, group: str) -> List[int]:
        return self._req(rid).tables[group]

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
        for name, alloc in self.allocators.items():
            alloc.check()
            seen = set()
            for rid, r in self._requests.items():
                for p in r.tables[name]:
                    if p == INVALID_PAGE:
                        continue
                    if p in seen:
                        raise CacheError(f"group {name}: page {p} is in two block tables")
                    if not alloc.is_allocated(p):
                        raise CacheError(f"group {name}: page {p} of request {rid!r} is not allocated")
                    seen.add(p)
            if len(seen) != alloc.num_used:
                raise CacheError(f"group {name}: {alloc.num_used} pages are out but tables hold {len(seen)}")
        self._slots.check()
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or len(slots) != self._slots.num_used:
            raise CacheError("state slots are inconsistent")
