"""Device memory of the cache: page pools per group and state arrays per entry.

Pool layout per group and per-token array: ``[entries, pages, *shape[:-1], page_size, shape[-1]]``;
for keys and values, ``[entries, pages, kv_heads, page_size, head_dim]`` each, in the run's
dtype, so one KV head's page is one contiguous run of ``page_size * head_dim`` elements.  (The reference's pool is ``[blocks, blockSize, kvHeads, headDim]`` per layer,
src/runtime/serving/PagedKvPool.hpp:24-33; heads are moved outward here so that a tile of
keys of one head is contiguous.)  State arrays are ``[slots, *shape]`` per entry.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache.manager import CacheManager
from ..parts.base import LayerCache, Runtime, StepContext
from .model import Model


class CacheStorage:
    def __init__(self, model: Model, manager: CacheManager, rt: Runtime):
        self.model = model
        self.manager = manager
        self.page_size = manager.page_size
        # group name -> array name -> [entries, pages, *shape[:-1], page_size, shape[-1]]
        self.pools: Dict[str, Dict[str, torch.Tensor]] = {}
        self._entry_group: Dict[int, tuple] = {}
        for name, g in manager.groups.items():
            pages = manager.allocators[name].num_pages
            self.pools[name] = {}
            for array, shape, dtype in g.token_arrays():
                dt = rt.dtype if dtype is None else getattr(torch, dtype)
                self.pools[name][array] = torch.zeros((len(g.entries), max(pages, 1)) + tuple(shape[:-1]) + (self.page_size, shape[-1]),
                                                      dtype=dt, device=rt.device)
            for j, e in enumerate(g.entries):
                self._entry_group[e] = (name, j)
        self.states: Dict[int, torch.Tensor] = {}
        for e, ss in model.state_specs().items():
            self.states[e] = torch.zeros((manager.max_requests,) + tuple(ss.shape), dtype=ss.dtype, device=rt.device)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for pool in self.pools.values() for t in pool.values()) + \
            sum(t.numel() * t.element_size() for t in self.states.values())

    def entry_pool(self, entry: int):
        """(group name, index in the group's pool) of a schedule entry that owns keys and values, else None."""
        return self._entry_group.get(entry)

    def zero_slot(self, slot: int) -> None:
        for t in self.states.values():
            t[slot].zero_()

    def layer_cache(self, entry: int, ctx: StepContext) -> LayerCache:
        sched = self.model.schedule[entry]
        owner = entry if sched.cache_from is None else sched.cache_from
        lc = LayerCache(page_size=self.page_size, writes=sched.cache_from is None)
        if owner in self._entry_group:
            name, j = self._entry_group[owner]
            lc.arrays = {array: t[j] for array, t in self.pools[name].items()}
            lc.k_pages, lc.v_pages = lc.arrays.get("k"), lc.arrays.get("v")
            lc.block_table = ctx.block_tables[name]
        if owner in self.states:
            lc.state = self.states[owner]
        return lc
