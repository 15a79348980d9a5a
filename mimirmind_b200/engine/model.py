"""A model put together from parts according to its spec.

The spec names, layer by layer, the kind of each part; the parts are looked up in the
registries and built from the weights.  The execution order is the spec's schedule: a
list of (layer, cache source) entries, so a layer may run twice or read another entry's
cache.  Nothing here is specific to an architecture.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..cache.manager import GroupSpec
from ..config.spec import ModelSpec
from ..parts.base import Block, KVCacheSpec, Runtime, StateSpec, WeightView
from ..registry import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, part_class


class Model:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        root = WeightView(tensors, "")
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding, root, rt)
        self.head = HEADS.get(spec.head.kind)(spec.head, root, rt)
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm, root, rt)
        self.layers: List[Block] = []
        for ls in spec.layers:
            w = root.sub(ls.prefix)
            mixer_norm = NORMS.get(ls.mixer_norm.kind)(ls.mixer_norm, w, rt)
            mixer = MIXERS.get(ls.mixer.kind)(ls.mixer, w, rt)
            ffn_norm = NORMS.get(ls.ffn_norm.kind)(ls.ffn_norm, w, rt)
            ffn = FEED_FORWARDS.get(ls.feed_forward.kind)(ls.feed_forward, w, rt)
            if ls.extras:
                extras = {name: part_class(ps)(ps, w, rt) for name, ps in ls.extras.items()}
                self.layers.append(BLOCKS.get(ls.block.kind)(ls.block, mixer_norm, mixer, ffn_norm, ffn, rt, extras=extras))
            else:
                self.layers.append(BLOCKS.get(ls.block.kind)(ls.block, mixer_norm, mixer, ffn_norm, ffn, rt))
        self.schedule = spec.schedule
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_from is not None and not (0 <= e.cache_from < i and self.schedule[e.cache_from].cache_from is None):
                raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_from}, which must be an "
                                 "earlier entry that owns a cache")
            if e.cache_from is not None:
                mine = self.layers[e.layer].mixer.kv_cache_spec()
                theirs = self.layers[self.schedule[e.cache_from].layer].mixer.kv_cache_spec()
                if mine is None or theirs is None:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_from}: both mixers must keep a paged cache")
                same = [(a.name, tuple(a.shape), a.dtype) for a in mine.token_arrays()] == \
                       [(a.name, tuple(a.shape), a.dtype) for a in theirs.token_arrays()]
                if not same:
                    raise ValueError(f"schedule entry {i} reads the cache of entry {e.cache_from}, whose per-token arrays differ from its own")
                if theirs.window and (not mine.window or mine.window > theirs.window):
                    raise ValueError(f"schedule entry {i} looks back {mine.window or 'over all'} tokens, entry {e.cache_from} keeps only "
                                     f"the last {theirs.window}")

    # ---- what the cache has to hold --------------------------------------------
    def cache_groups(self) -> List[GroupSpec]:
        """Schedule entries that own a paged cache, grouped by what they keep per token and how far back they look."""
        by_key: Dict[tuple, List[int]] = {}
        for i, e in enumerate(self.schedule):
            if e.cache_from is not None:
                continue
            ks: Optional[KVCacheSpec] = self.layers[e.layer].mixer.kv_cache_spec()
            if ks is None:
                continue
            arrays = tuple((a.name, tuple(int(x) for x in a.shape), None if a.dtype is None else str(a.dtype).replace("torch.", ""))
                           for a in ks.token_arrays())
            if any(len(shape) < 1 or min(shape) < 1 for _n, shape, _d in arrays) or len({n for n, _s, _d in arrays}) != len(arrays):
                raise ValueError(f"schedule entry {i}: per-token cache arrays need distinct names and at least one axis of positive sizes")
            by_key.setdefault((ks.num_kv_heads, ks.head_dim, ks.window, arrays if ks.arrays else ()), []).append(i)
        groups = []
        for (g, hd, w, arrays), entries in by_key.items():
            if arrays:
                name = "cache_" + "_".join(n + "x".join(str(x) for x in shape) for n, shape, _d in arrays)
            else:
                name = f"kv{g}x{hd}"
            groups.append(GroupSpec(name + (f"_w{w}" if w else "_full"), tuple(entries), g, hd, w, arrays))
        return groups

    def state_specs(self) -> Dict[int, StateSpec]:
        """Schedule entries that own fixed-size per-request state."""
        out = {}
        for i, e in enumerate(self.schedule):
            if e.cache_from is not None:
                continue
            ss = self.layers[e.layer].mixer.state_spec()
            if ss is not None:
                out[i] = ss
        return out
