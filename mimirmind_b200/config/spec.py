"""Architecture-neutral description of a model: which parts each layer is made of.

An architecture's builder turns its typed configuration into a :class:`ModelSpec`.
Everything below the builder (weights, cache manager, step function) reads only the
spec, so no part and no engine file knows which model it serves.  The reference keeps
the same information as per-layer vectors on its backend interface
(``kvDimPerLayer``, ``kvSourceLayerPerLayer``, src/runtime/arch/ArchBackend.hpp:113-125).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registry name of its kind and its constants."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    category: str = ""      # which registry holds the kind ("norm", "mixer", ...); needed only for a layer's extra parts

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward, and whatever else the arrangement needs.

    ``prefix`` is the tensor-name prefix of the layer's weights (with trailing dot).
    """

    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec
    # Further parts of the layer by name (a norm after each branch, a gate, a second feed-forward ...): each a
    # PartSpec with its ``category``; they are built like the four above, declare their tensors like them, and are
    # handed to the block arrangement, which alone knows what to do with them.
    extras: Mapping[str, PartSpec] = field(default_factory=dict)


@dataclass(frozen=True)
class ScheduleEntry:
    """One entry of the execution order.

    ``layer`` indexes :attr:`ModelSpec.layers`; a layer may be named more than once.
    ``cache_from`` is ``None`` when the entry owns a cache (it appends this step's keys
    and values or updates its state), or the index of an earlier schedule entry whose
    cache it reads without writing.
    """

    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    eos_token_ids: Tuple[int, ...] = ()

    def describe(self) -> Dict[str, Any]:
        return {
            "architecture": self.architecture,
            "hidden_size": self.hidden_size,
            "vocab_size": self.vocab_size,
            "layers": len(self.layers),
            "schedule": [(e.layer, e.cache_from) for e in self.schedule],
        }


@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part expects in the checkpoint.

    ``role`` tells the random-weights mode how to fill it: ``matrix`` and ``bias`` are
    drawn from N(0, std), ``norm`` from 1 + N(0, norm_std), ``table`` is an embedding
    table (same as matrix).  ``optional`` tensors may be absent.
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    optional: bool = False
