"""Interfaces of the parts a layer is made of, and what a step hands to them.

A part is built from its :class:`PartSpec` (all sizes and constants are parameters
there), a :class:`WeightView` that resolves tensor names under the layer's prefix, and a
:class:`Runtime` (activation dtype, device).  No part knows which model it is in.

The reference's backend interface carries the same per-layer facts as virtuals on the
architecture object (``kvDimPerLayer``, ``maxQKVDims``, ``scalesEmbedding``,
src/runtime/arch/ArchBackend.hpp:60-223); here each part answers for itself.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..config.spec import PartSpec, TensorSpec


@dataclass(frozen=True)
class Runtime:
    """Where and in which precision a model runs."""

    dtype: torch.dtype               # activation / cache dtype: torch.float32 or torch.bfloat16
    device: torch.device
    matmul: str = "auto"             # "auto": tensor-core kernels for bf16; "simt": fp32-FMA kernel everywhere


class WeightView:
    """Name → tensor lookup under a prefix; parts take what they need and may drop it after fusing."""

    def __init__(self, tensors: Dict[str, torch.Tensor], prefix: str = ""):
        self._tensors = tensors
        self.prefix = prefix

    def sub(self, prefix: str) -> "WeightView":
        return WeightView(self._tensors, self.prefix + prefix)

    def has(self, name: str) -> bool:
        return (self.prefix + name) in self._tensors

    def get(self, name: str) -> torch.Tensor:
        full = self.prefix + name
        try:
            return self._tensors[full]
        except KeyError:
            raise KeyError(f"tensor '{full}' not in model") from None

    def take(self, name: str) -> torch.Tensor:
        """Like get, but removes the tensor from the store (the part keeps a fused copy)."""
        full = self.prefix + name
        try:
            return self._tensors.pop(full)
        except KeyError:
            raise KeyError(f"tensor '{full}' not in model") from None


@dataclass(frozen=True)
class CacheArray:
    """One array a mixer keeps per token in the paged cache: ``shape`` per token (at least one axis), ``dtype`` None
    for the run's activation dtype.  Its pool is ``[pages, *shape[:-1], page_size, shape[-1]]``: the tokens of a page
    stand before the last axis, so that for keys ``(kv_heads, head_dim)`` one head's page is one contiguous block."""

    name: str
    shape: Tuple[int, ...]
    dtype: Optional[torch.dtype] = None


@dataclass(frozen=True)
class KVCacheSpec:
    """What a mixer keeps per token and how far back it looks.  The usual case is keys and values of one head
    geometry (``num_kv_heads``, ``head_dim``); a mixer that caches something else per token (one latent vector, keys
    and values of different widths) lists its ``arrays`` instead."""

    num_kv_heads: int = 0
    head_dim: int = 0
    window: int = 0  # 0: every earlier token; W: the last W tokens (the current one included)
    arrays: Tuple[CacheArray, ...] = ()

    def token_arrays(self) -> Tuple[CacheArray, ...]:
        if self.arrays:
            return self.arrays
        return (CacheArray("k", (self.num_kv_heads, self.head_dim)), CacheArray("v", (self.num_kv_heads, self.head_dim)))


@dataclass(frozen=True)
class StateSpec:
    """A mixer that keeps a fixed-size state per request."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """What one schedule entry sees of the cache during a step."""

    k_pages: Optional[torch.Tensor] = None   # [pages, kv_heads, page_size, head_dim]: the arrays "k" and "v", if the entry has them
    v_pages: Optional[torch.Tensor] = None
    arrays: Dict[str, torch.Tensor] = field(default_factory=dict)   # every per-token array of the entry by name, [pages, ..., page_size, last]
    block_table: Optional[torch.Tensor] = None  # int32 [requests, width] of the entry's cache group
    page_size: int = 0
    writes: bool = True                      # False: the entry reads another entry's cache
    state: Optional[torch.Tensor] = None     # [slots, *StateSpec.shape]


@dataclass
class StepContext:
    """One batch: tokens of several requests, portions of prompts beside single decoded tokens.

    Tokens of a request are consecutive; request r owns tokens
    [q_start[r], q_start[r] + q_len[r]) and, after the step, holds kv_len[r] tokens.
    """

    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor            # int32 [n_tokens]
    positions: torch.Tensor            # int32 [n_tokens] absolute position of each token
    token_req: torch.Tensor            # int32 [n_tokens] index of the token's request in this batch
    q_start: Sequence[int]             # host copies, per request
    q_len: Sequence[int]
    kv_len: Sequence[int]
    req_meta: torch.Tensor             # int32 [n_requests, 4]: q_start, q_len, kv_len, state slot
    state_slots: torch.Tensor          # int32 [n_requests]
    block_tables: Dict[str, torch.Tensor]  # cache group → int32 [n_requests, width]
    logit_rows: torch.Tensor           # int32 [n_wanted] token rows whose logits are returned
    n_logit_rows: int
    page_size: int
    runtime: Runtime
    plans: Dict[Any, Any] = field(default_factory=dict)  # per-step launch plans, shared between layers
    max_kv_len: int = 0
    max_q_len: int = 0
    # device tensors derived from this step's inputs and shared between layers (rotation tables, cache slots);
    # whoever runs a context more than once (a captured decode step) clears this before every forward
    derived: Dict[Any, torch.Tensor] = field(default_factory=dict)
    # diagnostics: ``dump(stage, tensor)`` writes a stage's rows for the layer that is running (None: off); with
    # ``plain_only`` no part fuses its neighbours' work into its own kernels, so every stage exists as a tensor
    dump: Any = None
    plain_only: bool = False


@dataclass
class FactoredRows:
    """Rows of ``norm(x)`` in factored form, for norms of the kind ``x * w / rms(x)``: ``xw`` holds ``x * w`` in the
    activation dtype and ``scale`` (kernels.ops.RowScale) what is needed for each row's ``1 / rms``.  The factor
    is a scalar per row, so a matrix product may apply it to its result instead of its input; a part that says
    ``fuses(n)`` takes its input in this form."""

    xw: torch.Tensor
    scale: Any

    @property
    def shape(self):
        return self.xw.shape


@dataclass
class ResidualSink:
    """Where a fusing part adds its output itself: the fp32 residual stream (in place) and, if a norm follows whose
    consumer takes factored rows, that norm's weight and eps.  The part then returns FactoredRows of the new
    residual (or None when ``norm_weight`` is None) instead of its output."""

    residual: torch.Tensor
    norm_weight: Optional[torch.Tensor] = None
    eps: float = 0.0


@dataclass
class NativeDesc:
    """What the native step executor (csrc/exec) needs to build its own object of a part: the kind under which a
    C++ class is registered, numbers, tensors (as the part holds them after fusing) and the parts inside it."""

    kind: str
    numbers: Dict[str, float] = field(default_factory=dict)
    tensors: Dict[str, torch.Tensor] = field(default_factory=dict)
    children: Dict[str, "NativeDesc"] = field(default_factory=dict)


class Part:
    """Base of every part: declares its tensors, builds from weights."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        return []

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        self.spec = spec
        self.rt = rt

    def native(self) -> Optional["NativeDesc"]:
        """The part's description for the native step executor, or None: the part exists in Python only, and a model
        that holds it runs its steps through the Python classes."""
        return None


class Norm(Part):
    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None) -> torch.Tensor:
        """residual (fp32, [n, width]) += delta; returns the normalised rows in the activation dtype.
        With ``rows`` only those rows are produced and the residual is not written."""
        raise NotImplementedError

    def factors(self) -> Optional[Tuple[torch.Tensor, float]]:
        """(weight, eps) if the norm is ``x * weight / sqrt(mean(x^2) + eps)``, so that a product's epilogue can
        prepare it in factored form (FactoredRows); None for any other norm."""
        return None


class PositionEncoding(Part):
    def fused_rotary(self) -> Optional[Tuple[int, float]]:
        """(rotary_dim, theta) if the encoding is a split-half rotation the fused kernel can apply."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Encode positions into q [n, H, hd] and k [n, G, hd] in place (unfused path)."""
        raise NotImplementedError


class Mixer(Part):
    def kv_cache_spec(self) -> Optional[KVCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        """x: normalised activations [n_tokens, hidden] → the mixer's output [n_tokens, hidden]."""
        raise NotImplementedError

    def fuses(self, n_tokens: int) -> bool:
        """True if, for a step of ``n_tokens``, ``forward`` takes FactoredRows as ``x`` and a keyword ``sink``
        (ResidualSink).  Parts that do not override this are never given either."""
        return False


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def fuses(self, n_tokens: int) -> bool:
        """True if, for a step of ``n_tokens``, ``forward`` takes FactoredRows as ``x`` and a keyword ``sink``
        (ResidualSink).  Parts that do not override this are never given either."""
        return False


class Block(Part):
    """Arrangement of norms, mixer and feed-forward around the residual stream."""

    def __init__(self, spec: PartSpec, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, feed_forward: FeedForward,
                 rt: Runtime, extras: Optional[Dict[str, Part]] = None):
        self.spec = spec
        self.rt = rt
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ffn_norm = ffn_norm
        self.feed_forward = feed_forward
        self.extras: Dict[str, Part] = dict(extras or {})     # the layer's further parts by name (LayerSpec.extras)

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: LayerCache,
                successor: Optional["Block"] = None):
        """Runs the layer.  ``pending`` is a branch output not yet added to ``residual`` (so the add
        fuses into the next norm), or FactoredRows of the up-to-date residual prepared for this block's first
        norm; returns the new pending value.  ``successor``: the block that runs next, if any."""
        raise NotImplementedError

    def entry_norm(self, n_tokens: int) -> Optional[Tuple[torch.Tensor, float]]:
        """(weight, eps) of this block's first norm if a predecessor may hand over FactoredRows for it."""
        return None
