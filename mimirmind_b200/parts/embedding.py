"""Token embedding and output head.

Embedding: ``x[t,:] = E[id_t,:]`` with an optional scale (none for this architecture,
src/runtime/arch/Qwen2Backend.hpp:50); an id outside the table gives a zero row
(src/compute/Embedding.cpp:46-67).  Head: ``logits = n·Wᵀ`` with W the ``lm_head`` tensor
if the checkpoint has one, else the embedding table (src/runtime/InferenceEngine.cpp:1374-1377),
computed only for the rows whose logits are wanted and returned as fp32.
"""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import EMBEDDINGS, HEADS
from .base import NativeDesc, Part, Runtime, WeightView
from .linear import linear


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """spec params: vocab, width, scale, weight (full tensor name)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(spec["weight"], (spec["vocab"], spec["width"]), role="table")]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.vocab = int(spec["vocab"])
        self.width = int(spec["width"])
        self.scale = float(spec.get("scale", 1.0))
        self.table = weights.get(spec["weight"]).contiguous()

    def native(self):
        if type(self) is not TokenEmbedding:
            return None
        return NativeDesc("token_embedding", {"vocab": self.vocab, "width": self.width, "scale": self.scale}, {"table": self.table})

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = torch.empty((token_ids.numel(), self.width), dtype=torch.float32, device=token_ids.device)
        return ops.embedding(token_ids, self.table, out, self.scale)


@HEADS.register("lm_head")
class LMHead(Part):
    """spec params: vocab, width, weight (full tensor name), tied_to (embedding tensor name or None)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        tied = spec.get("tied_to") is not None
        return [TensorSpec(spec["weight"], (spec["vocab"], spec["width"]), optional=tied)]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.vocab = int(spec["vocab"])
        if weights.has(spec["weight"]):
            self.weight = weights.get(spec["weight"]).contiguous()
        elif spec.get("tied_to") is not None:
            self.weight = weights.get(spec["tied_to"]).contiguous()
        else:
            raise KeyError(f"tensor '{spec['weight']}' not in model")

    def native(self):
        return NativeDesc("lm_head", {"vocab": self.vocab}, {"weight": self.weight}) if type(self) is LMHead else None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, None, self.rt, out_dtype=torch.float32)
