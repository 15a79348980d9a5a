"""RMSNorm with its eps as a parameter.

``y = x · w / sqrt(mean(x²) + eps)``: eps inside the root, added after the mean; the
weight multiplies directly (src/compute/Norm.cpp:21-37).  The residual add that precedes
a norm is fused into it, as the reference's add+norm kernel does
(kernels/cuda/common/add_rmsnorm.cu:32-81).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import NORMS
from .base import NativeDesc, Norm, Runtime, WeightView


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """spec params: width, eps, weight (tensor name under the prefix)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(prefix + spec["weight"], (spec["width"],), role="norm")]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.width = int(spec["width"])
        self.eps = float(spec["eps"])
        self.weight = weights.get(spec["weight"]).contiguous()

    def factors(self):
        return self.weight, self.eps

    def native(self):
        if type(self) is not RMSNorm:
            return None
        return NativeDesc("rmsnorm", {"width": self.width, "eps": self.eps}, {"weight": self.weight})

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                n_rows: Optional[int] = None) -> torch.Tensor:
        n = residual.shape[0] if rows is None else (n_rows if n_rows is not None else rows.numel())
        out = torch.empty((n, self.width), dtype=self.rt.dtype, device=residual.device)
        if rows is not None and rows.numel() != n:
            rows = rows[:n]
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows)
