"""Gated feed-forward: ``y = (act(x·Wgᵀ) ⊙ x·Wuᵀ)·Wdᵀ`` with SiLU as the activation.

No biases (src/runtime/arch/Qwen2Backend.cpp:443-458); ``silu(g) = g / (1 + exp(−g))``
(src/compute/Activations.cpp:25-36).  Gate and up weights are concatenated at load so
that one product feeds the activation kernel.
"""
from __future__ import annotations

from typing import List

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import FEED_FORWARDS
from .base import FeedForward, Runtime, StepContext, WeightView
from .linear import linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """spec params: hidden, intermediate, gate, up, down (tensor names under the prefix)."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> List[TensorSpec]:
        d, f = spec["hidden"], spec["intermediate"]
        return [
            TensorSpec(prefix + spec["gate"], (f, d)),
            TensorSpec(prefix + spec["up"], (f, d)),
            TensorSpec(prefix + spec["down"], (d, f)),
        ]

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.hidden = int(spec["hidden"])
        self.intermediate = int(spec["intermediate"])
        gate = weights.take(spec["gate"])
        up = weights.take(spec["up"])
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()  # [2F, d]
        del gate, up
        self.w_down = weights.take(spec["down"]).contiguous()       # [d, F]

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        gu = linear(x, self.w_gate_up, None, self.rt)
        act = torch.empty((x.shape[0], self.intermediate), dtype=x.dtype, device=x.device)
        ops.silu_mul(gu, act)
        return linear(act, self.w_down, None, self.rt)
