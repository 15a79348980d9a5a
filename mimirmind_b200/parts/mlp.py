"""Gated feed-forward: ``y = (act(x·Wgᵀ) ⊙ x·Wuᵀ)·Wdᵀ`` with SiLU as the activation.

No biases (src/runtime/arch/Qwen2Backend.cpp:443-458); ``silu(g) = g / (1 + exp(−g))``
(src/compute/Activations.cpp:25-36).  Gate and up weights are concatenated at load so
that one product feeds the activation kernel.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config.spec import PartSpec, TensorSpec
from ..kernels import ops
from ..registry import FEED_FORWARDS
from .base import FactoredRows, FeedForward, NativeDesc, ResidualSink, Runtime, StepContext, WeightView
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
        f, d = gate.shape
        # Interleave gate and up rows in blocks of 8 (rows 16j..16j+7 = gate[8j..], 16j+8..16j+15 = up[8j..]):
        # a tensor-core tile then holds a gate value and its up value together, so the activation can be
        # an epilogue of the product.  Plain concatenation when the width is not a multiple of 8.
        self.interleave = 8 if f % 8 == 0 else 0
        if self.interleave:
            self.w_gate_up = torch.stack([gate.view(f // 8, 8, d), up.view(f // 8, 8, d)], dim=1).reshape(2 * f, d).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()  # [2F, d]
        del gate, up
        self.w_down = weights.take(spec["down"]).contiguous()       # [d, F]

    def native(self):
        if type(self) is not SwiGLU:
            return None
        return NativeDesc("swiglu", {"hidden": self.hidden, "intermediate": self.intermediate, "interleave": self.interleave},
                          {"w_gate_up": self.w_gate_up, "w_down": self.w_down})

    def _tensor_cores(self) -> bool:
        return bool(self.interleave) and self.rt.dtype == torch.bfloat16 and self.w_gate_up.dtype == torch.bfloat16 \
            and self.w_down.dtype == torch.bfloat16 and self.rt.matmul != "simt"

    def fuses(self, n_tokens: int) -> bool:
        return (self._tensor_cores() and ops.small_batch_supported(n_tokens, 2 * self.intermediate, self.hidden)
                and ops.small_batch_supported(n_tokens, self.hidden, self.intermediate))

    def forward(self, x, ctx: StepContext, sink: Optional[ResidualSink] = None):
        m = x.shape[0]
        if self.fuses(m):
            # a few tokens: two weight-streaming products; 1/rms and activation in the first one's epilogue,
            # residual add and the next norm in the second one's
            xin, scale = (x.xw, x.scale) if isinstance(x, FactoredRows) else (x, None)
            act = ops.gemv_bf16(xin, self.w_gate_up, None, xin.dtype, swiglu=True, scale=scale)
            if sink is None:
                return ops.gemv_bf16(act, self.w_down, None, xin.dtype)
            made = ops.gemv_bf16_residual(act, self.w_down, sink.residual, sink.norm_weight, sink.eps)
            return FactoredRows(*made) if made is not None else None
        if self._tensor_cores() and m >= ops.TCGEN05_SWIGLU_MIN_ROWS and ops.gemm_tcgen05_supported(m, 2 * self.intermediate, self.hidden):
            # prefill-sized: tcgen05 product with the activation as its epilogue (the [m, 2F] intermediate never exists)
            act = ops.gemm_tcgen05(x, self.w_gate_up, None, x.dtype, swiglu=True)
        else:
            gu = linear(x, self.w_gate_up, None, self.rt)
            act = torch.empty((m, self.intermediate), dtype=x.dtype, device=x.device)
            ops.silu_mul(gu, act, self.interleave)
        return linear(act, self.w_down, None, self.rt)
