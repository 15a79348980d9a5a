"""Rotary position encoding, split-half pairing, with theta and the rotated width as parameters.

Pairs are ``(i, i + half)``; ``angle = pos · theta^(−2i/dim)``;
``x'_i = x_i cos − x_{i+half} sin``, ``x'_{i+half} = x_i sin + x_{i+half} cos``
(src/compute/Rope.cpp:23-41).  Applied to q and k after their bias, never to v
(src/runtime/arch/Qwen2Backend.cpp:369-375).  Angles are computed in fp32 on the device.
"""
from __future__ import annotations

from typing import Optional, Tuple

from ..config.spec import PartSpec
from ..registry import POSITION_ENCODINGS
from .base import NativeDesc, PositionEncoding, Runtime, WeightView


@POSITION_ENCODINGS.register("rotary_half")
class RotaryHalf(PositionEncoding):
    """spec params: theta, rotary_dim (leading dims of each head that rotate)."""

    def __init__(self, spec: PartSpec, weights: WeightView, rt: Runtime):
        super().__init__(spec, weights, rt)
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim % 2:
            raise ValueError("rotary_dim must be even")

    def fused_rotary(self) -> Optional[Tuple[int, float]]:
        return self.rotary_dim, self.theta

    def native(self):
        if type(self) is not RotaryHalf:
            return None
        return NativeDesc("rotary_half", {"theta": self.theta, "rotary_dim": self.rotary_dim})


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """No encoding: the fused kernel is told to rotate nothing."""

    def fused_rotary(self) -> Optional[Tuple[int, float]]:
        return 0, 1.0

    def native(self):
        return NativeDesc("none") if type(self) is NoPositionEncoding else None
