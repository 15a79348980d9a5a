"""Pre-norm residual block: ``x += mixer(norm1(x)); x += ffn(norm2(x))``.

Order per layer in the reference: norm → QKV(+bias) → RoPE → cache write → attention → O
→ (+residual, fused with the next norm) → gate, up → SiLU·up → down → (+residual)
(src/runtime/arch/Qwen2Backend.cpp:203-461).  The last add of a layer is left pending so
that it fuses into the norm that follows, whichever layer that norm belongs to.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..registry import BLOCKS
from .base import Block, LayerCache, StepContext


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    def forward(self, residual: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: LayerCache) -> Optional[torch.Tensor]:
        h = self.mixer_norm.forward(residual, pending)
        mixed = self.mixer.forward(h, ctx, cache)
        h = self.ffn_norm.forward(residual, mixed)
        return self.feed_forward.forward(h, ctx)
