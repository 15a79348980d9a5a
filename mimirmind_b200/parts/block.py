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
from .base import Block, FactoredRows, LayerCache, NativeDesc, ResidualSink, StepContext


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    """With parts that fuse (a few tokens in bfloat16), the residual add and the norm move into the epilogue of
    the branch's last matrix product and the 1/rms into the next product: a layer is five launches."""

    def entry_norm(self, n_tokens: int):
        f = self.mixer_norm.factors()
        return f if f is not None and self.mixer.fuses(n_tokens) else None

    def native(self):
        parts = {"mixer_norm": self.mixer_norm.native(), "mixer": self.mixer.native(), "ffn_norm": self.ffn_norm.native(),
                 "feed_forward": self.feed_forward.native()}
        if type(self) is not PreNormBlock or any(p is None for p in parts.values()):
            return None
        return NativeDesc("pre_norm", {}, {}, parts)

    def forward(self, residual: torch.Tensor, pending, ctx: StepContext, cache: LayerCache,
                successor: Optional[Block] = None):
        n = residual.shape[0]
        if ctx.plain_only:
            return self._forward_plain(residual, pending, ctx, cache)
        mixer_fuses, ffn_fuses = self.mixer.fuses(n), self.feed_forward.fuses(n)
        h = pending if isinstance(pending, FactoredRows) else self.mixer_norm.forward(residual, pending)
        between = self.ffn_norm.factors() if (mixer_fuses and ffn_fuses) else None
        if between is not None:
            h = self.mixer.forward(h, ctx, cache, sink=ResidualSink(residual, between[0], between[1]))
        else:
            h = self.ffn_norm.forward(residual, self.mixer.forward(h, ctx, cache))
        if not ffn_fuses:
            return self.feed_forward.forward(h, ctx)
        after = successor.entry_norm(n) if successor is not None else None
        if successor is not None and after is None:
            return self.feed_forward.forward(h, ctx)       # the next block wants a plain pending sum
        sink = ResidualSink(residual, after[0], after[1]) if after is not None else ResidualSink(residual)
        return self.feed_forward.forward(h, ctx, sink=sink)

    def _forward_plain(self, residual: torch.Tensor, pending, ctx: StepContext, cache: LayerCache):
        """Every stage as a tensor of its own, with the stage dumps of the reference
        (src/runtime/arch/Qwen2Backend.cpp:207, 431, 458, 462): the normalised input of the mixer, the two branch
        outputs, and the layer's output (the residual stream with both branches added)."""
        dump = ctx.dump or (lambda stage, t: None)
        h = self.mixer_norm.forward(residual, pending)
        dump("attn_norm", h)
        branch = self.mixer.forward(h, ctx, cache)
        dump("attn_out", branch)
        h = self.ffn_norm.forward(residual, branch)
        out = self.feed_forward.forward(h, ctx)
        dump("ffn_mlp", out)
        if ctx.dump is not None:
            dump("l_out", residual + out.to(residual.dtype))
        return out
