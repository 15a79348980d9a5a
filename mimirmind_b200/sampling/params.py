"""Sampling knobs of one request, with the reference's names, meanings and defaults.

src/compute/Sampling.hpp:40-87: ``temperature`` (<= 0: greedy), ``top_k`` (0 off, 1 greedy),
``top_p`` (1.0 off), ``seed`` (0: a random seed is drawn), ``frequency_penalty`` and
``presence_penalty`` (subtractive), ``repetition_penalty`` (divide positive logits, multiply
negative ones), ``penalty_window`` (how many recent tokens the penalties look at, 0 off),
``final_logit_softcap`` (cap·tanh(l/cap), 0 off).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, replace


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    repetition_penalty: float = 1.0
    penalty_window: int = 0
    final_logit_softcap: float = 0.0

    def __post_init__(self):
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not (0.0 <= self.top_p <= 1.0):
            raise ValueError("top_p must be in [0, 1]")
        if self.penalty_window < 0:
            raise ValueError("penalty_window must be >= 0")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1

    @property
    def penalties_active(self) -> bool:
        # src/compute/Sampling.cpp:29-34
        return self.penalty_window > 0 and (self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0
                                            or self.presence_penalty != 0.0)

    def resolved(self) -> "SamplingParams":
        """Seed 0 means "pick one" (the reference seeds from random_device, src/compute/Sampling.cpp:53-63)."""
        if self.seed != 0:
            return self
        s = int.from_bytes(os.urandom(8), "little") & 0x7FFFFFFFFFFFFFFF
        return replace(self, seed=s or 1)
