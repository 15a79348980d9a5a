"""Batched device-side sampling: one kernel launch for all rows of a step.

The reference has one host sampler per engine that reads the full logits back each token
(src/runtime/InferenceEngine.cpp:1167-1222).  Here every request carries its own
parameters, seed and draw counter, the logits stay on the GPU, and a request's stream does
not depend on what else is in the batch.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from .params import SamplingParams


class Sampler:
    def __init__(self, device):
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], counters: Sequence[int],
               recent: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """logits fp32 [R, V] (modified in place when soft-cap or penalties apply); ``counters[r]`` is the
        index of the draw in request r's stream; ``recent[r]`` its token history for the penalties.
        Returns int32 [R] on the device."""
        r = logits.shape[0]
        if len(params) != r or len(counters) != r:
            raise ValueError("one SamplingParams and one counter per logits row")
        need_pen = any(p.penalties_active and recent is not None and len(recent[i]) > 0 for i, p in enumerate(params))
        need_cap = any(p.final_logit_softcap > 0.0 for p in params)
        all_greedy = all(p.greedy for p in params)
        # greedy without penalties: soft-cap is monotonic, argmax is unchanged (src/compute/Sampling.cpp:134-145)
        if all_greedy and not need_pen:
            return ops.argmax_rows(logits)
        if need_pen or need_cap:
            w = max((min(p.penalty_window, len(recent[i])) if (recent is not None and p.penalties_active) else 0)
                    for i, p in enumerate(params))
            host = np.full((r, max(w, 1)), -1, dtype=np.int32)
            for i, p in enumerate(params):
                if recent is None or not p.penalties_active:
                    continue
                k = min(p.penalty_window, len(recent[i]))
                if k:
                    host[i, :k] = np.asarray(recent[i][-k:], dtype=np.int32)
            f = np.array([[p.repetition_penalty if p.penalties_active else 1.0,
                           p.frequency_penalty if p.penalties_active else 0.0,
                           p.presence_penalty if p.penalties_active else 0.0,
                           p.final_logit_softcap] for p in params], dtype=np.float32)
            d_recent = torch.from_numpy(host).to(self.device)
            d_f = torch.from_numpy(f.T.copy()).to(self.device)
            ops.apply_penalties(logits, d_recent if w > 0 else None, d_f[0], d_f[1], d_f[2], d_f[3] if need_cap else None)
            if all_greedy:
                return ops.argmax_rows(logits)
        fl = np.array([[p.temperature if not p.greedy else 0.0, p.top_p] for p in params], dtype=np.float32)
        d_fl = torch.from_numpy(fl.T.copy()).to(self.device)
        d_k = torch.tensor([p.top_k for p in params], dtype=torch.int32, device=self.device)
        d_seed = torch.tensor([p.seed & 0x7FFFFFFFFFFFFFFF for p in params], dtype=torch.int64, device=self.device)
        d_cnt = torch.tensor(list(counters), dtype=torch.int64, device=self.device)
        return ops.sample_rows(logits, d_fl[0], d_k, d_fl[1], d_seed, d_cnt)
