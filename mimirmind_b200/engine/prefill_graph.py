"""A prompt portion of one request as a replayed CUDA graph.

A long portion of a fixed number of tokens (the token budget, a whole prompt of a usual length) is the same
sequence of ~230 launches every time; only the token ids, the positions, the request's block table and the
first position of each attention tile change, and they live in device buffers that the graph reads.  Replaying
the captured step removes the launch latency between its dependent kernels (about 1-1.5 ms of a 24 ms step at
2,048 tokens of the 7B shape).  The reference captures its decode blocks only
(src/runtime/InferenceEngine.cpp:1944-1998); prefill there is eager.

The first run of a session is eager (it warms every kernel up and is a valid step of its own); the graph is
captured right after it, without running, and replayed from the second run on.
"""
from __future__ import annotations

from typing import Dict, Hashable, Optional, Sequence

import numpy as np
import torch

from ..parts.base import StepContext
from .capture import capture
from .runner import ModelRunner


class PrefillSession:
    def __init__(self, runner: ModelRunner, n_tokens: int, want_last: bool):
        self.runner, self.n, self.want_last = runner, n_tokens, want_last
        dev, ps = runner.rt.device, runner.page_size
        mgr = runner.manager
        self.width = max(1, (runner.max_seq_len + ps - 1) // ps)
        self.groups = list(mgr.groups)
        # one int32 buffer: token ids, positions, then a block-table row per group
        total = 2 * n_tokens + self.width * len(self.groups)
        self.dev_buf = torch.zeros(total, dtype=torch.int32, device=dev)
        # Two pinned staging buffers taken in turn, each with an event recorded after its copy: the host may be
        # several runs ahead of the device (portions whose logits nobody reads are never waited for), and a buffer
        # must not be rewritten before the copy that reads it has run.
        self.host_bufs = [torch.empty(total, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.copied = [None, None]
        self.token_ids = self.dev_buf[:n_tokens]
        self.positions = self.dev_buf[n_tokens:2 * n_tokens]
        self.tables = {g: self.dev_buf[2 * n_tokens + i * self.width:2 * n_tokens + (i + 1) * self.width].view(1, self.width)
                       for i, g in enumerate(self.groups)}
        self.slots = torch.zeros(1, dtype=torch.int32, device=dev)
        self.logit_rows = torch.tensor([n_tokens - 1], dtype=torch.int32, device=dev)
        self.ctx = StepContext(
            n_tokens=n_tokens, n_requests=1, token_ids=self.token_ids, positions=self.positions,
            token_req=torch.zeros(n_tokens, dtype=torch.int32, device=dev), q_start=[0], q_len=[n_tokens], kv_len=[n_tokens],
            req_meta=None, state_slots=self.slots, block_tables=self.tables, logit_rows=self.logit_rows,
            n_logit_rows=1 if want_last else 0, page_size=ps, runtime=runner.rt, max_kv_len=runner.max_seq_len, max_q_len=n_tokens)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None
        self.tile_base: Dict[int, torch.Tensor] = {}     # id(plan) -> its tiles for a portion starting at position 0
        self.start = torch.zeros(4, dtype=torch.int32, device=dev)
        self.runs = 0

    def _launch(self) -> None:
        self.ctx.derived.clear()
        self.logits = self.runner.forward(self.ctx)

    def run(self, rid: Hashable, tokens: Sequence[int], start: int) -> Optional[torch.Tensor]:
        """The step for ``tokens`` of request ``rid`` at positions [start, start + n); pages are reserved already.
        Returns fp32 logits [1, vocab] of the last token (a copy), or None if they were not wanted."""
        mgr, n = self.runner.manager, self.n
        turn = self.runs % 2
        host_buf = self.host_bufs[turn]
        if self.copied[turn] is not None:
            self.copied[turn].synchronize()
        hv = host_buf.numpy()
        hv[:n] = np.asarray(tokens, dtype=np.int32)
        hv[n:2 * n] = np.arange(start, start + n, dtype=np.int32)
        for i, g in enumerate(self.groups):
            mgr.fill_tables(g, [rid], self.width, host_buf.data_ptr() + 4 * (2 * n + i * self.width))
        self.dev_buf.copy_(host_buf, non_blocking=True)
        if self.copied[turn] is None:
            self.copied[turn] = torch.cuda.Event()
        self.copied[turn].record()
        self.slots.fill_(mgr.slot(rid))
        self.ctx.kv_len = [start + n]
        if self.graph is None:
            self.ctx.plans.clear()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._launch()                 # eager: a valid step, and the warm-up of every kernel and workspace
            torch.cuda.current_stream().wait_stream(side)
            out = self.logits.clone() if self.logits is not None else None
            torch.cuda.synchronize()
            # the plans' tiles hold absolute first positions; keep them relative so that later runs can shift them
            for plan in self.ctx.plans.values():
                tiles = getattr(plan, "tiles", None)
                if tiles is not None:
                    base = tiles.clone()
                    base[:, 3] -= start
                    self.tile_base[id(plan)] = base
            graph = torch.cuda.CUDAGraph()
            with capture(graph):                # records the launches; nothing runs
                self._launch()
            self.graph = graph
        else:
            self.start[3] = start
            for plan in self.ctx.plans.values():
                base = self.tile_base.get(id(plan))
                if base is not None:
                    torch.add(base, self.start, out=plan.tiles)
            self.graph.replay()
            out = self.logits.clone() if self.logits is not None else None
        self.runs += 1
        return out
