"""Steady-state decoding of a fixed set of requests as one replayed CUDA graph.

When every running request is decoding, a step is the same sequence of launches with the
same shapes each time: only token ids, positions and block-table entries change, and they
live in device buffers the graph reads.  The step (forward, sampling, position advance) is
captured once per (batch size, context bound, sampling kind) and replayed, which removes
the per-launch host cost of ~10 kernels per layer.  The reference has graph replay of its
decode blocks as an opt-in (src/runtime/InferenceEngine.cpp:1826-1842, 1944-1998) and names
the missing default as its largest single-user gap (doc/perf-notes-gb10.md:135-138).

A session is *bound* to a set of requests for a number of steps (the horizon); pages for
the whole horizon are reserved at binding, so the tables are final and no host work is
needed between replays except committing lengths.  The buffers and the captured graph
outlive the binding and serve the next set of requests of the same shape.
"""
from __future__ import annotations

from typing import Hashable, List, Optional, Sequence

import torch

from ..kernels import ops
from ..parts.base import StepContext
from ..sampling.params import SamplingParams
from .capture import capture
from .runner import ModelRunner


def context_bound(n: int, floor: int = 256) -> int:
    """Smallest power of two >= n (at least ``floor``): the bucket a session's buffers are sized for."""
    b = floor
    while b < n:
        b *= 2
    return b


class DecodeSession:
    def __init__(self, runner: ModelRunner, batch: int, kv_bound: int, greedy: bool = True, feed_back: bool = True,
                 penalty_window: int = 0):
        """``kv_bound``: no bound request may grow beyond this many tokens.  ``feed_back``: the graph writes
        each sampled token into the next step's input itself; otherwise the caller fills ``token_ids``
        before every step.  ``penalty_window`` > 0: the step applies soft-cap and repetition / frequency /
        presence penalties over per-request rings of that many recent tokens, kept on the device."""
        self.runner = runner
        self.batch = batch
        self.kv_bound = min(kv_bound, runner.max_seq_len)
        self.greedy = greedy
        self.feed_back = feed_back
        dev, ps = runner.rt.device, runner.page_size
        self.width = max(1, (self.kv_bound + ps - 1) // ps)
        b = batch
        self.token_ids = torch.zeros(b, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(b, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(b, dtype=torch.int32, device=dev)
        self.tables = {g: torch.full((b, self.width), -1, dtype=torch.int32, device=dev) for g in runner.manager.groups}
        ar = torch.arange(b, dtype=torch.int32, device=dev)
        self.ctx = StepContext(
            n_tokens=b, n_requests=b, token_ids=self.token_ids, positions=self.positions, token_req=ar,
            q_start=list(range(b)), q_len=[1] * b, kv_len=[self.kv_bound] * b, req_meta=None, state_slots=self.slots,
            block_tables=self.tables, logit_rows=ar, n_logit_rows=b, page_size=ps, runtime=runner.rt,
            max_kv_len=self.kv_bound, max_q_len=1)
        # the step's results in one buffer, so that one copy brings both to the host: the sampled tokens, then the flag
        # that a kernel sets when it gave up a bounded wait (kernels.ops.tcgen05_error_flag)
        self.out = torch.zeros(b + 1, dtype=torch.int32, device=dev)
        self.out_tokens = self.out[:b]
        self.error_flag = ops.tcgen05_error_flag(dev)
        self.logits: Optional[torch.Tensor] = None
        if not greedy:
            self.temperature = torch.zeros(b, dtype=torch.float32, device=dev)
            self.top_k = torch.zeros(b, dtype=torch.int32, device=dev)
            self.top_p = torch.ones(b, dtype=torch.float32, device=dev)
            self.seeds = torch.zeros(b, dtype=torch.int64, device=dev)
            self.counters = torch.zeros(b, dtype=torch.int64, device=dev)
        self.penalty_window = penalty_window
        if penalty_window > 0:
            self.recent = torch.full((b, penalty_window), -1, dtype=torch.int32, device=dev)
            self.widths = torch.zeros(b, dtype=torch.int32, device=dev)
            self.lengths = torch.zeros(b, dtype=torch.int64, device=dev)
            self.pen = torch.zeros((4, b), dtype=torch.float32, device=dev)     # repetition, frequency, presence, soft-cap
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.ids: List[Hashable] = []
        self.horizon = 0
        self.steps_done = 0

    # ---- binding -----------------------------------------------------------------------
    def bind(self, request_ids: Sequence[Hashable], horizon: int, first_tokens: Sequence[int],
             sampling: Optional[Sequence[SamplingParams]] = None, draw_counters: Optional[Sequence[int]] = None,
             histories: Optional[Sequence[Sequence[int]]] = None) -> None:
        """Points the session at ``request_ids`` for ``horizon`` steps.  Raises MemoryError (and changes
        nothing) when the pages for the horizon are not free, ValueError when the bound is too small."""
        mgr, dev = self.runner.manager, self.runner.rt.device
        if len(request_ids) != self.batch:
            raise ValueError("wrong number of requests for this session")
        lengths = [mgr.length(r) for r in request_ids]
        finals = [n + horizon for n in lengths]
        if max(finals) > self.kv_bound:
            raise ValueError(f"requests would grow to {max(finals)} tokens, the session is bound to {self.kv_bound}")
        need = {g: 0 for g in mgr.groups}
        for rid, fl in zip(request_ids, finals):
            for g, n in mgr.pages_needed(rid, fl).items():
                need[g] += n
        for g, n in need.items():
            if n > mgr.free_pages(g):
                raise MemoryError(f"decode session needs {n} pages in group {g}, {mgr.free_pages(g)} are free")
        for rid, fl in zip(request_ids, finals):
            ok = mgr.reserve(rid, fl)
            assert ok
        self.ids, self.horizon, self.steps_done = list(request_ids), horizon, 0
        for g in mgr.groups:
            t = torch.empty((self.batch, self.width), dtype=torch.int32)
            mgr.fill_tables(g, self.ids, self.width, t.data_ptr())     # -1 beyond a table's end
            self.tables[g].copy_(t.to(dev, non_blocking=False))
        self.positions.copy_(torch.tensor(lengths, dtype=torch.int32))
        self.slots.copy_(torch.tensor([mgr.slot(r) for r in self.ids], dtype=torch.int32))
        self.token_ids.copy_(torch.tensor(list(first_tokens), dtype=torch.int32))
        if not self.greedy:
            params = list(sampling)
            self.temperature.copy_(torch.tensor([0.0 if p.greedy else p.temperature for p in params], dtype=torch.float32))
            self.top_k.copy_(torch.tensor([p.top_k for p in params], dtype=torch.int32))
            self.top_p.copy_(torch.tensor([p.top_p for p in params], dtype=torch.float32))
            self.seeds.copy_(torch.tensor([p.seed & 0x7FFFFFFFFFFFFFFF for p in params], dtype=torch.int64))
            self.counters.copy_(torch.tensor(list(draw_counters or [0] * self.batch), dtype=torch.int64))
        if self.penalty_window > 0:
            # every request's ring holds its last `width` tokens, token number n at place n % width
            params = list(sampling)
            W = self.penalty_window
            ring = torch.full((self.batch, W), -1, dtype=torch.int32)
            widths, pen = [], torch.zeros((4, self.batch), dtype=torch.float32)
            for i, p in enumerate(params):
                w = min(p.penalty_window, W) if p.penalties_active else 0
                widths.append(w)
                hist = list(histories[i])
                for n in range(max(0, len(hist) - w), len(hist)):
                    ring[i, n % w] = hist[n]
                pen[0, i] = p.repetition_penalty if p.penalties_active else 1.0
                pen[1, i] = p.frequency_penalty if p.penalties_active else 0.0
                pen[2, i] = p.presence_penalty if p.penalties_active else 0.0
                pen[3, i] = p.final_logit_softcap
            self.recent.copy_(ring)
            self.widths.copy_(torch.tensor(widths, dtype=torch.int32))
            self.lengths.copy_(torch.tensor([len(h) for h in histories], dtype=torch.int64))
            self.pen.copy_(pen)

    # ---- one step's launches --------------------------------------------------------------
    def _launch(self) -> None:
        self.ctx.derived.clear()
        self.logits = self.runner.forward(self.ctx)
        if self.penalty_window > 0:
            ops.apply_penalties(self.logits, self.recent, self.pen[0], self.pen[1], self.pen[2], self.pen[3])
        if self.greedy:
            ops.argmax_rows(self.logits, self.out_tokens)
        else:
            ops.sample_rows(self.logits, self.temperature, self.top_k, self.top_p, self.seeds, self.counters, self.out_tokens)
            self.counters += 1
        if self.penalty_window > 0:
            ops.window_push(self.recent, self.widths, self.lengths, self.out_tokens)
        self.positions += 1
        self.out[self.batch:].copy_(self.error_flag)
        if self.feed_back:
            self.token_ids.copy_(self.out_tokens)

    def clear_error(self) -> None:
        self.error_flag.zero_()

    def step(self) -> torch.Tensor:
        """One decode step for every bound request; returns the device tensor of sampled tokens (valid
        until the next step).  The first step ever runs eagerly and is then captured."""
        if self.steps_done >= self.horizon:
            raise RuntimeError("decode session is past its horizon")
        if self.graph is None:
            self.ctx.plans.clear()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._launch()        # warms up every kernel and library workspace on a non-default stream
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with capture(graph):            # records the launches; nothing runs, buffers keep their contents
                self._launch()
            self.graph = graph
        else:
            self.graph.replay()
        mgr = self.runner.manager
        for rid in self.ids:
            if mgr.has(rid):          # a request may have been retired while this step was already in flight
                mgr.commit(rid, mgr.length(rid) + 1)
        self.steps_done += 1
        return self.out_tokens

    def remaining(self) -> int:
        return self.horizon - self.steps_done
