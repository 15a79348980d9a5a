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


def decode_session(runner: ModelRunner, batch: int, kv_bound: int, greedy: bool = True, feed_back: bool = True, penalty_window: int = 0):
    """A decode session for ``runner``: the library's own (capture, replay and the loop's turn inside the library) when the
    runner steps in the library, else the one of this module, which launches through the Python part classes."""
    if runner.native is not None:
        return LibraryDecodeSession(runner, batch, kv_bound, greedy, feed_back, penalty_window)
    return DecodeSession(runner, batch, kv_bound, greedy, feed_back, penalty_window)


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


class LibraryDecodeSession:
    """The same session inside the library (csrc/exec/executor.cu, DecodeSession): buffers, capture with the CUDA runtime's
    stream capture, replay, commit of the lengths, and one call per turn of the decode loop (``cycle``: wait for the step in
    flight, feed its tokens back, launch the next, account for the finished one in the scheduler)."""

    def __init__(self, runner: ModelRunner, batch: int, kv_bound: int, greedy: bool = True, feed_back: bool = True,
                 penalty_window: int = 0):
        import ctypes

        import numpy as np

        from . import native as nat
        self._np, self._ct = np, ctypes
        self.runner, self.batch = runner, batch
        self.kv_bound = min(kv_bound, runner.max_seq_len)
        self.greedy, self.feed_back, self.penalty_window = greedy, feed_back, penalty_window
        self._lib = nat._declare()
        self._exec = runner.native._exec
        self._h = self._lib.mmx_decode_create(self._exec, batch, self.kv_bound, int(greedy), int(feed_back), penalty_window)
        if not self._h:
            raise ops.KernelError(f"the decode session could not be created: {nat.last_error()}")
        self._last_error = nat.last_error
        self._toks = (ctypes.c_int * batch)()
        self._done = (ctypes.c_int * batch)()
        self.ids: List[Hashable] = []
        self.horizon = 0

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.mmx_decode_destroy(self._h)
            self._h = None

    def bind(self, request_ids: Sequence[Hashable], horizon: int, first_tokens: Sequence[int],
             sampling: Optional[Sequence[SamplingParams]] = None, draw_counters: Optional[Sequence[int]] = None,
             histories: Optional[Sequence[Sequence[int]]] = None) -> None:
        """As DecodeSession.bind: MemoryError when the pages for the horizon are not free, ValueError beyond the bound."""
        np, mgr, b = self._np, self.runner.manager, self.batch
        if len(request_ids) != b:
            raise ValueError("wrong number of requests for this session")
        rids = np.asarray([mgr.handle(r) for r in request_ids], dtype=np.int64)
        firsts = np.asarray(list(first_tokens), dtype=np.int32)
        keep = [rids, firsts]
        ptr = lambda a: a.ctypes.data if a is not None else None
        temp = topk = topp = seeds = counters = recent = widths = lengths = pen = None
        if not self.greedy:
            params = list(sampling)
            temp = np.asarray([0.0 if p.greedy else p.temperature for p in params], dtype=np.float32)
            topk = np.asarray([p.top_k for p in params], dtype=np.int32)
            topp = np.asarray([p.top_p for p in params], dtype=np.float32)
            seeds = np.asarray([p.seed & 0x7FFFFFFFFFFFFFFF for p in params], dtype=np.int64)
            counters = np.asarray(list(draw_counters or [0] * b), dtype=np.int64)
        if self.penalty_window > 0:
            # every request's ring holds its last `width` tokens, token number n at place n % width
            params, W = list(sampling), self.penalty_window
            recent = np.full((b, W), -1, dtype=np.int32)
            widths = np.zeros(b, dtype=np.int32)
            pen = np.zeros((4, b), dtype=np.float32)
            for i, p in enumerate(params):
                w = min(p.penalty_window, W) if p.penalties_active else 0
                widths[i] = w
                hist = histories[i]
                for n in range(max(0, len(hist) - w), len(hist)):
                    recent[i, n % w] = hist[n]
                pen[0, i] = p.repetition_penalty if p.penalties_active else 1.0
                pen[1, i] = p.frequency_penalty if p.penalties_active else 0.0
                pen[2, i] = p.presence_penalty if p.penalties_active else 0.0
                pen[3, i] = p.final_logit_softcap
            lengths = np.asarray([len(h) for h in histories], dtype=np.int64)
        rc = self._lib.mmx_decode_bind(self._h, ptr(rids), int(horizon), ptr(firsts), ptr(temp), ptr(topk), ptr(topp), ptr(seeds), ptr(counters),
                                       ptr(recent), ptr(widths), ptr(lengths), ptr(pen), ops._stream())
        del keep
        if rc == 1:
            raise MemoryError("the decode session's pages for the horizon are not free")
        if rc == 2:
            raise ValueError(f"requests would grow beyond the {self.kv_bound} tokens the session is bound to")
        if rc != 0:
            raise ops.KernelError(self._last_error())
        self.ids, self.horizon = list(request_ids), horizon

    def step(self) -> None:
        """One decode step for every bound request (launched eagerly and captured the first time, replayed afterwards);
        the sampled tokens stay on the device (``tokens()`` copies them)."""
        if self._lib.mmx_decode_step(self._h, ops._stream()) != 0:
            raise ops.KernelError(self._last_error())

    def begin(self) -> None:
        """The first step of a run whose results come back through ``cycle``."""
        if self._lib.mmx_decode_begin(self._h, ops._stream()) != 0:
            raise ops.KernelError(self._last_error())

    def cycle(self, scheduler_handle, launch_next: bool):
        """One turn of the decode loop in one call.  Returns (tokens of the finished step, per request: 1 finished with this
        token / 0 goes on / -1 had left before, whether any finished)."""
        rc = self._lib.mmx_decode_cycle(self._exec, self._h, scheduler_handle, int(launch_next), self._toks, self._done, ops._stream())
        if rc < 0:
            raise ops.KernelError(self._last_error())
        return list(self._toks), list(self._done), rc == 1

    def drop(self, index: int) -> None:
        """Request ``index`` of the binding has left (cancelled by its caller): its further tokens are not accounted for."""
        self._lib.mmx_decode_drop(self._h, int(index))

    def remaining(self) -> int:
        return int(self._lib.mmx_decode_info(self._h, 0))

    @property
    def steps_done(self) -> int:
        return int(self._lib.mmx_decode_info(self._h, 1))

    @property
    def graph(self):
        return True if self._lib.mmx_decode_info(self._h, 2) else None
