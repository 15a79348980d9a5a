"""Continuous-batching scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees; decides what happens when pages run out.

Policy, after the reference's serving substrate:
* per step, decodes first (one token each, in admission order, dropped beyond the budget),
  then prompt portions ``min(remaining, budget left)`` in admission order
  (src/runtime/serving/ChunkedPrefillScheduler.cpp:20-51), with an optional cap per portion;
* waiting requests are admitted first-in first-out while fewer than ``max_active`` run
  (src/runtime/serving/RequestScheduler.cpp:84-103) and the pages of their first portion exist;
* the last portion of a prompt yields the first generated token
  (src/runtime/serving/ContinuousBatcher.cpp:269-271);
* a request finishes on a stop id, on ``max_new`` tokens or when the context is full; the
  stop token is part of the output (src/runtime/InferenceEngine.cpp:1693, 1863-1866,
  2012); its pages and state slot go back at once;
* when pages run out the most recently admitted running request is preempted (last in,
  first out; src/runtime/serving/RequestScheduler.cpp:164-188): its pages are freed and it
  goes back to the *front* of the waiting queue.  Unlike the reference, which discards what
  a preempted request generated, its tokens are kept and recomputed as part of its prompt,
  so its output is the same as without preemption.  A request that is alone and still does
  not fit fails with ``out_of_pages`` (src/runtime/serving/PreemptionPolicy.hpp:32-41).

Pure host logic over the cache manager, in C++ (``csrc/host/runtime.cpp``); the classes here are its Python face:
they hold what the caller reads (token lists, state, reasons) and are brought up to date from the events the
library reports after every call.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache import host
from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
_FINISH = {1: "stop", 2: "length", 3: "context", 4: "out_of_pages", 6: "cancelled"}
_EV_ADMITTED, _EV_PREEMPTED, _EV_FINISHED = 1, 2, 3


class SchedulerError(RuntimeError):
    pass


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    max_new: int = 256                      # src/runtime/InferenceEngine.hpp:95-99
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: Tuple[int, ...] = ()
    # --- scheduler state (kept in step with the library) ---
    state: str = WAITING
    tokens: List[int] = field(default_factory=list)   # prompt ⧺ generated
    generated: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None     # "stop", "length", "context", "out_of_pages", "cancelled", "rejected: ..."
    preemptions: int = 0
    admit_seq: int = -1

    def __post_init__(self):
        self.tokens = list(self.prompt)

    @property
    def hit_stop(self) -> bool:
        return self.finish_reason == "stop"


@dataclass
class SchedulerConfig:
    token_budget: int = 512                 # reference default, range 1..8192 (src/core/config/Config.hpp:285-351)
    max_active: int = 32                    # reference default, range 1..256
    prefill_chunk: int = 0                  # cap of one prompt portion; 0: only the budget limits it
    max_seq_len: int = 8192                 # reference runtime.maxContextTokens default

    def __post_init__(self):
        if not (1 <= self.token_budget <= 8192 * 16):
            raise ValueError("token_budget out of range")
        if not (1 <= self.max_active <= 256):
            raise ValueError("max_active must be in 1..256")
        if self.prefill_chunk < 0:
            raise ValueError("prefill_chunk must be >= 0")


@dataclass
class PlannedEntry:
    request: Request
    start: int          # index into request.tokens of the first token fed
    count: int
    samples: bool       # the last fed token is the request's last known token: its logits are sampled

    @property
    def tokens(self) -> List[int]:
        return self.request.tokens[self.start:self.start + self.count]


class Metrics:
    """Counters of the library's scheduler, read when asked for."""

    _NAMES = ("admitted", "finished", "preempted", "rejected", "steps", "tokens_scheduled")

    def __init__(self, sched: "Scheduler"):
        self._sched = sched

    def __getattr__(self, name: str) -> int:
        try:
            what = Metrics._NAMES.index(name)
        except ValueError:
            raise AttributeError(name) from None
        return int(self._sched._lib.mmh_sched_metric(self._sched._h, what))


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, manager: CacheManager):
        self.cfg = cfg
        self.manager = manager
        self._lib = host.load()
        self._h = self._lib.mmh_sched_create(manager._h, cfg.token_budget, cfg.max_active, cfg.prefill_chunk, cfg.max_seq_len)
        if not self._h:
            raise SchedulerError("the scheduler could not be created")
        self._by_handle: Dict[int, Request] = {}
        self._handle: Dict[Hashable, int] = {}
        self.metrics = Metrics(self)
        cap = 4096
        self._rids = (ctypes.c_longlong * cap)()
        self._a = (ctypes.c_int * cap)()
        self._b = (ctypes.c_int * cap)()
        self._c = (ctypes.c_int * cap)()
        self._cap = cap

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.mmh_sched_destroy(self._h)
            self._h = None

    def _check(self, rc: int) -> int:
        if rc == -2:
            raise SchedulerError(host.last_error())
        return rc

    # ---- keeping the Python face in step ----------------------------------------------------
    def _apply_events(self) -> List[Request]:
        """Reads what the last call did to requests; returns those that finished."""
        n = self._lib.mmh_sched_events(self._h, self._rids, self._a, self._b, self._cap)
        return self.apply_events([(self._rids[i], self._a[i], self._b[i]) for i in range(min(n, self._cap))])

    def apply_events(self, events) -> List[Request]:
        """Brings the Python face up to date from (request handle, kind, code) events; returns the requests that finished."""
        done: List[Request] = []
        for handle, kind, code in events:
            req = self._by_handle[handle]
            if kind == _EV_ADMITTED:
                req.state, req.admit_seq = RUNNING, code
                self.manager.adopt(req.id, self._handle[req.id])
            elif kind == _EV_PREEMPTED:
                req.state, req.preemptions = WAITING, code
                self.manager.forget(req.id)
            elif kind == _EV_FINISHED:
                req.state, req.finish_reason = FINISHED, _FINISH[code]
                self.manager.forget(req.id)
                done.append(req)
        return done

    def _listed(self, which: int) -> List[Request]:
        n = self._lib.mmh_sched_list(self._h, which, self._rids, self._cap)
        if n > self._cap:
            buf = (ctypes.c_longlong * n)()
            self._lib.mmh_sched_list(self._h, which, buf, n)
            return [self._by_handle[h] for h in buf[:n]]
        return [self._by_handle[self._rids[i]] for i in range(n)]

    @property
    def waiting(self) -> List[Request]:
        return self._listed(0)

    @property
    def running(self) -> List[Request]:
        """In admission order."""
        return self._listed(1)

    @property
    def finished(self) -> List[Request]:
        return self._listed(2)

    # ---- admission ---------------------------------------------------------------
    def add(self, req: Request) -> bool:
        """Queues a request.  Returns False (and finishes it as rejected) when it can never run."""
        if req.id in self._handle:
            raise SchedulerError(f"request id {req.id!r} already used")
        h = self.manager.new_handle()
        prompt = host.int_array([int(t) for t in req.prompt])
        stops = host.int_array([int(t) for t in req.stop_ids])
        rc = self._check(self._lib.mmh_sched_add(self._h, h, prompt, len(req.prompt), int(req.max_new), stops, len(req.stop_ids)))
        self._handle[req.id] = h
        self._by_handle[h] = req
        req.tokens = list(req.prompt)
        sp = req.sampling
        self._check(self._lib.mmh_sched_set_sampling(self._h, h, float(sp.temperature), int(sp.top_k), float(sp.top_p),
                                                     int(sp.seed) & 0x7FFFFFFFFFFFFFFF, float(sp.frequency_penalty), float(sp.presence_penalty),
                                                     float(sp.repetition_penalty), int(sp.penalty_window), float(sp.final_logit_softcap)))
        if rc == 0:
            req.state = FINISHED
            req.finish_reason = "rejected: " + self._lib.mmh_sched_reject_reason(self._h, h).decode()
            return False
        req.state = WAITING
        return True

    def has_work(self) -> bool:
        return bool(self._lib.mmh_sched_has_work(self._h))

    # ---- one step's plan -------------------------------------------------------------
    def schedule(self) -> List[PlannedEntry]:
        """Chooses what the next step runs and reserves its pages.  May preempt or fail requests."""
        n = self._check(self._lib.mmh_sched_schedule(self._h))
        self._apply_events()
        if n > self._cap:
            raise SchedulerError(f"a plan of {n} entries exceeds the buffer of {self._cap}")
        self._lib.mmh_sched_plan(self._h, self._rids, self._a, self._b, self._c, self._cap)
        return [PlannedEntry(self._by_handle[self._rids[i]], self._a[i], self._b[i], bool(self._c[i])) for i in range(n)]

    def last_plan(self, n: int) -> List[PlannedEntry]:
        """The plan of the last ``schedule`` (made here or inside the library's step), ``n`` entries."""
        if n > self._cap:
            raise SchedulerError(f"a plan of {n} entries exceeds the buffer of {self._cap}")
        self._lib.mmh_sched_plan(self._h, self._rids, self._a, self._b, self._c, self._cap)
        return [PlannedEntry(self._by_handle[self._rids[i]], self._a[i], self._b[i], bool(self._c[i])) for i in range(n)]

    def request_of(self, handle: int) -> Request:
        return self._by_handle[handle]

    # ---- after the step ------------------------------------------------------------------
    def commit(self, plan: Sequence[PlannedEntry], sampled: Dict[Hashable, int]) -> List[Request]:
        """Advances the cache lengths, appends the sampled tokens and retires finished requests.
        ``sampled`` maps request id → token for the entries with ``samples``.  Returns the requests
        that finished in this step."""
        n = len(plan)
        rids = (ctypes.c_longlong * max(1, n))()
        starts, counts = (ctypes.c_int * max(1, n))(), (ctypes.c_int * max(1, n))()
        samples, toks = (ctypes.c_int * max(1, n))(), (ctypes.c_int * max(1, n))()
        for i, p in enumerate(plan):
            rids[i], starts[i], counts[i], samples[i] = self._handle[p.request.id], p.start, p.count, int(p.samples)
            if p.samples:
                toks[i] = int(sampled[p.request.id])
                p.request.tokens.append(toks[i])
                p.request.generated.append(toks[i])
        self._check(self._lib.mmh_sched_commit(self._h, n, rids, starts, counts, samples, toks))
        return self._apply_events()

    def accept_token(self, req: Request, tok: int) -> bool:
        """Appends a sampled token to a running request whose cache length is already advanced; retires
        the request and frees its pages if it is finished.  Returns True when it finished."""
        tok = int(tok)
        req.tokens.append(tok)
        req.generated.append(tok)
        rc = self._check(self._lib.mmh_sched_accept_token(self._h, self._handle[req.id], tok))
        self._apply_events()
        return rc == 1

    def all_decoding(self) -> bool:
        """Nothing waits and every running request has exactly its last token left to feed."""
        return bool(self._lib.mmh_sched_all_decoding(self._h))

    def cancel(self, rid: Hashable, reason: str = "cancelled") -> bool:
        """Ends a waiting or running request and gives back what it holds.  ``reason`` becomes its finish reason
        (a step that failed ends its requests with "error: ...")."""
        h = self._handle.get(rid)
        if h is None:
            return False
        rc = self._check(self._lib.mmh_sched_cancel(self._h, h))
        if rc == 1:
            req = self._by_handle[h]
            req.state, req.finish_reason = FINISHED, reason
            self.manager.forget(rid)
        return rc == 1
