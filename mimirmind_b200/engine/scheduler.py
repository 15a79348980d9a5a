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

Pure host logic over the cache manager; no tensors.
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    max_new: int = 256                      # src/runtime/InferenceEngine.hpp:95-99
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: Tuple[int, ...] = ()
    # --- scheduler state ---
    state: str = WAITING
    tokens: List[int] = field(default_factory=list)   # prompt ⧺ generated
    generated: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None     # "stop", "length", "context", "out_of_pages", "rejected: ..."
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


@dataclass
class Metrics:
    admitted: int = 0
    finished: int = 0
    preempted: int = 0
    rejected: int = 0
    steps: int = 0
    tokens_scheduled: int = 0


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, manager: CacheManager):
        self.cfg = cfg
        self.manager = manager
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []       # in admission order
        self.finished: List[Request] = []
        self.metrics = Metrics()
        self._seq = itertools.count()

    # ---- admission ---------------------------------------------------------------
    def add(self, req: Request) -> bool:
        """Queues a request.  Returns False (and finishes it as rejected) when it can never run."""
        reason = None
        if not req.prompt:
            reason = "empty prompt"
        elif req.max_new < 1:
            reason = "max_new must be at least 1"
        elif len(req.prompt) >= self.cfg.max_seq_len:
            # src/runtime/serving/ContinuousBatcher.cpp:87-123 rejects prompt >= context
            reason = f"prompt of {len(req.prompt)} tokens does not fit the context of {self.cfg.max_seq_len}"
        else:
            ps = self.manager.page_size
            need = (len(req.prompt) + ps - 1) // ps
            for name, g in self.manager.groups.items():
                if g.window <= 0 and need > self.manager.total_pages(name):
                    reason = f"prompt needs {need} pages, the pool has {self.manager.total_pages(name)}"
        if reason is not None:
            req.state, req.finish_reason = FINISHED, "rejected: " + reason
            self.finished.append(req)
            self.metrics.rejected += 1
            return False
        req.state = WAITING
        self.waiting.append(req)
        return True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- one step's plan -------------------------------------------------------------
    def _remaining(self, req: Request) -> int:
        return len(req.tokens) - self.manager.length(req.id)

    def _portion(self, req: Request, budget: int) -> int:
        n = min(self._remaining(req), budget)
        if self.cfg.prefill_chunk > 0 and n > 1:
            n = min(n, self.cfg.prefill_chunk)
        return n

    def _preempt(self, victim: Request) -> None:
        self.manager.release(victim.id)
        self.running.remove(victim)
        victim.state = WAITING
        victim.preemptions += 1
        self.waiting.appendleft(victim)
        self.metrics.preempted += 1

    def schedule(self) -> List[PlannedEntry]:
        """Chooses what the next step runs and reserves its pages.  May preempt or fail requests."""
        mgr = self.manager
        preempted_now = False
        while True:
            budget = self.cfg.token_budget
            plan: List[PlannedEntry] = []
            failed: Optional[Request] = None
            # decodes first, then prompt portions, both in admission order
            decodes = [r for r in self.running if self._remaining(r) == 1]
            prefills = [r for r in self.running if self._remaining(r) > 1]
            for req in decodes + prefills:
                if budget <= 0:
                    break
                n = self._portion(req, budget)
                start = mgr.length(req.id)
                if not mgr.reserve(req.id, start + n):
                    failed = req
                    break
                plan.append(PlannedEntry(req, start, n, start + n == len(req.tokens)))
                budget -= n
            if failed is not None:
                # pages ran out: undo nothing (reserved pages stay with their requests), preempt the
                # most recently admitted request and plan again
                victim = self.running[-1]
                if len(self.running) == 1:
                    self.manager.release(victim.id)
                    self.running.remove(victim)
                    victim.state, victim.finish_reason = FINISHED, "out_of_pages"
                    self.finished.append(victim)
                    self.metrics.finished += 1
                else:
                    self._preempt(victim)
                preempted_now = True
                continue
            # admit waiting requests, first in first out (not in a step that had to preempt: the
            # freed pages first serve the requests that were short of them)
            while not preempted_now and self.waiting and len(self.running) < self.cfg.max_active and budget > 0:
                req = self.waiting[0]
                if not mgr.has(req.id):
                    if mgr.add_request(req.id) is None:
                        break                      # no state slot free
                n = self._portion(req, budget)
                if not mgr.reserve(req.id, n):
                    mgr.release(req.id)
                    if not self.running and not plan:
                        # alone and still too large for the free pages: it can never run
                        self.waiting.popleft()
                        req.state, req.finish_reason = FINISHED, "out_of_pages"
                        self.finished.append(req)
                        self.metrics.finished += 1
                        continue
                    break
                self.waiting.popleft()
                req.state = RUNNING
                req.admit_seq = next(self._seq)
                self.running.append(req)
                self.metrics.admitted += 1
                plan.append(PlannedEntry(req, 0, n, n == len(req.tokens)))
                budget -= n
            self.metrics.steps += 1 if plan else 0
            self.metrics.tokens_scheduled += sum(p.count for p in plan)
            return plan

    # ---- after the step ------------------------------------------------------------------
    def commit(self, plan: Sequence[PlannedEntry], sampled: Dict[Hashable, int]) -> List[Request]:
        """Advances the cache lengths, appends the sampled tokens and retires finished requests.
        ``sampled`` maps request id → token for the entries with ``samples``.  Returns the requests
        that finished in this step."""
        done: List[Request] = []
        for p in plan:
            req = p.request
            self.manager.commit(req.id, p.start + p.count)
            if not p.samples:
                continue
            if self.accept_token(req, int(sampled[req.id])):
                done.append(req)
        return done

    def accept_token(self, req: Request, tok: int) -> bool:
        """Appends a sampled token to a running request whose cache length is already advanced; retires
        the request and frees its pages if it is finished.  Returns True when it finished."""
        req.tokens.append(tok)
        req.generated.append(tok)
        reason = None
        if tok in req.stop_ids:
            reason = "stop"
        elif len(req.generated) >= req.max_new:
            reason = "length"
        elif len(req.tokens) >= self.cfg.max_seq_len:
            reason = "context"
        if reason is None:
            return False
        req.state, req.finish_reason = FINISHED, reason
        self.manager.release(req.id)
        self.running.remove(req)
        self.finished.append(req)
        self.metrics.finished += 1
        return True

    def all_decoding(self) -> bool:
        """Nothing waits and every running request has exactly its last token left to feed."""
        return bool(self.running) and not self.waiting and all(self._remaining(r) == 1 for r in self.running)

    def cancel(self, rid: Hashable) -> bool:
        for req in list(self.running):
            if req.id == rid:
                self.manager.release(rid)
                self.running.remove(req)
                req.state, req.finish_reason = FINISHED, "cancelled"
                self.finished.append(req)
                return True
        for req in list(self.waiting):
            if req.id == rid:
                self.waiting.remove(req)
                if self.manager.has(rid):
                    self.manager.release(rid)
                req.state, req.finish_reason = FINISHED, "cancelled"
                self.finished.append(req)
                return True
        return False
