"""The Python entry point: load a model, generate tokens for a list of prompts.

``Engine.generate`` is the counterpart of the reference's
``InferenceEngine::generate(promptIds, GenerateParams, onToken, stats)``
(src/runtime/InferenceEngine.hpp:207-380; .cpp:1304-2131), for many prompts at once under
the continuous-batching scheduler: token ids in, token ids out, ``max_new`` counts the first
token, a stop token is part of the output, statistics give prompt and generated token
counts, prefill and decode time and whether a stop id was hit.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, Dict, Hashable, List, Optional, Sequence

import torch

from ..kernels.lib import KernelError
from ..sampling import Sampler, SamplingParams
from .decode_graph import DecodeSession, LibraryDecodeSession, context_bound, decode_session
from .loader import load_model, random_model
from .model import Model
from .runner import ModelRunner, StepEntry
from .scheduler import PlannedEntry, Request, Scheduler, SchedulerConfig


@dataclass
class GenerateStats:
    """After the reference's GenerateStats (src/runtime/InferenceEngine.hpp:104-133)."""

    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_ms: float = 0.0       # time to the request's first token
    decode_ms: float = 0.0        # time from the first to the last token
    hit_stop: bool = False
    finish_reason: str = ""
    preemptions: int = 0


@dataclass
class GenerateResult:
    tokens: List[int]
    stats: GenerateStats


class Engine:
    def __init__(self, model: Model, *, page_size: int = 16, cache_tokens: int = 0, max_context: int = 8192,
                 token_budget: int = 512, max_active: int = 32, prefill_chunk: int = 0, use_graphs: bool = True,
                 cache_memory_fraction: float = 0.9):
        self.model = model
        max_context = min(max_context, model.spec.max_positions)
        if cache_tokens <= 0:
            cache_tokens = self.cache_tokens_that_fit(model, page_size, max_context, token_budget, max_active, cache_memory_fraction)
        num_pages = (cache_tokens + page_size - 1) // page_size
        self.runner = ModelRunner(model, page_size=page_size, num_pages=num_pages, max_requests=max_active,
                                  max_seq_len=max_context)
        self.sched_cfg = SchedulerConfig(token_budget=token_budget, max_active=max_active,
                                         prefill_chunk=prefill_chunk, max_seq_len=max_context)
        self.sampler = Sampler(model.rt.device)
        self.eos_ids = tuple(model.spec.eos_token_ids)
        self.last_metrics = None
        self.use_graphs = use_graphs
        self.graph_min_steps = 8            # shorter decode runs are stepped eagerly
        self.max_decode_graphs = 48         # captured decode steps kept at a time
        self._sessions: Dict[tuple, DecodeSession] = {}
        self.graph_steps = 0                # decode steps that were graph replays (statistics)
        self.h2d_bytes = 0                  # bytes copied host→device / device→host by generate()
        self.d2h_bytes = 0
        self.decode_trace = None            # engine.diagnostics.DecodeTrace: a line per decode step
        self._pinned: Dict[int, tuple] = {}

    @staticmethod
    def cache_tokens_that_fit(model: Model, page_size: int, max_context: int, token_budget: int, max_active: int,
                              fraction: float) -> int:
        """The pool size when none is configured: what fits in ``fraction`` of the device memory that is free now
        (the weights are loaded), less what a step of ``token_budget`` tokens needs, at most
        ``max_context x max_active`` tokens."""
        from ..cache import sizing
        from ..weights.store import layer_tensor_shapes
        esz = 4 if model.rt.dtype == torch.float32 else 2
        shapes = layer_tensor_shapes(model.spec)
        free, _total = torch.cuda.mem_get_info(model.rt.device)
        return sizing.pool_tokens(free, fraction, sizing.step_reserve_bytes(model.spec, shapes, esz, token_budget, max_active),
                                  sizing.cache_bytes_per_token(model.cache_groups(), esz), page_size, max_context, max_active)

    def set_diagnostics(self, parity_dump: str = "", trace_decode_file: str = "") -> None:
        """Stage dumps of the steps that hold a prompt portion (file prefix) and a per-step decode trace (file)."""
        from .diagnostics import DecodeTrace, StageDump
        self.runner.stage_dump = StageDump(parity_dump) if parity_dump else None
        if self.decode_trace is not None:
            self.decode_trace.close()
        self.decode_trace = DecodeTrace(trace_decode_file, self.model.rt.device.index or 0) if trace_decode_file else None

    # ---- construction ----------------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype: str = "bfloat16", **kw) -> "Engine":
        model, _ = load_model(model_dir, dtype)
        return cls(model, **kw)

    @classmethod
    def from_config(cls, cfg, model_id: Optional[str] = None) -> "Engine":
        """From an :class:`EngineConfig` (the JSON file of the command line)."""
        from ..registry import get_architecture
        entry = cfg.model(model_id)
        if entry.random:
            arch = get_architecture(entry.random["config"]["architectures"][0])
            spec = arch.build_spec(arch.parse_config(entry.random["config"], f"models[{entry.id}].random.config"))
            model = random_model(spec, int(entry.random.get("seed", 0)), cfg.runtime.dtype)
        else:
            model, _ = load_model(entry.path, cfg.runtime.dtype)
        eng = cls(model, page_size=cfg.serving.blockSize, cache_tokens=cfg.runtime.cacheTokens,
                  max_context=cfg.runtime.maxContextTokens, token_budget=cfg.serving.tokenBudget,
                  max_active=cfg.serving.maxActiveRequests, prefill_chunk=cfg.serving.prefillChunk,
                  cache_memory_fraction=cfg.runtime.cacheMemoryFraction)
        if cfg.diagnostics.parityDump or cfg.diagnostics.traceDecodeFile:
            eng.set_diagnostics(cfg.diagnostics.parityDump, cfg.diagnostics.traceDecodeFile)
        return eng

    # ---- generation --------------------------------------------------------------------
    def serve(self, max_graph_steps: int = 0) -> "ServingLoop":
        """A loop to which requests can be added while others run (the counterpart of the reference's
        ContinuousBatcher::submit, src/runtime/serving/ContinuousBatcher.cpp:87-123).  ``max_graph_steps`` > 0 caps
        how many captured decode steps run between two chances to admit a new request."""
        return ServingLoop(self, max_graph_steps)

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 256,
                 sampling=None, stop_ids: Sequence[int] = (), use_eos: bool = True,
                 on_token: Optional[Callable[[int, int], bool]] = None) -> List[GenerateResult]:
        """Generates for every prompt (lists of token ids).  ``sampling`` is one SamplingParams for all
        or one per prompt; ``on_token(prompt index, token)`` may return False to stop that request."""
        n = len(prompts)
        if sampling is None:
            sampling = SamplingParams()
        params = list(sampling) if isinstance(sampling, (list, tuple)) else [sampling] * n
        if len(params) != n:
            raise ValueError("one SamplingParams per prompt")
        loop = self.serve()
        handles = [loop.submit(p, max_new_tokens, params[i], stop_ids, use_eos,
                               (lambda tok, i=i: on_token(i, tok)) if on_token is not None else None)
                   for i, p in enumerate(prompts)]
        loop.run_until_idle()
        self.last_metrics = loop.sched.metrics
        return [loop.result(h) for h in handles]

    def _decode_run(self, loop: "ServingLoop") -> bool:
        """Runs the current set of decoding requests through a captured graph until one of them finishes
        or the horizon ends.  Returns False (nothing done) when a graph run is not possible or not worth it."""
        sched, first_at, last_at = loop.sched, loop.first_at, loop.last_at
        reqs = list(sched.running)
        if len(reqs) > self.sched_cfg.token_budget:
            return False          # the scheduler would leave some of them out of a step: its plan decides, not this
        # soft-cap and penalties run inside the captured step, over rings of recent tokens kept on the device
        window = 0
        if any(r.sampling.penalties_active or r.sampling.final_logit_softcap > 0 for r in reqs):
            window = context_bound(max([r.sampling.penalty_window for r in reqs if r.sampling.penalties_active] + [1]), floor=16)
        mgr = self.runner.manager
        horizon = min(min(r.max_new - len(r.generated) for r in reqs),
                      min(self.sched_cfg.max_seq_len - len(r.tokens) for r in reqs))
        if horizon < self.graph_min_steps:
            return False
        if loop.max_graph_steps > 0:
            horizon = min(horizon, max(loop.max_graph_steps, self.graph_min_steps))
        longest = max(len(r.tokens) for r in reqs)
        bound = context_bound(longest + horizon)
        if bound > self.runner.max_seq_len:
            bound = self.runner.max_seq_len
        greedy = all(r.sampling.greedy for r in reqs)
        key = (len(reqs), bound, greedy, window)
        sess = self._sessions.pop(key, None)
        if sess is None:
            # every (batch size, bound, sampling kind) has a captured step of its own; the least recently used one goes
            # when there are too many (a graph keeps its activations and logits)
            while len(self._sessions) >= self.max_decode_graphs:
                self._sessions.pop(next(iter(self._sessions)))
            sess = decode_session(self.runner, len(reqs), bound, greedy=greedy, feed_back=False, penalty_window=window)
        self._sessions[key] = sess                # most recently used last
        ids = [r.id for r in reqs]
        firsts = [r.tokens[-1] for r in reqs]
        while True:
            try:
                sess.bind(ids, horizon, firsts, [r.sampling for r in reqs], [len(r.generated) for r in reqs],
                          [r.tokens for r in reqs] if window else None)
                break
            except MemoryError:
                horizon //= 2          # fewer pages ahead; below the threshold the eager path (and preemption) decides
                if horizon < self.graph_min_steps:
                    return False
        if isinstance(sess, LibraryDecodeSession):
            return self._decode_run_library(loop, sess, reqs)
        # One step of look-ahead: as soon as a step's tokens are on the host they are copied back as the next
        # step's inputs and that step is launched; the host's bookkeeping for the step runs while the GPU works.
        # If the bookkeeping finds that a request stopped (a stop id, a callback), the step already in flight is
        # still valid for the others; the stopped request's extra token is dropped.
        n = len(reqs)
        # pinned buffers are kept per batch size: allocating page-locked memory takes milliseconds and waits for the device
        if n not in self._pinned:
            self._pinned[n] = (torch.empty(n, dtype=torch.int32, pin_memory=True),
                               [torch.empty(n + 1, dtype=torch.int32, pin_memory=True) for _ in range(2)])    # tokens + the kernels' error flag
        host_in, host_out = self._pinned[n]
        stream = torch.cuda.current_stream()
        alive = [True] * n

        def account(toks, now) -> bool:
            stop = False
            for i, (r, tok) in enumerate(zip(reqs, toks)):
                if not alive[i]:
                    continue
                first_at.setdefault(r.id, now)
                last_at[r.id] = now
                done = sched.accept_token(r, tok)
                if loop.deliver(r, tok) is False and not done:
                    sched.cancel(r.id)
                    done = True
                if done:
                    alive[i] = False
                    stop = True
            return stop

        def tokens_of(buf) -> List[int]:
            vals = buf.tolist()
            if vals[n] != 0:                      # a kernel of that step gave up a bounded wait: its tokens are not valid
                sess.clear_error()
                raise KernelError("a kernel of the decode step gave up waiting on its pipeline; the step's output is not valid")
            return vals[:n]

        cur = 0
        t_prev = time.perf_counter()
        sess.step()
        host_out[cur].copy_(sess.out, non_blocking=True)
        stream.synchronize()
        while True:
            self.d2h_bytes += (n + 1) * 4
            self.graph_steps += 1
            now = time.perf_counter()
            if self.decode_trace is not None:
                self.decode_trace.step(n, (now - t_prev) * 1e3)
                t_prev = now
            toks = tokens_of(host_out[cur])
            more = sess.remaining() > 0
            if more:
                host_in.copy_(host_out[cur][:n])
                sess.token_ids.copy_(host_in, non_blocking=True)      # next step's inputs, from pinned memory
                self.h2d_bytes += n * 4
                sess.step()
                host_out[cur ^ 1].copy_(sess.out, non_blocking=True)
            stop = account(toks, now)
            if not more:
                break
            stream.synchronize()
            cur ^= 1
            if stop:
                self.d2h_bytes += (n + 1) * 4
                self.graph_steps += 1
                now = time.perf_counter()
                if self.decode_trace is not None:
                    self.decode_trace.step(n, (now - t_prev) * 1e3)
                account(tokens_of(host_out[cur]), now)
                break
        if self.decode_trace is not None:
            self.decode_trace.flush()
        return True

    def _decode_run_library(self, loop: "ServingLoop", sess: LibraryDecodeSession, reqs) -> bool:
        """The decode run with the library's session: one call per step (``cycle``) waits for the step in flight, copies its
        tokens back as the next step's inputs (from pinned memory), launches that step and accounts for the finished one in
        the library's scheduler; here the Python requests are brought up to date and the callbacks called.  A request that
        stops is dropped one step late: the step already in flight is still valid for the others."""
        sched, native = loop.sched, self.runner.native
        n = len(reqs)
        alive = [True] * n
        t_prev = time.perf_counter()
        sess.begin()
        stop_seen = False
        while True:
            more = sess.remaining() > 0 and not stop_seen
            self.graph_steps += 1                      # the step in flight, whose results this turn waits for
            toks, done, _ = sess.cycle(sched._h, more)
            sched.apply_events(native.events())
            now = time.perf_counter()
            self.d2h_bytes += (n + 1) * 4
            if more:
                self.h2d_bytes += n * 4
            if self.decode_trace is not None:
                self.decode_trace.step(n, (now - t_prev) * 1e3)
                t_prev = now
            for i, (r, tok, d) in enumerate(zip(reqs, toks, done)):
                if d < 0 or not alive[i]:
                    continue
                r.tokens.append(tok)
                r.generated.append(tok)
                loop.first_at.setdefault(r.id, now)
                loop.last_at[r.id] = now
                if d == 1:
                    alive[i] = False
                    stop_seen = True
                if loop.deliver(r, tok) is False and d == 0:
                    sched.cancel(r.id)
                    sess.drop(i)
                    alive[i] = False
                    stop_seen = True
            if not more:
                break
        if self.decode_trace is not None:
            self.decode_trace.flush()
        return True

    def _run_plan(self, plan: Sequence[PlannedEntry]) -> Dict[Hashable, int]:
        entries = [StepEntry(p.request.id, p.tokens, [p.count - 1] if p.samples else []) for p in plan]
        logits = self.runner.execute(entries)
        sampled: Dict[Hashable, int] = {}
        rows = [p for p in plan if p.samples]
        if rows:
            toks = self.sampler.sample(logits, [p.request.sampling for p in rows],
                                       [len(p.request.generated) for p in rows],
                                       [p.request.tokens for p in rows])
            host = toks.cpu().tolist()
            self.runner.check_errors()        # the copy above waited for the step: a kernel that gave up fails the step
            self.d2h_bytes += 4 * len(host)
            for p, t in zip(rows, host):
                sampled[p.request.id] = t
        return sampled


class ServingLoop:
    """Requests in, tokens out, one scheduler step (or one run of captured decode steps) per ``step()``."""

    def __init__(self, engine: Engine, max_graph_steps: int = 0):
        self.engine = engine
        self.sched = Scheduler(engine.sched_cfg, engine.runner.manager)
        self.max_graph_steps = max_graph_steps
        self.first_at: Dict[Hashable, float] = {}
        self.last_at: Dict[Hashable, float] = {}
        self._requests: Dict[int, Request] = {}
        self._callbacks: Dict[Hashable, Callable[[int], Optional[bool]]] = {}
        self._submitted_at: Dict[Hashable, float] = {}
        self._next = 0

    def submit(self, prompt: Sequence[int], max_new_tokens: int = 256, sampling: Optional[SamplingParams] = None,
               stop_ids: Sequence[int] = (), use_eos: bool = True,
               on_token: Optional[Callable[[int], Optional[bool]]] = None) -> int:
        """Queues a request and returns its handle.  ``on_token(token)`` is called for every generated token and may
        return False to stop the request.  A request that can never run is finished at once (``result`` says why)."""
        handle = self._next
        self._next += 1
        stops = tuple(stop_ids) + (self.engine.eos_ids if use_eos else ())
        req = Request(id=("gen", handle), prompt=list(prompt), max_new=max_new_tokens,
                      sampling=(sampling or SamplingParams()).resolved(), stop_ids=stops)
        self._requests[handle] = req
        self._submitted_at[req.id] = time.perf_counter()
        if on_token is not None:
            self._callbacks[req.id] = on_token
        self.sched.add(req)
        return handle

    def deliver(self, req: Request, tok: int) -> Optional[bool]:
        cb = self._callbacks.get(req.id)
        return cb(tok) if cb is not None else None

    def has_work(self) -> bool:
        return self.sched.has_work()

    def step(self) -> bool:
        """One unit of work.  Returns whether anything is left to do."""
        eng, sched = self.engine, self.sched
        if not sched.has_work():
            return False
        if eng.use_graphs and sched.all_decoding():
            running = list(sched.running)
            try:
                ran = eng._decode_run(self)
            except Exception as e:
                self._fail(running, e)
                raise
            if ran:
                return sched.has_work()
        if eng.runner.native is not None and eng.runner.stage_dump is None:
            return self._library_step()
        plan = sched.schedule()
        if not plan:
            if sched.has_work():
                raise RuntimeError("scheduler made no progress")   # cannot happen: a lone request fails instead
            return False
        t_step = time.perf_counter()
        try:
            sampled = eng._run_plan(plan)
        except Exception as e:
            self._fail([p.request for p in plan], e)
            raise
        now = time.perf_counter()
        if eng.decode_trace is not None and all(p.count == 1 and p.samples for p in plan):
            eng.decode_trace.step(len(plan), (now - t_step) * 1e3)
            eng.decode_trace.flush()
        for p in plan:
            if p.samples:
                self.first_at.setdefault(p.request.id, now)
                self.last_at[p.request.id] = now
        sched.commit(plan, sampled)
        for p in plan:
            if p.samples and self.deliver(p.request, sampled[p.request.id]) is False and p.request.state != "finished":
                sched.cancel(p.request.id)
        return sched.has_work()

    def _library_step(self) -> bool:
        """A scheduler step inside the library: plan, step, sampling, the wait for the tokens and the commit are one call
        (csrc/exec/executor.cu, run_plan); what is left here is to bring the Python requests up to date and to call back."""
        eng, sched = self.engine, self.sched
        native = eng.runner.native
        t_step = time.perf_counter()
        try:
            handles, toks = native.run_plan(sched._h)
        except Exception as e:
            sched.apply_events(native.events())            # what the call did before it failed (admissions, preemptions)
            self._fail([p.request for p in sched.last_plan(native.planned())], e)
            raise
        sched.apply_events(native.events())
        planned = native.planned()
        if planned == 0:
            if sched.has_work():
                raise RuntimeError("scheduler made no progress")   # cannot happen: a lone request fails instead
            return False
        now = time.perf_counter()
        eng.d2h_bytes += 4 * len(toks)
        if eng.decode_trace is not None and len(toks) == planned and all(p.count == 1 for p in sched.last_plan(planned)):
            eng.decode_trace.step(planned, (now - t_step) * 1e3)
            eng.decode_trace.flush()
        for h, tok in zip(handles, toks):
            req = sched.request_of(h)
            req.tokens.append(tok)
            req.generated.append(tok)
            self.first_at.setdefault(req.id, now)
            self.last_at[req.id] = now
        for h, tok in zip(handles, toks):
            req = sched.request_of(h)
            if self.deliver(req, tok) is False and req.state != "finished":
                sched.cancel(req.id)
        return sched.has_work()

    def _fail(self, requests, error: Exception) -> None:
        """A step that raised ends the requests it held (finish reason "error: ..."), as a failed batched step fails its
        requests in the reference (src/runtime/serving/ContinuousBatcher.cpp:417-429); their pages and slots go back, the
        requests that were not in the step and the loop itself stay usable, and the caller gets the exception."""
        for r in requests:
            if r.state != "finished":
                self.sched.cancel(r.id, reason=f"error: {type(error).__name__}: {error}"[:200])

    def run_until_idle(self) -> None:
        while self.step():
            pass

    def cancel(self, handle: int) -> bool:
        return self.sched.cancel(self._requests[handle].id)

    def finished(self, handle: int) -> bool:
        return self._requests[handle].state == "finished"

    def result(self, handle: int) -> GenerateResult:
        """Tokens and statistics of a request (complete once ``finished(handle)``)."""
        r = self._requests[handle]
        st = GenerateStats(prompt_tokens=len(r.prompt), generated_tokens=len(r.generated),
                           hit_stop=r.hit_stop, finish_reason=r.finish_reason or "", preemptions=r.preemptions)
        if r.id in self.first_at:
            st.prefill_ms = (self.first_at[r.id] - self._submitted_at[r.id]) * 1e3
            st.decode_ms = (self.last_at[r.id] - self.first_at[r.id]) * 1e3
        return GenerateResult(list(r.generated), st)
