"""The step function: one batch of (request, its next tokens) through the model.

A batch holds, for each request in it, the request's next tokens: a portion of a prompt of
any length, or a single decoded token.  The step runs only those tokens, reading earlier
keys and values from the cache, writes the new ones at positions ``[len, len + n)``, and
returns fp32 logits at the wanted places only (final norm and head run on the gathered
rows).  The reference has two separate calls for this, a one-token-per-slot step and a
per-request prefill (src/runtime/engine/ServingSession.cpp:856-947, 949-1093), and a
per-position logits primitive (src/runtime/InferenceEngine.cpp:2332-2441); its
``BatchSchedule{decodes, prefills}`` describes a mixed iteration that nothing executes
(src/runtime/serving/ChunkedPrefillScheduler.hpp:65-72).  Here it is one call.

Commit protocol: pages are reserved before the launch, the cache lengths advance only
after the step was enqueued without error (src/runtime/KvCache.hpp:90-103).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..kernels import ops
from ..parts.base import Runtime, StepContext
from . import native
from .model import Model
from .storage import CacheStorage

class StepError(RuntimeError):
    pass


@dataclass
class StepEntry:
    """One request's share of a step."""

    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()   # indices into ``tokens`` whose logits are returned


class ModelRunner:
    def __init__(self, model: Model, page_size: int, num_pages, max_requests: int, max_seq_len: Optional[int] = None):
        self.model = model
        self.rt: Runtime = model.rt
        self.max_seq_len = int(max_seq_len or model.spec.max_positions)
        self.manager = CacheManager(model.cache_groups(), page_size, num_pages, max_requests)
        self.storage = CacheStorage(model, self.manager, self.rt)
        self.page_size = page_size
        self.vocab = model.spec.vocab_size
        self.steps_run = 0
        self.stage_dump = None       # engine.diagnostics.StageDump: steps with a prompt portion write their stages
        # The library's executor when every part of the model has a native class, else None: then steps are put
        # together and launched here, part by part, through the Python classes.
        self.native: Optional[native.NativeExecutor] = native.NativeExecutor.build(model, self.storage, self.manager, self.max_seq_len)

    # ---- request life cycle ---------------------------------------------------
    def add_request(self, rid: Hashable) -> bool:
        return self.manager.add_request(rid) is not None

    def release(self, rid: Hashable) -> None:
        self.manager.release(rid)

    def length(self, rid: Hashable) -> int:
        return self.manager.length(rid)

    # ---- batch assembly ---------------------------------------------------------
    def _build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        mgr, ps = self.manager, self.page_size
        n_req = len(entries)
        q_start, q_len, kv_len, slots = [], [], [], []
        n_tok = 0
        for e in entries:
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r}: an entry needs at least one token")
            start = mgr.length(e.request)
            q_start.append(n_tok)
            q_len.append(n)
            kv_len.append(start + n)
            slots.append(mgr.slot(e.request))
            n_tok += n
        ids = np.empty(n_tok, dtype=np.int32)
        pos = np.empty(n_tok, dtype=np.int32)
        req = np.empty(n_tok, dtype=np.int32)
        rows: List[int] = []
        for r, e in enumerate(entries):
            s, n = q_start[r], q_len[r]
            toks = np.asarray(e.tokens, dtype=np.int64)
            if toks.min() < 0 or toks.max() >= self.vocab:
                raise StepError(f"request {e.request!r}: token id outside [0, {self.vocab})")
            ids[s:s + n] = toks
            pos[s:s + n] = np.arange(kv_len[r] - n, kv_len[r], dtype=np.int32)
            req[s:s + n] = r
            for w in e.want:
                if not (0 <= w < n):
                    raise StepError(f"request {e.request!r}: wanted place {w} is outside its {n} tokens")
                rows.append(s + w)
        max_kv = max(kv_len)
        width = max(1, (max_kv + ps - 1) // ps)
        tables = {}
        rids = [e.request for e in entries]
        for name in mgr.groups:
            t = np.empty((n_req, width), dtype=np.int32)
            mgr.fill_tables(name, rids, width, t.ctypes.data)      # -1 beyond a table's end
            tables[name] = t
        meta = np.stack([np.asarray(q_start, np.int32), np.asarray(q_len, np.int32), np.asarray(kv_len, np.int32),
                         np.asarray(slots, np.int32)], axis=1)
        # one pinned staging buffer, one copy
        parts = [ids, pos, req, meta.reshape(-1), np.asarray(rows, dtype=np.int32)] + [tables[g].reshape(-1) for g in tables]
        sizes = [p.size for p in parts]
        total = sum(sizes)
        host = torch.empty(max(total, 1), dtype=torch.int32, pin_memory=True)
        hv = host.numpy()
        off = 0
        for p in parts:
            hv[off:off + p.size] = p
            off += p.size
        dev = host.to(self.rt.device, non_blocking=True)
        views = []
        off = 0
        for sz in sizes:
            views.append(dev[off:off + sz])
            off += sz
        d_ids, d_pos, d_req, d_meta, d_rows = views[:5]
        d_tables = {g: views[5 + i].view(n_req, width) for i, g in enumerate(tables)}
        return StepContext(
            n_tokens=n_tok, n_requests=n_req, token_ids=d_ids, positions=d_pos, token_req=d_req,
            q_start=q_start, q_len=q_len, kv_len=kv_len, req_meta=d_meta.view(n_req, 4),
            state_slots=d_meta.view(n_req, 4)[:, 3].contiguous(), block_tables=d_tables, logit_rows=d_rows,
            n_logit_rows=len(rows), page_size=ps, runtime=self.rt, max_kv_len=max_kv, max_q_len=max(q_len))

    # ---- the step -----------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs one batch.  Returns fp32 logits [wanted, vocab] in the order of the entries and of
        their ``want`` lists, or None if nothing was wanted."""
        if not entries:
            return None
        mgr = self.manager
        if self.native is not None and self.stage_dump is None:
            logits = self._run_native(entries, reserve=True, commit=True)       # checks, pages, launches, lengths: one call
            self.steps_run += 1
            return logits
        seen = set()
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if not mgr.has(e.request):
                raise StepError(f"unknown request {e.request!r}")
            new_len = mgr.length(e.request) + len(e.tokens)
            if new_len > self.max_seq_len:
                raise StepError(f"request {e.request!r}: {new_len} tokens exceed the context of {self.max_seq_len}")
        # pages for every entry: the step runs fully or not at all
        need: Dict[str, int] = {g: 0 for g in mgr.groups}
        for e in entries:
            for g, n in mgr.pages_needed(e.request, mgr.length(e.request) + len(e.tokens)).items():
                need[g] += n
        for g, n in need.items():
            if n > mgr.free_pages(g):
                raise StepError(f"out of cache pages in group {g}: the step needs {n}, "
                                f"{mgr.free_pages(g)} of {mgr.total_pages(g)} are free")
        for e in entries:
            ok = mgr.reserve(e.request, mgr.length(e.request) + len(e.tokens))
            assert ok
        logits = self.execute(entries)
        for e in entries:
            mgr.commit(e.request, mgr.length(e.request) + len(e.tokens))
        self.steps_run += 1
        return logits

    def execute(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the model on entries whose pages are reserved (by ``step`` or by a scheduler); lengths are not
        committed here.  Returns fp32 logits [wanted, vocab] or None."""
        mgr = self.manager
        if self.native is not None and not (self.stage_dump is not None and any(len(e.tokens) > 1 for e in entries)):
            return self._run_native(entries, reserve=False, commit=False)
        for e in entries:
            if mgr.mark_started(e.request):
                self.storage.zero_slot(mgr.slot(e.request))
        ctx = self._build_context(entries)
        if self.stage_dump is not None and any(len(e.tokens) > 1 for e in entries):
            ctx.plain_only = True
            return self.forward(ctx, dump=self.stage_dump)
        return self.forward(ctx)

    def _run_native(self, entries: Sequence[StepEntry], reserve: bool, commit: bool) -> Optional[torch.Tensor]:
        mgr = self.manager
        try:
            handles = [mgr.handle(e.request) for e in entries]
        except Exception:
            missing = next(e.request for e in entries if not mgr.has(e.request))
            raise StepError(f"unknown request {missing!r}") from None
        try:
            return self.native.run(handles, [e.tokens for e in entries], [e.want for e in entries], reserve, commit)
        except native.StepRefused as e:
            raise StepError(str(e)) from None

    def check_errors(self) -> None:
        """To be called after the host has waited for a step's results (a copy of tokens or logits): raises if one of
        the step's kernels gave up a bounded wait, since its output is then not valid.  With the library's executor
        the flag came back with the step (no further synchronisation); otherwise it is read here."""
        if self.native is not None:
            if self.native.take_error_flag() == 0:
                return
            ops.tcgen05_error_flag(self.rt.device).zero_()
            raise ops.KernelError("a kernel of the step gave up waiting on its pipeline; the step's output is not valid")
        ops.check_tcgen05_errors(self.rt.device)

    def forward(self, ctx: StepContext, dump=None) -> Optional[torch.Tensor]:
        """The launches of a step whose context is on the device: by the library's executor, or part by part here."""
        if self.native is not None and dump is None and not ctx.plain_only:
            return self.native.forward(ctx)
        m = self.model
        residual = m.embedding.forward(ctx.token_ids)
        if dump is not None:
            dump.write(0, "inp_scaled", residual)
        pending = None
        last = len(m.schedule) - 1
        for i, e in enumerate(m.schedule):
            if dump is not None:
                ctx.dump = lambda stage, rows, block=i: dump.write(block, stage, rows)
            successor = m.layers[m.schedule[i + 1].layer] if i < last else None
            pending = m.layers[e.layer].forward(residual, pending, ctx, self.storage.layer_cache(i, ctx), successor=successor)
        if ctx.n_logit_rows == 0:
            return None
        normed = m.final_norm.forward(residual, pending, rows=ctx.logit_rows, n_rows=ctx.n_logit_rows)
        return m.head.forward(normed)
