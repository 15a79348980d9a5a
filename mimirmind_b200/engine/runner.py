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
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..kernels import ops
from ..parts.base import Runtime, StepContext
from .model import Model
from .storage import CacheStorage

# A prompt portion of one request with at least this many tokens, of a size seen before, runs as a replayed CUDA
# graph (engine/prefill_graph.py); at most PREFILL_GRAPHS sizes are kept.  0 turns it off.
PREFILL_GRAPH_MIN_TOKENS = 512
PREFILL_GRAPHS = 4


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
        self._prefill_sessions: Dict[Tuple[int, bool], object] = {}
        self._prefill_seen: Dict[Tuple[int, bool], int] = {}
        self.stage_dump = None       # engine.diagnostics.StageDump: steps with a prompt portion write their stages

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
        for e in entries:
            if mgr.mark_started(e.request):
                self.storage.zero_slot(mgr.slot(e.request))
        if self.stage_dump is not None and any(len(e.tokens) > 1 for e in entries):
            ctx = self._build_context(entries)
            ctx.plain_only = True
            return self.forward(ctx, dump=self.stage_dump)
        session = self._prefill_session(entries)
        if session is not None:
            e = entries[0]
            return session.run(e.request, e.tokens, mgr.length(e.request))
        return self.forward(self._build_context(entries))

    def _prefill_session(self, entries: Sequence[StepEntry]):
        """The graph session for this step, or None: one request, bfloat16, a long portion whose size was seen
        before, logits wanted at its last token or nowhere."""
        if (PREFILL_GRAPH_MIN_TOKENS <= 0 or len(entries) != 1 or self.rt.dtype != torch.bfloat16
                or len(entries[0].tokens) < PREFILL_GRAPH_MIN_TOKENS):
            return None
        e = entries[0]
        n = len(e.tokens)
        want = list(e.want)
        if want not in ([], [n - 1]):
            return None
        if min(e.tokens) < 0 or max(e.tokens) >= self.vocab:
            raise StepError(f"request {e.request!r}: token id outside [0, {self.vocab})")
        key = (n, bool(want))
        sess = self._prefill_sessions.get(key)
        if sess is None:
            self._prefill_seen[key] = self._prefill_seen.get(key, 0) + 1
            if self._prefill_seen[key] < 2:
                return None                      # a size seen once is not worth a capture
            if len(self._prefill_sessions) >= PREFILL_GRAPHS:
                self._prefill_sessions.pop(next(iter(self._prefill_sessions)))
            from .prefill_graph import PrefillSession
            sess = PrefillSession(self, n, bool(want))
            self._prefill_sessions[key] = sess
        return sess

    def forward(self, ctx: StepContext, dump=None) -> Optional[torch.Tensor]:
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
