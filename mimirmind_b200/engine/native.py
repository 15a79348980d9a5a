"""The native step executor's Python side: hands a model's parts over as descriptions and calls the step.

A model whose parts all describe themselves (``Part.native``) and whose kinds all have a C++ class
(``csrc/exec/parts_builtin.cu``) runs its steps in the library: one call assembles the step's integers, copies
them to the device and launches every layer, as the reference's native backend does for a block
(src/runtime/arch/Qwen2Backend.cpp:132-466).  A model with a part that exists in Python only (the toy parts of
the tests, a new part that has no C++ class yet) gets no executor and steps through the Python part classes.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_double, c_int, c_longlong, c_void_p
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..kernels import lib as _lib
from ..kernels import ops
from ..kernels.lib import KernelError
from ..parts.base import NativeDesc, StepContext

ENABLED = True          # False: every model steps through the Python part classes (tests compare the two)
MAX_GROUPS = 8
RUN_RESERVE, RUN_COMMIT = 1, 2
REFUSED = -10


class StepRefused(RuntimeError):
    """The step was refused before anything ran: the message says why."""


class _StepDesc(ctypes.Structure):
    _fields_ = [("n_tokens", c_int), ("n_requests", c_int), ("n_logit_rows", c_int), ("max_kv_len", c_int), ("max_q_len", c_int),
                ("table_width", c_int), ("token_ids", c_void_p), ("positions", c_void_p), ("token_req", c_void_p),
                ("logit_rows", c_void_p), ("tables", c_void_p * MAX_GROUPS), ("q_start", POINTER(c_int)),
                ("q_len", POINTER(c_int)), ("kv_len", POINTER(c_int))]


_declared = False


def _declare():
    global _declared
    lib = _lib.load()
    if _declared:
        return lib
    P, I, L = c_void_p, c_int, c_longlong
    for name, res, args in (
        ("mmx_last_error", c_char_p, []),
        ("mmx_desc_new", P, [c_char_p]),
        ("mmx_desc_free", None, [P]),
        ("mmx_desc_num", None, [P, c_char_p, c_double]),
        ("mmx_desc_tensor", I, [P, c_char_p, P, I, I, POINTER(L)]),
        ("mmx_desc_child", None, [P, c_char_p, P]),
        ("mmx_model_create", P, [P, P, P, I, POINTER(P), I, POINTER(I), POINTER(I), I, I]),
        ("mmx_model_destroy", None, [P]),
        ("mmx_exec_create", P, [P, P, I, I, POINTER(I), I, POINTER(P), POINTER(P), POINTER(I), POINTER(I), I, I, P]),
        ("mmx_exec_destroy", None, [P]),
        ("mmx_exec_run", I, [P, I, P, P, P, P, P, I, P, L, P]),
        ("mmx_exec_forward", I, [P, POINTER(_StepDesc), P, P]),
        ("mmx_exec_run_plan", I, [P, P, POINTER(L), POINTER(I), I, P]),
        ("mmx_exec_planned", I, [P]),
        ("mmx_exec_events", I, [P, POINTER(L), POINTER(I), POINTER(I), I]),
        ("mmx_decode_create", P, [P, I, I, I, I, I]),
        ("mmx_decode_destroy", None, [P]),
        ("mmx_decode_bind", I, [P, P, I, P, P, P, P, P, P, P, P, P, P, P]),
        ("mmx_decode_step", I, [P, P]),
        ("mmx_decode_begin", I, [P, P]),
        ("mmx_decode_cycle", I, [P, P, P, I, P, P, P]),
        ("mmx_decode_drop", None, [P, I]),
        ("mmx_decode_info", I, [P, I]),
        ("mmx_decode_buffer", P, [P, I]),
        ("mmx_exec_take_error_flag", I, [P]),
        ("mmx_exec_stat", L, [P, I]),
        ("mmx_option", I, [c_char_p, I]),
    ):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _declared = True
    return lib


def last_error() -> str:
    return _declare().mmx_last_error().decode("utf-8", "replace")


def option(name: str, value: int = -1) -> int:
    """Reads (value < 0) or sets a tunable of the native dispatch; returns the old value."""
    old = _declare().mmx_option(name.encode(), int(value))
    if old < 0:
        raise KeyError(name)
    return old


def _to_c(lib, d: NativeDesc):
    h = lib.mmx_desc_new(d.kind.encode())
    for k, v in d.numbers.items():
        lib.mmx_desc_num(h, k.encode(), float(v))
    for k, t in d.tensors.items():
        if not t.is_cuda or not t.is_contiguous():
            lib.mmx_desc_free(h)
            raise KernelError(f"part '{d.kind}': tensor '{k}' must be a contiguous CUDA tensor")
        shape = (c_longlong * max(1, t.dim()))(*t.shape)
        if lib.mmx_desc_tensor(h, k.encode(), t.data_ptr(), ops.dtype_code(t.dtype), t.dim(), shape) != 0:
            lib.mmx_desc_free(h)
            raise KernelError(f"part '{d.kind}': tensor '{k}' cannot be described")
    for k, c in d.children.items():
        lib.mmx_desc_child(h, k.encode(), _to_c(lib, c))
    return h


class NativeExecutor:
    """Owns the library's model and executor objects of one ModelRunner."""

    def __init__(self, lib, model_h, exec_h, keep, vocab: int, device, groups: List[str]):
        self._lib, self._model, self._exec, self._keep = lib, model_h, exec_h, keep
        self.vocab, self.device, self.groups = vocab, device, groups

    def __del__(self):
        lib = getattr(self, "_lib", None)
        if lib is None:
            return
        if getattr(self, "_exec", None):
            lib.mmx_exec_destroy(self._exec)
            self._exec = None
        if getattr(self, "_model", None):
            lib.mmx_model_destroy(self._model)
            self._model = None

    # ---- construction -------------------------------------------------------------------------------------------
    @classmethod
    def build(cls, model, storage, manager, max_seq_len: int) -> Optional["NativeExecutor"]:
        """The executor of ``model`` over ``storage``'s pools, or None when a part of the model has no native class."""
        if not ENABLED or model.state_specs():
            return None
        descs = {"embedding": model.embedding.native(), "final_norm": model.final_norm.native(), "head": model.head.native()}
        blocks = [layer.native() for layer in model.layers]
        if any(d is None for d in descs.values()) or any(b is None for b in blocks) or len(manager.groups) > MAX_GROUPS:
            return None
        lib = _declare()
        handles = []
        try:
            c_top = {k: _to_c(lib, d) for k, d in descs.items()}
            handles += list(c_top.values())
            c_blocks = [_to_c(lib, b) for b in blocks]
            handles += c_blocks
            n_sched = len(model.schedule)
            sched_layer = (c_int * n_sched)(*[e.layer for e in model.schedule])
            sched_from = (c_int * n_sched)(*[-1 if e.cache_from is None else e.cache_from for e in model.schedule])
            model_h = lib.mmx_model_create(c_top["embedding"], c_top["final_norm"], c_top["head"], len(c_blocks),
                                           (c_void_p * max(1, len(c_blocks)))(*c_blocks), n_sched, sched_layer, sched_from,
                                           ops.dtype_code(model.rt.dtype), int(model.rt.matmul == "simt"))
        finally:
            for h in handles:
                lib.mmx_desc_free(h)
        if not model_h:
            return None                       # a kind without a native class: the message is in last_error()
        group_names = list(manager.groups)
        pages = (c_int * max(1, len(group_names)))(*[manager.allocators[g].num_pages for g in group_names])
        k_ptrs, v_ptrs, entry_group, entry_writes = [], [], [], []
        for i, e in enumerate(model.schedule):
            owner = i if e.cache_from is None else e.cache_from
            where = storage.entry_pool(owner)
            if where is None:
                k_ptrs.append(None), v_ptrs.append(None), entry_group.append(-1)
            else:
                name, j = where
                pool = storage.pools[name]
                k_ptrs.append(pool["k"][j].data_ptr()), v_ptrs.append(pool["v"][j].data_ptr()), entry_group.append(group_names.index(name))
            entry_writes.append(int(e.cache_from is None))
        n = len(model.schedule)
        exec_h = lib.mmx_exec_create(model_h, manager._h, len(group_names), manager.page_size, pages, n,
                                     (c_void_p * max(1, n))(*k_ptrs), (c_void_p * max(1, n))(*v_ptrs),
                                     (c_int * max(1, n))(*entry_group), (c_int * max(1, n))(*entry_writes),
                                     model.spec.vocab_size, int(max_seq_len), ops.tcgen05_error_flag(model.rt.device).data_ptr())
        if not exec_h:
            msg = last_error()
            lib.mmx_model_destroy(model_h)
            raise KernelError(f"the native executor could not be created: {msg}")
        # the model's tensors, the pools and the manager must outlive the executor
        return cls(lib, model_h, exec_h, (model, storage, manager), model.spec.vocab_size, model.rt.device, group_names)

    # ---- steps --------------------------------------------------------------------------------------------------------
    def run(self, handles: Sequence[int], tokens: Sequence[Sequence[int]], wants: Sequence[Sequence[int]],
            reserve: bool, commit: bool) -> Optional[torch.Tensor]:
        """One step for the requests with the library's ids ``handles``.  Returns fp32 logits [wanted, vocab] or None."""
        n = len(handles)
        counts = np.fromiter((len(t) for t in tokens), dtype=np.int32, count=n)
        n_want = np.fromiter((len(w) for w in wants), dtype=np.int32, count=n)
        rows = int(n_want.sum())
        try:
            flat = np.concatenate([np.asarray(t, dtype=np.int64) for t in tokens]) if n else np.zeros(0, np.int64)
        except (TypeError, ValueError) as e:
            raise StepRefused(f"token ids must be integers: {e}") from None
        if flat.size and (flat.min() < 0 or flat.max() >= self.vocab):
            raise StepRefused(f"token id outside [0, {self.vocab})")
        flat = flat.astype(np.int32)
        want = np.fromiter((w for ws in wants for w in ws), dtype=np.int32, count=rows)
        rids = np.asarray(handles, dtype=np.int64)
        logits = torch.empty((rows, self.vocab), dtype=torch.float32, device=self.device) if rows else None
        rc = self._lib.mmx_exec_run(self._exec, n, rids.ctypes.data, counts.ctypes.data, flat.ctypes.data, n_want.ctypes.data,
                                    want.ctypes.data, (RUN_RESERVE if reserve else 0) | (RUN_COMMIT if commit else 0),
                                    logits.data_ptr() if logits is not None else None, rows, ops._stream())
        if rc == REFUSED:
            raise StepRefused(last_error())
        if rc < 0:
            raise KernelError(last_error())
        return logits

    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """The launches of a step whose integers the caller keeps on the device (a captured decode step)."""
        d = _StepDesc()
        nr = ctx.n_requests
        d.n_tokens, d.n_requests, d.n_logit_rows = ctx.n_tokens, nr, ctx.n_logit_rows
        d.max_kv_len, d.max_q_len = ctx.max_kv_len, ctx.max_q_len
        width = 1
        for i, g in enumerate(self.groups):
            t = ctx.block_tables[g]
            d.tables[i] = t.data_ptr()
            width = t.shape[1]
        d.table_width = width
        d.token_ids, d.positions, d.token_req = ctx.token_ids.data_ptr(), ctx.positions.data_ptr(), ctx.token_req.data_ptr()
        d.logit_rows = ctx.logit_rows.data_ptr() if ctx.n_logit_rows else None
        qs, ql, kl = (c_int * nr)(*ctx.q_start), (c_int * nr)(*ctx.q_len), (c_int * nr)(*ctx.kv_len)
        d.q_start, d.q_len, d.kv_len = qs, ql, kl
        logits = torch.empty((ctx.n_logit_rows, self.vocab), dtype=torch.float32, device=self.device) if ctx.n_logit_rows else None
        rc = self._lib.mmx_exec_forward(self._exec, ctypes.byref(d), logits.data_ptr() if logits is not None else None, ops._stream())
        if rc < 0:
            raise KernelError(last_error())
        return logits

    def run_plan(self, scheduler_handle) -> "tuple[list, list]":
        """One step of the library's scheduler: plan, launches, sampling, the wait for the tokens, commit, all in one
        call.  Returns (request ids, sampled tokens) of the entries that sampled; ``planned()`` and ``events()`` tell
        the rest.  Raises KernelError when the step failed (the plan stays readable from the scheduler)."""
        cap = 1024
        if not hasattr(self, "_plan_rids"):
            self._plan_rids, self._plan_toks = (c_longlong * cap)(), (c_int * cap)()
            self._ev = ((c_longlong * 512)(), (c_int * 512)(), (c_int * 512)())
        n = self._lib.mmx_exec_run_plan(self._exec, scheduler_handle, self._plan_rids, self._plan_toks, cap, ops._stream())
        if n < 0:
            raise KernelError(last_error())
        return list(self._plan_rids[:n]), list(self._plan_toks[:n])

    def planned(self) -> int:
        """Entries of the plan that the last ``run_plan`` ran (0: the scheduler had nothing to run)."""
        return int(self._lib.mmx_exec_planned(self._exec))

    def events(self):
        """What the last ``run_plan`` did to requests: (request id, kind, code) in order."""
        if not hasattr(self, "_ev"):
            return []
        r, k, c = self._ev
        n = self._lib.mmx_exec_events(self._exec, r, k, c, len(r))
        if n > len(r):
            self._ev = r, k, c = (c_longlong * n)(), (c_int * n)(), (c_int * n)()
            n = self._lib.mmx_exec_events(self._exec, r, k, c, n)
        return [(r[i], k[i], c[i]) for i in range(n)]

    def take_error_flag(self) -> int:
        """The kernels' error flag as the last ``run`` copied it back (after a synchronisation); reading clears it."""
        return int(self._lib.mmx_exec_take_error_flag(self._exec))

    def steps(self) -> int:
        return int(self._lib.mmx_exec_stat(self._exec, 0))

    def memory_bytes(self) -> int:
        return int(self._lib.mmx_exec_stat(self._exec, 1))
