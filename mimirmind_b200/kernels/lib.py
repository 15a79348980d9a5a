"""ctypes binding of the CUDA kernel library.

The library exports plain C entry points (``mm_*``) that take device pointers, sizes
and a stream and return an error code; this module loads it, declares the prototypes
and turns a non-zero code into :class:`KernelError` carrying the library's message.
There is no fallback: if the library cannot be built or loaded, the error surfaces.
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p
from typing import Optional

from .build import library_path


class KernelError(RuntimeError):
    pass


_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None

P = c_void_p
I = c_int
F = c_float

_PROTOTYPES = {
    "mm_embedding": [P, P, I, P, I, I, I, F, P],
    "mm_add_rmsnorm": [P, P, P, P, I, P, I, I, I, F, P],
    "mm_add_residual": [P, P, I, c_longlong, P],
    "mm_silu_mul": [P, P, I, I, I, I, P],
    "mm_gemm_tcgen05": [P, P, P, I, P, I, I, I, I, I, I, P, P],
    "mm_gemm_tcgen05_pair": [P, P, P, I, P, I, I, I, I, I, I, P, P],
    "mm_gemv_bf16": [P, P, P, I, P, I, I, I, I, I, I, I, I, I, P, I, I, F, P],
    "mm_gemv_bf16_residual": [P, P, P, P, I, P, P, I, I, I, I, I, I, P, I, I, F, P],
    "mm_gemv_bf16_qkv_rope": [P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, I, P, I, I, F, P],
    "mm_gemm_skinny": [P, P, P, I, P, I, I, I, I, I, I, I, I, P, I, I, I, F, P, P],
    "mm_gemm_skinny_residual": [P, P, P, P, I, P, P, I, I, I, I, I, I, P, I, I, I, F, P, P],
    "mm_gemm_skinny_qkv_rope": [P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, I, P, I, I, I, F, P, P],
    "mm_rope_table": [P, P, I, I, F, P],
    "mm_slot_mapping": [P, P, P, I, I, I, P, P],
    "mm_qkv_rope_kvwrite": [P, P, I, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, I, P],
    "mm_qkv_rope_tables": [P, P, I, P, P, P, P, P, I, I, I, I, I, I, P],
    "mm_gather_rows": [P, P, P, I, I, I, P],
    "mm_attention_generic": [P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, P],
    "mm_gemm_simt": [P, I, P, I, P, I, P, I, I, I, I, I, I, P],
    "mm_argmax_rows": [P, P, I, I, P],
    "mm_argmax_rows_split": [P, P, P, P, I, I, I, P],
    "mm_sample_rows": [P, P, I, I, P, P, P, P, P, P],
    "mm_apply_penalties": [P, I, I, P, I, P, P, P, P, P],
    "mm_window_push": [P, I, I, P, P, P, P],
}


def load(verbose: bool = True) -> ctypes.CDLL:
    global _lib
    if _lib is not None:          # the usual case, without the lock: every launch comes through here
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = library_path(build_if_needed=True, verbose=verbose)
        lib = ctypes.CDLL(path)
        lib.mm_last_error.restype = ctypes.c_char_p
        lib.mm_last_error.argtypes = []
        lib.mm_set_pdl.argtypes = [c_int]
        lib.mm_set_pdl.restype = None
        lib.mm_get_pdl.argtypes = []
        lib.mm_get_pdl.restype = c_int
        lib.mm_set_gemv_blocks.argtypes = [c_int]
        lib.mm_set_gemv_blocks.restype = c_int
        lib.mm_launch_count.argtypes = []
        lib.mm_launch_count.restype = c_longlong
        lib.mm_uniform_from.restype = c_float
        lib.mm_uniform_from.argtypes = [c_ulonglong, c_ulonglong]
        for name, args in _PROTOTYPES.items():
            fn = getattr(lib, name, None)
            if fn is None:
                continue  # optional kernels are declared by the module that binds them
            fn.restype = c_int
            fn.argtypes = args
        _lib = lib
        return lib


def declare(name: str, argtypes, restype=c_int):
    """Declare the prototype of an entry point that is not in the core table."""
    lib = load()
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


def launch_count() -> int:
    """Kernels of this library launched (or recorded into a graph under capture) so far."""
    return int(load().mm_launch_count())


def check(code: int, what: str) -> None:
    if code != 0:
        msg = load().mm_last_error().decode("utf-8", "replace")
        raise KernelError(f"{what} failed (code {code}): {msg}")
