"""Loads the host runtime library (``csrc/host``: page allocator, cache manager, scheduler in C++) and declares
its C interface.  The library has no CUDA in it: it is built with the host compiler at first use and works on a
machine without a GPU."""
from __future__ import annotations

import ctypes
import threading
from ctypes import POINTER, c_char_p, c_float, c_int, c_longlong, c_void_p
from typing import Optional

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None

P, I, L = c_void_p, c_int, c_longlong
PI, PL = POINTER(c_int), POINTER(c_longlong)

_PROTOTYPES = {
    # name: (result type, argument types)
    "mmh_last_error": (c_char_p, []),
    "mmh_alloc_create": (P, [I]),
    "mmh_alloc_destroy": (None, [P]),
    "mmh_alloc_alloc": (I, [P]),
    "mmh_alloc_free": (I, [P, I]),
    "mmh_alloc_is_allocated": (I, [P, I]),
    "mmh_alloc_check": (I, [P]),
    "mmh_alloc_stat": (L, [P, I]),
    "mmh_cache_create": (P, [I, PI, PI, I, I]),
    "mmh_cache_destroy": (None, [P]),
    "mmh_cache_has": (I, [P, L]),
    "mmh_cache_add": (I, [P, L]),
    "mmh_cache_request": (I, [P, L, I]),
    "mmh_cache_pages_needed": (I, [P, L, I, PI]),
    "mmh_cache_reserve": (I, [P, L, I]),
    "mmh_cache_commit": (I, [P, L, I]),
    "mmh_cache_release": (I, [P, L]),
    "mmh_cache_table": (I, [P, L, I, PI, I]),
    "mmh_cache_tables": (I, [P, I, I, PL, I, c_void_p]),
    "mmh_cache_allocator": (P, [P, I]),
    "mmh_cache_info": (I, [P, I, I]),
    "mmh_cache_live": (I, [P, PL, I]),
    "mmh_cache_check": (I, [P]),
    "mmh_engine_config": (c_char_p, [c_char_p, L, c_char_p]),
    "mmh_config_qwen2": (c_char_p, [c_char_p, L, c_char_p]),
    "mmh_config_qwen2_folder": (c_char_p, [c_char_p]),
    "mmh_st_parse_header": (P, [c_void_p, L, L, c_char_p]),
    "mmh_st_open_folder": (P, [c_char_p]),
    "mmh_st_close": (None, [P]),
    "mmh_st_count": (I, [P]),
    "mmh_st_name": (c_char_p, [P, I]),
    "mmh_st_dtype": (c_char_p, [P, I]),
    "mmh_st_shard": (c_char_p, [P, I]),
    "mmh_st_shape": (I, [P, I, PL, I]),
    "mmh_st_offset": (L, [P, I, I]),
    "mmh_st_read": (I, [P, I, c_void_p, L]),
    "mmh_st_check": (I, [P, c_char_p, I, POINTER(c_char_p), PI, PL, PI]),
    "mmh_st_write": (I, [c_char_p, I, POINTER(c_char_p), POINTER(c_char_p), PI, PL, POINTER(c_void_p), PL, I, POINTER(c_char_p)]),
    "mmh_sched_create": (P, [P, I, I, I, I]),
    "mmh_sched_destroy": (None, [P]),
    "mmh_sched_add": (I, [P, L, PI, I, I, PI, I]),
    "mmh_sched_reject_reason": (c_char_p, [P, L]),
    "mmh_sched_has_work": (I, [P]),
    "mmh_sched_all_decoding": (I, [P]),
    "mmh_sched_schedule": (I, [P]),
    "mmh_sched_plan": (I, [P, PL, PI, PI, PI, I]),
    "mmh_sched_events": (I, [P, PL, PI, PI, I]),
    "mmh_sched_commit": (I, [P, I, PL, PI, PI, PI, PI]),
    "mmh_sched_accept_token": (I, [P, L, I]),
    "mmh_sched_set_sampling": (I, [P, L, c_float, I, c_float, L, c_float, c_float, c_float, I, c_float]),
    "mmh_sched_cancel": (I, [P, L]),
    "mmh_sched_request": (L, [P, L, I]),
    "mmh_sched_tokens": (I, [P, L, I, I, PI]),
    "mmh_sched_list": (I, [P, I, PL, I]),
    "mmh_sched_metric": (L, [P, I]),
}


def load() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is None:
            from ..kernels.build import host_library_path
            lib = ctypes.CDLL(host_library_path())
            for name, (res, args) in _PROTOTYPES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
        return _lib


def last_error() -> str:
    msg = load().mmh_last_error()
    return msg.decode() if msg else ""


def int_array(values):
    arr = (c_int * len(values))(*values)
    return arr


def long_array(values):
    arr = (c_longlong * len(values))(*values)
    return arr
