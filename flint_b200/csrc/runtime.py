"""The face of the native host runtime (``host/runtime.cpp``): the shared library, loaded once,
with its functions' types declared, and the mapping of its failure codes to exceptions.

The library is plain C++ (no device code); it is compiled with the host compiler the first
time it is needed, like the CUDA modules.  The reference's engine, pool and row metadata are
native too (crates/thuban_generate/src/engine.rs, crates/thuban_model/src/pool.rs, rows.rs).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_longlong, c_void_p

from ..errors import CacheError, ModelError
from . import build

_INT_P = POINTER(c_int)
_lib = None

_SIGNATURES = {
    "flint_rt_last_error": (c_char_p, []),
    "flint_rt_group_create": (c_void_p, [c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "flint_rt_group_destroy": (None, [c_void_p]),
    "flint_rt_group_take": (c_int, [c_void_p]),
    "flint_rt_group_give_back": (c_int, [c_void_p, c_int]),
    "flint_rt_group_free_pages": (c_int, [c_void_p]),
    "flint_rt_group_total_allocations": (c_longlong, [c_void_p]),
    "flint_rt_group_served": (None, [c_void_p, _INT_P]),
    "flint_rt_group_pages_needed": (c_int, [c_void_p, c_int, c_int, c_int]),
    "flint_rt_group_ensure": (c_int, [c_void_p, c_int, c_int, c_int]),
    "flint_rt_group_release_behind": (c_int, [c_void_p, c_int, c_int]),
    "flint_rt_group_release_all": (c_int, [c_void_p, c_int]),
    "flint_rt_group_truncate": (c_int, [c_void_p, c_int, c_int]),
    "flint_rt_group_check": (c_int, [c_void_p, c_int]),
    "flint_rt_group_table": (c_int, [c_void_p, c_int, _INT_P, c_int]),
    "flint_rt_group_first_live": (c_int, [c_void_p, c_int]),
    "flint_rt_group_take_dirty": (None, [c_void_p, _INT_P, _INT_P]),
    "flint_rt_cache_create": (c_void_p, [c_int, c_int, c_int]),
    "flint_rt_cache_destroy": (None, [c_void_p]),
    "flint_rt_cache_add_group": (None, [c_void_p, c_void_p]),
    "flint_rt_cache_admit": (c_int, [c_void_p]),
    "flint_rt_cache_release": (c_int, [c_void_p, c_int]),
    "flint_rt_cache_free_slots": (c_int, [c_void_p]),
    "flint_rt_cache_is_live": (c_int, [c_void_p, c_int]),
    "flint_rt_cache_pages_needed": (c_int, [c_void_p, c_int, c_int, c_int]),
    "flint_rt_cache_free_pages": (c_int, [c_void_p]),
    "flint_rt_cache_can_run": (c_int, [c_void_p, c_int, c_int, c_int]),
    "flint_rt_cache_ensure": (c_int, [c_void_p, c_int, c_int, c_int]),
    "flint_rt_cache_advance": (c_int, [c_void_p, c_int, c_int]),
    "flint_rt_cache_check": (c_int, [c_void_p]),
    "flint_rt_sched_create": (c_void_p, [c_void_p, c_int, c_int, c_int, c_int, c_int]),
    "flint_rt_sched_destroy": (None, [c_void_p]),
    "flint_rt_sched_add": (c_int, [c_void_p, c_int, c_int, c_int, _INT_P, c_int]),
    "flint_rt_sched_set_stop": (None, [c_void_p, c_int, _INT_P, c_int]),
    "flint_rt_sched_plan": (c_int, [c_void_p, _INT_P, c_int]),
    "flint_rt_sched_commit": (c_int, [c_void_p, _INT_P, c_int, _INT_P, c_int, _INT_P, c_int]),
    "flint_rt_sched_abort": (c_int, [c_void_p, c_int]),
    "flint_rt_sched_forget": (c_int, [c_void_p, c_int]),
    "flint_rt_sched_records": (c_int, [c_void_p]),
    "flint_rt_sched_resolve": (c_int, [c_void_p, c_int, c_int]),
    "flint_rt_sched_steady": (c_int, [c_void_p]),
    "flint_rt_sched_has_work": (c_int, [c_void_p]),
    "flint_rt_sched_request": (None, [c_void_p, c_int, _INT_P]),
    "flint_rt_sched_request_error": (c_char_p, [c_void_p, c_int]),
    "flint_rt_sched_list": (c_int, [c_void_p, c_int, _INT_P, c_int]),
    "flint_rt_sched_take_touched": (c_int, [c_void_p, _INT_P, c_int]),
    "flint_rt_sched_counters": (None, [c_void_p, _INT_P, _INT_P]),
    "flint_rt_pack_step": (c_int, [c_int, _INT_P, _INT_P, _INT_P, _INT_P, _INT_P, _INT_P, _INT_P, c_int, c_int, c_int,
                                   c_int, c_int, c_int, c_int, c_void_p, _INT_P, _INT_P]),
}

E_CACHE, E_MODEL, E_CHECK = -1, -2, -3


def lib():
    """The runtime library (compiled on first use)."""
    global _lib
    if _lib is None:
        loaded = build.load_module("runtime")
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(loaded, name)
            fn.restype, fn.argtypes = res, args
        _lib = loaded
    return _lib


def ints(values):
    """A C array of ints from a Python sequence."""
    return (c_int * len(values))(*values)


def checked(rc: int) -> int:
    """Pass a count through; turn a failure code into the exception it stands for."""
    if rc >= 0:
        return rc
    msg = (lib().flint_rt_last_error() or b"runtime error").decode()
    if rc == E_CACHE:
        raise CacheError(msg)
    if rc == E_MODEL:
        raise ModelError(msg)
    raise AssertionError(msg)
