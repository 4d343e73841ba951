"""The host runtime's C++ library (csrc/host_runtime.cpp): page pools, the cache manager and
the scheduler's decisions, reached through ctypes.  ``lib()`` compiles it on first use
(a C++ compiler is all it needs) and declares every entry point's types."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_int, c_int64, c_longlong, c_void_p

_LIB = None


class HostRuntimeError(RuntimeError):
    pass


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    from ..kernels import build
    try:
        path = build.ensure_host_built()
        L = ctypes.CDLL(path)
    except (build.BuildError, OSError) as e:
        raise HostRuntimeError(f"the host runtime library is not available: {e}") from None
    ip, lp = POINTER(c_int), POINTER(c_int64)
    sig = {
        "bw_host_last_error": (c_char_p, []),
        "bw_pool_create": (c_void_p, [c_int]), "bw_pool_destroy": (None, [c_void_p]),
        "bw_pool_available": (c_int, [c_void_p]), "bw_pool_allocate": (c_int, [c_void_p]),
        "bw_pool_fork": (c_int, [c_void_p, c_int]), "bw_pool_release": (c_int, [c_void_p, c_int]),
        "bw_pool_refcount": (c_int, [c_void_p, c_int]),
        "bw_cm_create": (c_void_p, [c_int, ip, ip, c_int, c_int]), "bw_cm_destroy": (None, [c_void_p]),
        "bw_cm_begin": (c_int, [c_void_p, c_int64]), "bw_cm_has": (c_int, [c_void_p, c_int64]),
        "bw_cm_ensure": (c_int, [c_void_p, c_int64, c_int]), "bw_cm_advance": (c_int, [c_void_p, c_int64, c_int]),
        "bw_cm_release": (c_int, [c_void_p, c_int64, c_int]), "bw_cm_fork": (c_int, [c_void_p, c_int64, c_int64]),
        "bw_cm_info": (c_int, [c_void_p, c_int64, ip]),
        "bw_cm_table": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_int]),
        "bw_cm_pages_needed": (c_int, [c_void_p, c_int64, c_int, ip]),
        "bw_rows_create": (c_void_p, [c_int, c_int]), "bw_rows_destroy": (None, [c_void_p]),
        "bw_cm_prepare": (c_int, [c_void_p, c_void_p, c_int, lp, ip, c_void_p, ip, ip, ip, ip]),
        "bw_cm_available": (c_int, [c_void_p, c_int]), "bw_cm_refcount": (c_int, [c_void_p, c_int, c_int]),
        "bw_cm_free_slots": (c_int, [c_void_p]), "bw_cm_all_free": (c_int, [c_void_p]), "bw_cm_live": (c_int, [c_void_p]),
        "bw_cm_max_blocks": (c_int, [c_void_p, c_int]), "bw_cm_check": (c_int, [c_void_p]),
        "bw_sched_create": (c_void_p, [c_void_p, c_int, c_int]), "bw_sched_destroy": (None, [c_void_p]),
        "bw_sched_add": (c_int, [c_void_p, c_int64, c_longlong, c_int, c_int]),
        "bw_sched_update_many": (c_int, [c_void_p, c_int, lp, ip, ip]),
        "bw_sched_update": (c_int, [c_void_p, c_int64, c_int, c_int]),
        "bw_sched_finish": (c_int, [c_void_p, c_int64]), "bw_sched_preempt": (c_int, [c_void_p, c_int64]),
        "bw_sched_plan": (c_int, [c_void_p]),
        "bw_sched_plan_entries": (c_int, [c_void_p, lp, ip, c_int]),
        "bw_sched_preempted": (c_int, [c_void_p, lp, ip, c_int]),
        "bw_sched_running": (c_int, [c_void_p, lp, c_int]), "bw_sched_waiting": (c_int, [c_void_p, lp, c_int]),
        "bw_sched_state": (c_int, [c_void_p, c_int64, ip, ip]),
        "bw_sched_stat": (c_longlong, [c_void_p, c_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _LIB = L
    return L


def last_error() -> str:
    return lib().bw_host_last_error().decode("utf-8", "replace")
