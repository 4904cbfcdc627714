"""The host runtime library (``csrc/host/*.cpp``) loaded through ctypes: page pools, the cache
manager's books and the scheduler's decisions in C++.  Built with the system's C++ compiler at
first use."""
from __future__ import annotations

import ctypes
from typing import Optional

_dll: Optional[ctypes.CDLL] = None


def library() -> ctypes.CDLL:
    global _dll
    if _dll is None:
        from ..kernels.build import build_host
        dll = ctypes.CDLL(build_host())
        P, I = ctypes.c_void_p, ctypes.c_int
        IP = ctypes.POINTER(ctypes.c_int)
        L, LP = ctypes.c_int64, ctypes.POINTER(ctypes.c_int64)
        signatures = {
            "mrun_pool_create": (P, [I]), "mrun_pool_destroy": (None, [P]), "mrun_pool_free_count": (I, [P]),
            "mrun_pool_alloc": (I, [P, I, IP]), "mrun_pool_free": (I, [P, IP, I, IP]),
            "mrun_pool_is_held": (I, [P, I]), "mrun_pool_check": (ctypes.c_char_p, [P]),
            "mrun_cache_create": (P, [I, IP, I, I, I, I]), "mrun_cache_destroy": (None, [P]),
            "mrun_cache_error": (ctypes.c_char_p, [P]), "mrun_cache_table": (IP, [P, I]),
            "mrun_cache_free_pages": (I, [P, I]), "mrun_cache_free_slots": (I, [P]),
            "mrun_cache_length": (I, [P, I]), "mrun_cache_pending": (I, [P, I]), "mrun_cache_blocks": (I, [P, I, I]),
            "mrun_cache_is_held": (I, [P, I, I]), "mrun_cache_shortage": (None, [P, IP, IP, IP, IP]),
            "mrun_cache_admit": (I, [P]), "mrun_cache_release": (I, [P, I]), "mrun_cache_trim": (I, [P, I, I]),
            "mrun_cache_plan": (I, [P, I, IP, IP]), "mrun_cache_commit": (I, [P, I]),
            "mrun_cache_rollback": (I, [P, I]), "mrun_cache_drain": (I, [P, I, IP, IP, I]),
            "mrun_cache_pending_updates": (I, [P, I]), "mrun_cache_check": (ctypes.c_char_p, [P]),
            "mrun_cache_layout_step": (I, [P, I, IP, IP, IP, IP, IP, IP, IP, ctypes.POINTER(IP)]),
            "mrun_sched_chunk_len": (I, [L, I]), "mrun_sched_looping": (I, [IP, L]),
            "mrun_sched_loop_check_every": (I, []),
            "mrun_sched_submit_check": (I, [L, L, L, L, L, LP]),
            "mrun_sched_can_admit": (I, [I, I, I, I, L, L, I, L, L, L, I, LP, LP]),
            "mrun_sched_plan": (I, [I, LP, LP, IP, LP, LP, IP, LP, I, IP, IP, IP, IP]),
            "mrun_sched_end_reason": (I, [I, I, L, L, IP, L]),
            "mrun_sched_preemption_victim": (I, [I, IP, LP]),
            "mrun_sched_next_turn": (I, [I, IP, IP, IP, I, I]),
            "mrun_sched_stop_match": (I, [IP, I, IP, IP, I]), "mrun_sched_stop_held": (I, [IP, I, IP, IP, I]),
        }
        for name, (restype, argtypes) in signatures.items():
            fn = getattr(dll, name)
            fn.restype, fn.argtypes = restype, argtypes
        _dll = dll
    return _dll


def int_array(values) -> ctypes.Array:
    values = list(values)
    return (ctypes.c_int * max(1, len(values)))(*values)


def long_array(values) -> ctypes.Array:
    values = list(values)
    return (ctypes.c_int64 * max(1, len(values)))(*values)
