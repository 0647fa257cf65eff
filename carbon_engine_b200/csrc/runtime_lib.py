"""Loads libcarbon_runtime.so (built on first use) and declares its C interface."""
from __future__ import annotations

import ctypes
import threading

from . import build

_lib = None
_lock = threading.Lock()

_i, _i64, _p = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p
_pi = ctypes.POINTER(ctypes.c_int)
_pi32 = ctypes.POINTER(ctypes.c_int32)
_pi64 = ctypes.POINTER(ctypes.c_int64)

_SIGNATURES = {
    "cm_create": (_p, [_i, _pi, _pi, _pi, _i, _i]),
    "cm_destroy": (None, [_p]),
    "cm_open": (_i, [_p, _i64]),
    "cm_reserve": (_i, [_p, _i64, _i]),
    "cm_commit": (_i, [_p, _i64, _i]),
    "cm_commit_many": (_i, [_p, _pi64, _pi32, _i]),
    "cm_close": (_i, [_p, _i64]),
    "cm_slot_of": (_i, [_p, _i64]),
    "cm_length_of": (_i, [_p, _i64]),
    "cm_reserved_of": (_i, [_p, _i64]),
    "cm_free_pages": (_i, [_p, _i]),
    "cm_held_pages": (_i, [_p, _i64, _i]),
    "cm_free_slots": (_i, [_p]),
    "cm_open_requests": (_i, [_p]),
    "cm_pages_for_lifetime": (_i, [_p, _i, _i, _i]),
    "cm_pages_to_reserve": (_i, [_p, _i64, _i, _i]),
    "cm_table": (_pi32, [_p, _i]),
    "cm_check": (_i, [_p]),
    "step_layout": (_i, [_p, _p]),
    "sched_create": (_p, [_p, _i, _i, _i, _i, _pi, _i]),
    "sched_destroy": (None, [_p]),
    "sched_submit": (_i, [_p, _i64, _pi32, _i, _i, _i, _pi32, _i]),
    "sched_plan": (_i, [_p, _pi64, _i, _pi32, _i, _pi]),
    "sched_plan_for": (_i, [_p, _pi64, _i, _pi64, _i, _pi32, _i, _pi]),
    "sched_remaining": (_i, [_p, _i64]),
    "sched_waiting": (_i, [_p]),
    "sched_running": (_i, [_p]),
    "sched_commit": (_i, [_p, _pi32, _i]),
    "sched_fail_step": (None, [_p]),
    "sched_abort": (_i, [_p, _i64]),
    "sched_pop_finished": (_i, [_p, _pi64, _pi, _i]),
    "sched_num_tokens": (_i, [_p, _i64]),
    "sched_prompt_len": (_i, [_p, _i64]),
    "sched_copy_tokens": (_i, [_p, _i64, _pi32, _i]),
    "sched_forget": (None, [_p, _i64]),
    "sched_idle": (_i, [_p]),
    "sched_stats": (None, [_p, _pi64]),
}


def runtime() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is None:
            lib = ctypes.CDLL(build.build_runtime())
            for name, (res, args) in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


class StepLayoutArgs(ctypes.Structure):
    """``carbon::StepLayoutArgs`` of csrc/runtime/step_layout.h, field for field."""
    _fields_ = [("n", _i), ("ids", _p), ("counts", _p), ("tokens", _p), ("want_counts", _p), ("wants", _p),
                ("max_step_tokens", _i),
                ("tok", _p), ("pos", _p), ("seq_of_token", _p), ("seq_slot", _p), ("q_start", _p), ("ctx_len", _p), ("rows", _p),
                ("synced", _p), ("upd_idx", _p), ("upd_val", _p), ("upd_stride", _i), ("n_upd", _p),
                ("out_ids", _p), ("out_slot", _p), ("out_ctx_before", _p), ("out_new_len", _p), ("out", _p), ("detail", _p)]
