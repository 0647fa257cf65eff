"""Python face of the native scheduler (csrc/runtime/scheduler.cpp): admission, portions of
prompts under a token budget, decoding, finishing and freeing.  See that file for the policy."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Sequence, Tuple

import numpy as np

from ..cache.manager import CacheManager
from ..csrc.runtime_lib import runtime

FINISH_REASONS = {1: "stop", 2: "length", 3: "abort", 4: "error"}

_SUBMIT_ERRORS = {
    -1: "the prompt is empty",
    -2: "the prompt leaves no room for a new token within max_seq_len",
    -3: "a token id is outside the vocabulary",
    -4: "request does not fit in the KV cache",
    -5: "the request id is already in use",
}


class SubmitError(ValueError):
    pass


@dataclass
class PlanEntry:
    request_id: int
    slot: int
    start: int
    count: int
    sample: bool
    tokens: List[int]


class Scheduler:
    def __init__(self, cache: CacheManager, max_running: int, max_step_tokens: int, max_seq_len: int,
                 vocab_size: int, eos_token_ids: Sequence[int] = ()):
        self._lib = runtime()
        self.cache = cache
        eos = (ctypes.c_int * max(len(eos_token_ids), 1))(*eos_token_ids)
        self._h = self._lib.sched_create(cache.handle, max_running, max_step_tokens, max_seq_len, vocab_size,
                                         eos, len(eos_token_ids))
        if not self._h:
            raise ValueError("bad scheduler parameters")
        self.max_running = min(max_running, cache.max_requests)
        self.max_step_tokens = max(max_step_tokens, self.max_running)
        self._entries = np.zeros(5 * (self.max_running + 1), dtype=np.int64)
        self._tokens = np.zeros(self.max_step_tokens + 1, dtype=np.int32)
        self._fin = None                     # buffers of pop_finished, made at its first call

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.sched_destroy(h)

    def submit(self, request_id: int, prompt: Sequence[int], max_tokens: int, ignore_eos: bool = False,
               stop_token_ids: Sequence[int] = ()) -> None:
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        s = np.ascontiguousarray(stop_token_ids, dtype=np.int32)
        code = self._lib.sched_submit(self._h, request_id, p.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), len(p),
                                      int(max_tokens), 1 if ignore_eos else 0,
                                      s.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), len(s))
        if code != 0:
            raise SubmitError(_SUBMIT_ERRORS.get(code, f"submit failed ({code})"))

    def plan(self) -> List[PlanEntry]:
        n_tok = ctypes.c_int(0)
        n = self._lib.sched_plan(self._h, self._entries.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)),
                                 len(self._entries) // 5, self._tokens.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
                                 len(self._tokens), ctypes.byref(n_tok))
        return self._read_plan(n, n_tok.value)

    def plan_for(self, request_ids: Sequence[int]) -> List[PlanEntry]:
        """The step that is already on the device for ``request_ids`` (one token each, fed there from the last
        step's picks): its entries for those of them that still run.  Nothing is admitted."""
        ids = np.ascontiguousarray(request_ids, dtype=np.int64)
        n_tok = ctypes.c_int(0)
        n = self._lib.sched_plan_for(self._h, ids.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)), len(ids),
                                     self._entries.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)), len(self._entries) // 5,
                                     self._tokens.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), len(self._tokens),
                                     ctypes.byref(n_tok))
        return self._read_plan(n, n_tok.value)

    def _read_plan(self, n: int, n_tok: int) -> List[PlanEntry]:
        if n < 0:
            raise RuntimeError("the scheduler's plan does not fit its buffers")
        ent = self._entries[:5 * n].tolist()             # (one conversion each: this runs between two steps)
        toks = self._tokens[:n_tok].tolist()
        out, off = [], 0
        for i in range(n):
            rid, slot, start, count, sample = ent[5 * i:5 * i + 5]
            out.append(PlanEntry(rid, slot, start, count, bool(sample), toks[off:off + count]))
            off += count
        return out

    def remaining(self, request_id: int) -> int:
        """Tokens the request may still generate (-1: unknown or ended)."""
        return self._lib.sched_remaining(self._h, request_id)

    def waiting(self) -> int:
        return self._lib.sched_waiting(self._h)

    def running(self) -> int:
        """Requests that hold a slot (they decode, or their prompts are under way)."""
        return self._lib.sched_running(self._h)

    def commit(self, sampled: Sequence[int]) -> None:
        s = np.ascontiguousarray(sampled, dtype=np.int32)
        if self._lib.sched_commit(self._h, s.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), len(s)) != 0:
            raise RuntimeError("commit: the number of sampled tokens does not match the plan")

    def fail_step(self) -> None:
        self._lib.sched_fail_step(self._h)

    def abort(self, request_id: int) -> bool:
        return self._lib.sched_abort(self._h, request_id) == 0

    def pop_finished(self) -> List[Tuple[int, str]]:
        if self._fin is None:
            ids, reasons = np.zeros(4096, dtype=np.int64), np.zeros(4096, dtype=np.int32)
            self._fin = (ids, reasons, ids.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)),
                         reasons.ctypes.data_as(ctypes.POINTER(ctypes.c_int)))
        ids, reasons, p_ids, p_reasons = self._fin
        n = self._lib.sched_pop_finished(self._h, p_ids, p_reasons, len(ids))
        return [(int(ids[i]), FINISH_REASONS.get(int(reasons[i]), "error")) for i in range(n)]

    def tokens_of(self, request_id: int) -> List[int]:
        n = self._lib.sched_num_tokens(self._h, request_id)
        if n < 0:
            raise KeyError(request_id)
        buf = np.zeros(max(n, 1), dtype=np.int32)
        self._lib.sched_copy_tokens(self._h, request_id, buf.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), n)
        return buf[:n].tolist()

    def num_tokens(self, request_id: int) -> int:
        """Prompt plus generated tokens of a request so far."""
        n = self._lib.sched_num_tokens(self._h, request_id)
        if n < 0:
            raise KeyError(request_id)
        return n

    def prompt_len_of(self, request_id: int) -> int:
        return self._lib.sched_prompt_len(self._h, request_id)

    def forget(self, request_id: int) -> None:
        self._lib.sched_forget(self._h, request_id)

    def idle(self) -> bool:
        return bool(self._lib.sched_idle(self._h))

    def stats(self) -> dict:
        buf = np.zeros(7, dtype=np.int64)
        self._lib.sched_stats(self._h, buf.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)))
        keys = ("steps", "prefill_tokens", "decode_tokens", "finished", "failed", "running", "waiting")
        return {k: int(v) for k, v in zip(keys, buf)}
