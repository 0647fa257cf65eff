"""Turns logits rows into tokens on the device.

All-greedy batches without penalties go to the argmax kernel; anything else goes through the
penalty kernel (if any row has penalties) and the sampling kernel, which handles greedy rows too.
Log-probabilities, when asked for, are taken from the model's distribution before penalties and
filters, as the reference does (src/sampling.rs:22-25, 66-93).
"""
from __future__ import annotations

import math
import os
from collections import Counter
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from .params import SamplingParams

_M64 = (1 << 64) - 1


def mix64(x: int) -> int:
    """splitmix64 finaliser (src/kernels/sampling.cu:30-36)."""
    x = (x + 0x9E3779B97F4A7C15) & _M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M64
    return x ^ (x >> 31)


def step_seed(seed: int, step: int) -> int:
    """The seed of a request's ``step``-th draw."""
    return mix64((seed & _M64) ^ mix64(step))


def fresh_seed() -> int:
    return int.from_bytes(os.urandom(8), "little")


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device
        # pinned staging for the per-row parameters, a few in turn: the copy never blocks the host, and a
        # buffer is rewritten only after the copy that read it has passed (two steps may be on the device)
        self._rows_host: List[Optional[torch.Tensor]] = [None] * 4
        self._rows_free: List[Optional["torch.cuda.Event"]] = [None] * 4
        self._rows_turn = 0
        self._rows_dev = None

    def _upload_rows(self, blob: bytes) -> torch.Tensor:
        n = len(blob)
        if self._rows_dev is None or self._rows_dev.numel() < n:
            self._rows_dev = torch.empty(max(4096, 2 * n), dtype=torch.uint8, device=self.device)
        k = self._rows_turn = (self._rows_turn + 1) % len(self._rows_host)
        if self._rows_host[k] is None or self._rows_host[k].numel() < n:
            self._rows_host[k] = torch.empty(max(4096, 2 * n), dtype=torch.uint8, pin_memory=self.device.type == "cuda")
            self._rows_free[k] = None
        if self._rows_free[k] is not None:
            self._rows_free[k].synchronize()
        self._rows_host[k][:n] = torch.frombuffer(bytearray(blob), dtype=torch.uint8)
        self._rows_dev[:n].copy_(self._rows_host[k][:n], non_blocking=True)
        if self.device.type == "cuda":
            if self._rows_free[k] is None:
                self._rows_free[k] = torch.cuda.Event()
            self._rows_free[k].record()
        return self._rows_dev[:n]

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], seeds: Sequence[int],
               steps: Sequence[int], prompts: Optional[Sequence[Sequence[int]]] = None,
               outputs: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """One token per row of ``logits`` (float32 [rows, vocab]); returns int32 [rows] on the device.

        ``seeds[i]`` is row i's request seed and ``steps[i]`` how many tokens it has drawn so far;
        ``prompts``/``outputs`` are needed only by rows with penalties.  ``logits`` is modified in
        place when penalties apply.
        """
        R = logits.shape[0]
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        if R == 0:
            return out
        if any(p.has_penalties() for p in params):
            self._penalties(logits, params, prompts, outputs)
        if all(p.is_greedy() for p in params):
            ops.argmax(logits, out)
            return out
        rows = [(p.temperature, p.top_p, p.min_p, p.top_k if p.top_k > 0 else 0, step_seed(s, st))
                for p, s, st in zip(params, seeds, steps)]
        ops.sample(logits, self._upload_rows(ops.pack_sample_rows(rows)), out)
        return out

    def _penalties(self, logits, params, prompts, outputs) -> None:
        entries: List[Tuple[int, int, int, int]] = []
        row_params = np.zeros((logits.shape[0], 3), dtype=np.float32)
        for r, p in enumerate(params):
            row_params[r] = (p.repetition_penalty, p.presence_penalty, p.frequency_penalty)
            if not p.has_penalties():
                continue
            counts = Counter(outputs[r]) if outputs is not None else Counter()
            seen = set(prompts[r]) if prompts is not None else set()
            seen.update(counts)
            for tok in seen:
                entries.append((r, int(tok), 1, int(counts.get(tok, 0))))
        if not entries:
            return
        ent = torch.tensor(entries, dtype=torch.int32).to(self.device)
        ops.apply_penalties(logits, ent, torch.from_numpy(row_params).to(self.device))


def top_logprobs(row: np.ndarray, token: int, n: int) -> Dict:
    """Log-probability of ``token`` and of the ``n`` most likely tokens of a float32 logits row
    (src/sampling.rs:66-93; lower index first on ties)."""
    r = row.astype(np.float64)
    m = r.max()
    lse = m + math.log(np.exp(r - m).sum())
    order = np.lexsort((np.arange(r.shape[0]), -r))[:n]
    return {"token": int(token), "logprob": float(r[token] - lse),
            "top": [(int(t), float(r[t] - lse)) for t in order]}
