"""What one step is given and what the parts see of it.

A step is a list of :class:`StepEntry`: for each request its next tokens (a portion of a prompt, or
one decoded token) and the places among them whose logits are wanted.  The reference describes a
step with ``BatchMeta``/``SeqMeta`` (src/batch.rs:10-83): positions, per-token cache locations and
per-sequence slot lists, rebuilt and uploaded every step.  Here the per-token and per-sequence
integers travel in ONE pinned buffer with fixed offsets (so that kernels captured in a CUDA graph
keep reading the same addresses), and the block tables stay resident on the device.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch


@dataclass
class StepEntry:
    request_id: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)     # places among ``tokens`` whose logits are asked for


class StepBuffers:
    """The pinned host buffer and its device twin, with fixed sections."""

    def __init__(self, max_tokens: int, max_seqs: int, num_groups: int, device: torch.device,
                 extra_sections: Sequence[Tuple[str, int]] = ()):
        """``extra_sections``: (name, int32 count) of what the model's mixers lay out per step for their
        own kernels (see ``Mixer.step_sections``)."""
        self.max_tokens, self.max_seqs = int(max_tokens), int(max_seqs)
        T, B = self.max_tokens, self.max_seqs
        upd = T + 2 * B + 8                      # the most table entries one step can add per group
        sizes = [("tokens", T), ("positions", T), ("seq_of_token", T), ("seq_slot", B), ("q_start", B + 1),
                 ("ctx_len", B), ("rows", T)]
        sizes += [(str(n), int(c)) for n, c in extra_sections]
        for g in range(num_groups):
            sizes += [(f"upd_idx{g}", upd), (f"upd_val{g}", upd)]
        self.offsets = {}
        off = 0
        for name, n in sizes:
            self.offsets[name] = (off, n)
            off += (n + 3) // 4 * 4              # sections start on 16-byte boundaries
        self.total = off
        self.host = torch.zeros(self.total, dtype=torch.int32).pin_memory() if torch.cuda.is_available() \
            else torch.zeros(self.total, dtype=torch.int32)
        self.host_np = self.host.numpy()
        self.dev = torch.zeros(self.total, dtype=torch.int32, device=device)
        # The device status word: kernels flag a bad index or a wait that gave up here.  On a GPU it is the
        # word the tensor-core products report to as well, so one read covers every kernel of a step.
        if torch.device(device).type == "cuda":
            from .. import ops_tensor
            self.status = ops_tensor.gemm_workspace(torch.device(device)).status
        else:
            self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._uploaded = None

    def host_section(self, name: str) -> np.ndarray:
        off, n = self.offsets[name]
        return self.host_np[off:off + n]

    def dev_section(self, name: str, n: Optional[int] = None) -> torch.Tensor:
        off, cap = self.offsets[name]
        return self.dev[off:off + (cap if n is None else n)]

    def wait_host_free(self) -> None:
        """Block until the last upload has left the pinned buffer, so that it may be rewritten."""
        if self._uploaded is not None:
            self._uploaded.synchronize()

    def upload(self) -> int:
        self.dev.copy_(self.host, non_blocking=True)
        if self.dev.is_cuda:
            if self._uploaded is None:
                self._uploaded = torch.cuda.Event()
            self._uploaded.record()
        return self.total * 4


class StepContext:
    """What parts read during a step.  Integer tensors are int32 on the device; fields starting
    with ``h_`` are host copies for parts that need to loop over sequences (state mixers)."""

    def __init__(self, bufs: StepBuffers, T: int, B: int, dtype: torch.dtype, device: torch.device,
                 block_tables: List[torch.Tensor]):
        self.T, self.B, self.dtype, self.device = T, B, dtype, device
        self.tokens = bufs.dev_section("tokens", T)
        self.positions = bufs.dev_section("positions", T)
        self.seq_of_token = bufs.dev_section("seq_of_token", T)
        self.seq_slot = bufs.dev_section("seq_slot", B)
        self.q_start = bufs.dev_section("q_start", B + 1)
        self.ctx_len = bufs.dev_section("ctx_len", B)
        self.status = bufs.status
        self.block_tables = block_tables
        self.h_slots: List[int] = []
        self.h_q_start: List[int] = []       # B + 1 entries
        self.h_ctx_before: List[int] = []    # tokens of each sequence already in the cache
        self.bufs = bufs
        #: what each kind of mixer laid out for this step (``Mixer.plan_step``), by the mixer's ``plan_key``
        self.plans: Dict[str, Any] = {}
        self._scratch = {}
        self.n_decode = 0                    # the first n_decode sequences bring exactly one token
        self.max_position = 0
        self.max_ctx = 0
        self.fast_attention = True

    def scratch(self, name: str, numel: int) -> torch.Tensor:
        """float32 scratch memory shared by the layers of this step."""
        t = self._scratch.get(name)
        if t is None or t.numel() < numel:
            t = torch.empty(max(int(numel), 1), dtype=torch.float32, device=self.device)
            self._scratch[name] = t
        return t

    def buffer(self, shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)
