"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

It runs only the tokens it is given, as one batch, against the cache that earlier steps left:
portions of prompts beside single decoded tokens, cut anywhere.  The reference's counterpart is
``Engine::forward(meta, tokens, sample_rows) -> f32 [rows, vocab]`` (src/engine.rs:407-446), fed
by either a prefill batch or a decode batch; here one call takes any mixture.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache.storage import CacheStorage
from .batch import StepBuffers, StepContext, StepEntry


class StepError(RuntimeError):
    pass


_STATUS = {
    1: "a token id outside the vocabulary reached the embedding",
    2: "a token was to be written to a page its request does not hold",
    3: "a position beyond the rotary table (raise max_seq_len)",
    4: "attention read a page its request does not hold",
    5: "a bounded wait inside a tensor-core product gave up (the step's results are not valid)",
    7: "a bounded wait inside the decode attention kernel gave up (the step's results are not valid)",
}


def _status_text(code: int) -> str:
    if 50 <= code < 60:
        return f"a bounded wait inside a tensor-core product gave up (site {code}; the step's results are not valid)"
    if code >= 10:
        return "a bounded wait inside the flash attention kernel gave up (the step's results are not valid)"
    return _STATUS.get(code, "unknown")


class _Commits:
    """The requests of a laid-out step with their new lengths, to be committed once the step is on its way;
    iterates as (request, new length) pairs."""

    def __init__(self, ids: np.ndarray, new_lens: np.ndarray):
        self.ids, self.new_lens = ids, new_lens

    def __iter__(self):
        return iter(zip(self.ids.tolist(), self.new_lens.tolist()))

    def __len__(self):
        return len(self.ids)


class _NativeLayout:
    """The arrays the host runtime's ``step_layout`` reads and fills, made once: the flattened entries, the
    block-table entries a step adds, the per-sequence results; and its argument block, whose pointers into the
    pinned buffer's sections never change."""

    def __init__(self, bufs: StepBuffers, storage: CacheStorage, max_step_tokens: int):
        from ..csrc.runtime_lib import StepLayoutArgs, runtime
        self.lib = runtime()
        n, groups = storage.max_requests, max(len(storage.groups), 1)
        self.ids = np.zeros(n, dtype=np.int64)
        self.counts = np.zeros(n, dtype=np.int32)
        self.want_counts = np.zeros(n, dtype=np.int32)
        self.tokens = np.zeros(max_step_tokens, dtype=np.int32)
        self.wants = np.zeros(max_step_tokens, dtype=np.int32)
        stride = n * storage.max_pages_per_request          # every entry of every row: a step can never add more
        self.upd_idx = np.zeros((groups, stride), dtype=np.int32)
        self.upd_val = np.zeros((groups, stride), dtype=np.int32)
        self.n_upd = np.zeros(groups, dtype=np.int32)
        self.out_ids = np.zeros(n, dtype=np.int64)
        self.out_slot = np.zeros(n, dtype=np.int32)
        self.out_ctx_before = np.zeros(n, dtype=np.int32)
        self.out_new_len = np.zeros(n, dtype=np.int32)
        self.out = np.zeros(8, dtype=np.int32)
        self.detail = np.zeros(3, dtype=np.int64)
        a = self.args = StepLayoutArgs()
        ptr = lambda arr: arr.ctypes.data
        a.ids, a.counts, a.tokens, a.want_counts, a.wants = map(ptr, (self.ids, self.counts, self.tokens, self.want_counts, self.wants))
        a.max_step_tokens = int(max_step_tokens)
        a.tok, a.pos, a.seq_of_token = (ptr(bufs.host_section(k)) for k in ("tokens", "positions", "seq_of_token"))
        a.seq_slot, a.q_start, a.ctx_len, a.rows = (ptr(bufs.host_section(k)) for k in ("seq_slot", "q_start", "ctx_len", "rows"))
        a.synced = ptr(storage._synced)
        a.upd_idx, a.upd_val, a.upd_stride, a.n_upd = ptr(self.upd_idx), ptr(self.upd_val), stride, ptr(self.n_upd)
        a.out_ids, a.out_slot, a.out_ctx_before, a.out_new_len = map(ptr, (self.out_ids, self.out_slot, self.out_ctx_before, self.out_new_len))
        a.out, a.detail = ptr(self.out), ptr(self.detail)


class ModelRunner:
    #: steps of more tokens than this run their kernels strictly one after another (see ``step``)
    DEPENDENT_LAUNCH_MAX_TOKENS = 128

    def __init__(self, model, storage: CacheStorage, max_step_tokens: int):
        self.model, self.storage = model, storage
        self.device, self.dtype = model.device, model.dtype
        self.max_step_tokens = int(max_step_tokens)
        # one planner per kind of mixer that lays out tables of its own for a step
        self._planners = {}
        for block in model.blocks:
            key = getattr(block.mixer, "plan_key", None)
            if key is not None and key not in self._planners:
                self._planners[key] = block.mixer
        sections = [s for m in self._planners.values() for s in m.step_sections(self.max_step_tokens, storage.max_requests)]
        self.bufs = StepBuffers(self.max_step_tokens, storage.max_requests, len(storage.groups), self.device, sections)
        self.fast_attention = True
        self.graphs_enabled = False
        self._graphs = {}
        self._ahead = None                   # a next step laid out on the host in advance (prepare_decode_ahead)
        self._graph_pool = None
        self.h2d_bytes_last = 0
        self._back = [None] * 4              # pinned int32 buffers of read_back with their events, used in turn
        self._back_turn = 0
        self._copy_stream = None             # the stream the read-back copies run on
        self._status_read = None             # the status word read_back brought along, until check_status takes it
        self.kernel_launches = 0
        self._native = _NativeLayout(self.bufs, storage, self.max_step_tokens)

    # -- requests -------------------------------------------------------------------------------
    def open_request(self, request_id: int) -> int:
        self._discard_ahead()
        slot = self.storage.manager.open(request_id)
        self.storage.slot_opened(slot)
        self.storage.zero_state(slot)
        return slot

    def adopt_request(self, request_id: int) -> int:
        """A request the scheduler opened in the cache manager: prepare its slot on the device."""
        self._discard_ahead()
        slot = self.storage.manager.slot_of(request_id)
        self.storage.slot_opened(slot)
        self.storage.zero_state(slot)
        return slot

    def close_request(self, request_id: int) -> None:
        self._discard_ahead()
        self.storage.manager.close(request_id)

    # -- the step -------------------------------------------------------------------------------
    def prepare(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None):
        """Reserve pages, lay the step out in the pinned buffer and upload it.  Returns the context,
        the device tensor of wanted rows and the requests with their new lengths to commit.

        ``device_tokens`` (int32, one for every entry, each entry bringing ONE token): the token ids are not
        known on the host yet; they are copied on the device from this tensor, which an earlier step's
        sampling fills, so that the step can be launched before that one has been read back."""
        if device_tokens is not None:
            if any(len(e.tokens) != 1 for e in entries) or device_tokens.numel() != len(entries):
                raise StepError("token ids on the device: every entry brings exactly one token")
            self._discard_ahead()
            out = self._send(*self._layout_restoring(entries))
            self.bufs.dev_section("tokens", len(entries)).copy_(device_tokens.reshape(-1))
            return out
        ahead, self._ahead = self._ahead, None
        if ahead is not None:
            if self._ahead_matches(ahead, entries):
                ctx, n_rows, commits, n_upd = ahead["layout"]
                tokens = [e.tokens[0] for e in entries]
                self.bufs.host_section("tokens")[:len(tokens)] = np.asarray(tokens, dtype=np.int32)
                return self._send(ctx, n_rows, commits, n_upd)
            self.storage._synced[:] = ahead["synced"]        # its table updates were never sent
        return self._send(*self._layout_restoring(entries))

    def _layout_restoring(self, entries: Sequence[StepEntry]):
        synced = self.storage._synced.copy()
        try:
            return self._layout(entries)
        except Exception:
            # entries laid out before the faulty one took table updates that will never be sent
            self.storage._synced[:] = synced
            raise

    def prepare_decode_ahead(self, request_ids: Sequence[int]) -> None:
        """Lay out the NEXT step on the host while the current one runs, on the guess that these requests
        each bring one token and nothing else changes: pages reserved, positions, slots and table updates
        written to the pinned buffer; only the token ids are missing.  ``prepare`` uses the layout if its
        entries are exactly these requests with one token and one wanted place each, and throws it away
        otherwise (a request finished, one arrived, a prompt portion joined)."""
        self._discard_ahead()
        if not request_ids:
            return
        synced = self.storage._synced.copy()
        try:
            layout = self._layout([StepEntry(r, [0], [0]) for r in request_ids])
        except Exception:
            self.storage._synced[:] = synced                # the step itself will meet the same error, and report it
            return
        self._ahead = {"ids": tuple(request_ids), "layout": layout, "synced": synced}

    def _discard_ahead(self) -> None:
        ahead, self._ahead = self._ahead, None
        if ahead is not None:
            self.storage._synced[:] = ahead["synced"]

    @staticmethod
    def _ahead_matches(ahead, entries: Sequence[StepEntry]) -> bool:
        ids = ahead["ids"]
        return len(entries) == len(ids) and all(
            e.request_id == r and len(e.tokens) == 1 and len(e.want) == 1 and e.want[0] == 0 for e, r in zip(entries, ids))

    def _send(self, ctx, n_rows: int, commits, n_upd):
        b = self.bufs
        self.h2d_bytes_last = b.upload()
        prof = ops.profiling()
        if prof is not None:
            prof.mark()                  # the layout on the host and the upload are not the first kernel's time
        for g, n in enumerate(n_upd):
            if n:
                ops.scatter_i32(self.storage.device_tables[g], b.dev_section(f"upd_idx{g}", n),
                                b.dev_section(f"upd_val{g}", n))
        return ctx, b.dev_section("rows", n_rows), commits

    def _write_table_entries(self, group: int, idx: np.ndarray, val: np.ndarray) -> None:
        d_idx = torch.from_numpy(np.ascontiguousarray(idx, dtype=np.int32)).to(self.device)
        d_val = torch.from_numpy(np.ascontiguousarray(val, dtype=np.int32)).to(self.device)
        ops.scatter_i32(self.storage.device_tables[group], d_idx, d_val)

    def _layout(self, entries: Sequence[StepEntry]):
        """Checks, page reservations and the step's layout in the pinned host buffer (nothing is sent).  The
        work is done by the host runtime (csrc/runtime/step_layout.cpp); here the entries are flattened into
        its arrays, its errors become exceptions, and the mixers plan their own tables."""
        n = len(entries)
        if n == 0:
            raise StepError("a step needs at least one entry")
        if n > self.storage.max_requests:
            raise StepError(f"{n} entries, but only {self.storage.max_requests} requests may be live")
        L = self._native
        T = W = 0
        for i, e in enumerate(entries):
            c, w = len(e.tokens), len(e.want)
            if c == 0:
                raise StepError(f"request {e.request_id}: an entry needs at least one token")
            if T + c > self.max_step_tokens:
                raise StepError(f"{sum(len(x.tokens) for x in entries)} tokens in one step, but the engine was built for "
                                f"{self.max_step_tokens}")
            if W + w > self.max_step_tokens:
                raise StepError("more wanted places than tokens in the step (a place is named twice)")
            L.ids[i], L.counts[i], L.want_counts[i] = e.request_id, c, w
            L.tokens[T:T + c] = e.tokens
            if w:
                L.wants[W:W + w] = e.want
            T += c
            W += w
        b = self.bufs
        b.wait_host_free()
        L.args.n = n
        code = L.lib.step_layout(self.storage.manager.handle, ctypes.byref(L.args))
        if code != 0:
            self._raise_layout_error(code, L.detail.tolist())
        T, n_rows, n_decode, max_position, max_ctx = L.out[:5].tolist()
        ctx = StepContext(b, T, n, self.dtype, self.device, self.storage.device_tables)
        ctx.fast_attention = self.fast_attention
        ctx.h_slots = L.out_slot[:n].tolist()
        ctx.h_q_start = b.host_section("q_start")[:n + 1].tolist()
        ctx.h_ctx_before = L.out_ctx_before[:n].tolist()
        ctx.n_decode, ctx.max_position, ctx.max_ctx = n_decode, max_position, max_ctx
        commits = _Commits(L.out_ids[:n].copy(), L.out_new_len[:n].copy())
        for key, mixer in self._planners.items():
            ctx.plans[key] = mixer.plan_step(ctx)
        n_upd = []
        for g in range(len(self.storage.groups)):
            k = int(L.n_upd[g])
            if k:
                idx, val = L.upd_idx[g, :k], L.upd_val[g, :k]
                cap = len(b.host_section(f"upd_idx{g}"))
                if k > cap:
                    # more new table entries than a step's section holds (requests that arrive with long contexts
                    # already in the cache): the surplus goes to the device tables at once, by a copy of its own
                    self._write_table_entries(g, idx[cap:], val[cap:])
                    idx, val, k = idx[:cap], val[:cap], cap
                b.host_section(f"upd_idx{g}")[:k] = idx
                b.host_section(f"upd_val{g}")[:k] = val
            n_upd.append(k)
        return ctx, n_rows, commits, n_upd

    @staticmethod
    def _raise_layout_error(code: int, detail) -> None:
        from ..cache.manager import CacheError, OutOfPages
        if code == -101:
            raise StepError("a step needs at least one entry")
        if code == -102:
            raise StepError(f"{detail[0]} entries, but only {detail[1]} requests may be live")
        if code == -103:
            raise StepError(f"{detail[0]} tokens in one step, but the engine was built for {detail[1]}")
        if code == -104:
            raise StepError("more wanted places than tokens in the step (a place is named twice)")
        if code == -105:
            raise StepError(f"request {detail[0]}: an entry needs at least one token")
        if code == -106:
            raise StepError(f"request {detail[0]} appears twice in one step")
        if code == -107:
            raise StepError(f"request {detail[0]}: wanted place {detail[1]} is outside its {detail[2]} tokens")
        what = f"reserve({detail[0]}, {detail[1]})"
        if code == -4:
            raise OutOfPages(f"{what}: out of pages")
        from ..cache.manager import _MESSAGES
        raise CacheError(f"{what}: {_MESSAGES.get(code, code)}")

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run one step and return float32 logits [wanted, vocab] on the device, in the order of the
        entries and of their ``want`` lists.  With CUDA graphs on, the logits of a pure decode step
        live in a buffer that the next such step overwrites.  ``device_tokens``: see :meth:`prepare`."""
        ctx, rows, commits = self.prepare(entries, device_tokens)
        # Dependent launches (a kernel starts, and streams its first weights, while the kernel before it still
        # runs) are what makes the short kernels of small steps overlap.  Steps of more than 128 tokens may run the
        # persistent CTA-pair product, whose grid wants every pair of SMs: with its dependents already resident
        # and waiting beside it, such a step was seen, rarely (once in a few thousand layers at 4,096 tokens a
        # step), never to finish: the pair kernel did not complete although all of its blocks that ran had left,
        # and the next kernel's blocks waited for it for good.  Large steps gain little from the overlap, so
        # they run without it.
        ops.set_dependent_launches(ctx.T <= self.DEPENDENT_LAUNCH_MAX_TOKENS and os.environ.get("CE_PDL", "1") != "0")
        if self.graphs_enabled and ctx.n_decode == ctx.B and all(len(e.want) == 1 for e in entries):
            logits = self._replay_decode(ctx, rows)
        else:
            x = self.model.forward(ctx, self.storage)
            logits = self.model.logits(ctx, x, rows)
        self.storage.manager.commit_many(commits.ids, commits.new_lens)
        return logits

    # -- CUDA graphs for decode steps -----------------------------------------------------------
    def enable_graphs(self) -> bool:
        """Replay pure decode steps as CUDA graphs, one per (batch size, the mixers' graph keys), captured at
        first use (the reference does the same per batch size, src/model/graph.rs:50-120).  Only
        models whose mixers read the step from device buffers alone can be captured."""
        self.graphs_enabled = bool(getattr(self.model, "graph_safe", False))
        return self.graphs_enabled

    def _replay_decode(self, ctx: StepContext, rows: torch.Tensor) -> torch.Tensor:
        key = (ctx.B,) + tuple(getattr(ctx.plans[k], "graph_key", None) for k in self._planners)
        entry = self._graphs.get(key)
        if entry is None:
            # once eagerly, so that lazy initialisation (library handles, kernel attributes) is not captured
            x = self.model.forward(ctx, self.storage)
            self.model.logits(ctx, x, rows)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                x = self.model.forward(ctx, self.storage)
                logits = self.model.logits(ctx, x, rows)
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            entry = (graph, logits, ops.launch_count() - before)
            self._graphs[key] = entry
        graph, logits, launches = entry
        graph.replay()
        ops.add_launches(launches)
        return logits

    def read_back(self, values: torch.Tensor) -> List[int]:
        """A step's small int32 result (the sampled tokens) and the device status word in ONE wait: both are
        copied to pinned memory behind the step on its stream, then the stream is waited for once.  The
        status is kept for the next :meth:`check_status`, which then does not wait again."""
        return self.finish_read_back(self.begin_read_back(values))

    def begin_read_back(self, values: torch.Tensor):
        """Queue the copies of :meth:`read_back` and return a ticket.  They run on a stream of their own, behind
        what has been launched so far on the current one: the upload and the kernels of the NEXT step, launched
        after this call, neither wait for them nor delay them."""
        n = values.numel()
        k = self._back_turn = (self._back_turn + 1) % len(self._back)
        if self._back[k] is None or self._back[k][0].numel() < n + 1:
            self._back[k] = (torch.empty(max(n + 1, 257), dtype=torch.int32, pin_memory=True), torch.cuda.Event(),
                             torch.cuda.Event())
        buf, done, computed = self._back[k]
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        side = self._copy_stream
        computed.record()
        side.wait_event(computed)
        with torch.cuda.stream(side):
            buf[:n].copy_(values.reshape(-1), non_blocking=True)
            buf[n:n + 1].copy_(self.bufs.status.reshape(-1)[:1], non_blocking=True)
            done.record()
        values.record_stream(side)
        return k, n

    def finish_read_back(self, ticket) -> List[int]:
        k, n = ticket
        buf, done, _ = self._back[k]
        done.synchronize()
        self._status_read = int(buf[n])
        return buf[:n].tolist()

    def check_status(self) -> None:
        """Raise if a kernel of an earlier step flagged a bad index (this waits for the device, unless
        :meth:`read_back` has just brought the status word along)."""
        code, self._status_read = self._status_read, None
        if code is None:
            code = int(self.bufs.status.item())
        if code != 0:
            self.bufs.status.zero_()
            if self.device.type == "cuda":      # a kernel that gave up may have left its split counters half counted
                from .. import ops_tensor
                ops_tensor.reset_counters(self.device)
            raise StepError(f"device status {code}: {_status_text(code)}")
