"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

It runs only the tokens it is given, as one batch, against the cache that earlier steps left:
portions of prompts beside single decoded tokens, cut anywhere.  The reference's counterpart is
``Engine::forward(meta, tokens, sample_rows) -> f32 [rows, vocab]`` (src/engine.rs:407-446), fed
by either a prefill batch or a decode batch; here one call takes any mixture.
"""
from __future__ import annotations

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
        self._status_read = None             # the status word read_back brought along, until check_status takes it
        self.kernel_launches = 0

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
        the device tensor of wanted rows and the (request, new length) pairs to commit.

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
                ctx.h_tokens = tokens
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
        """Checks, page reservations and the step's layout in the pinned host buffer (nothing is sent)."""
        mgr = self.storage.manager
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.storage.max_requests:
            raise StepError(f"{len(entries)} entries, but only {self.storage.max_requests} requests may be live")
        order = sorted(range(len(entries)), key=lambda i: 0 if len(entries[i].tokens) == 1 else 1)
        T = sum(len(e.tokens) for e in entries)
        if T > self.max_step_tokens:
            raise StepError(f"{T} tokens in one step, but the engine was built for {self.max_step_tokens}")
        seen = set()
        if sum(len(e.want) for e in entries) > T:
            raise StepError("more wanted places than tokens in the step (a place is named twice)")
        for e in entries:
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request_id}: an entry needs at least one token")
            if e.request_id in seen:
                raise StepError(f"request {e.request_id} appears twice in one step")
            seen.add(e.request_id)
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise StepError(f"request {e.request_id}: wanted place {w} is outside its {len(e.tokens)} tokens")

        b = self.bufs
        b.wait_host_free()
        h_tok, h_pos, h_seq = b.host_section("tokens"), b.host_section("positions"), b.host_section("seq_of_token")
        h_slot, h_qs, h_ctx = b.host_section("seq_slot"), b.host_section("q_start"), b.host_section("ctx_len")
        ctx = StepContext(b, T, len(entries), self.dtype, self.device, self.storage.device_tables)
        ctx.fast_attention = self.fast_attention
        commits = []
        starts_sorted = {}
        upd = [([], []) for _ in self.storage.groups]
        off = 0
        for bi, i in enumerate(order):
            e = entries[i]
            n = len(e.tokens)
            start = mgr.length_of(e.request_id)
            slot = mgr.slot_of(e.request_id)
            mgr.reserve(e.request_id, start + n)
            h_tok[off:off + n] = np.asarray(e.tokens, dtype=np.int32)
            h_pos[off:off + n] = np.arange(start, start + n, dtype=np.int32)
            h_seq[off:off + n] = bi
            h_slot[bi] = slot
            h_qs[bi] = off
            h_ctx[bi] = start + n
            starts_sorted[i] = off
            ctx.h_slots.append(slot)
            ctx.h_q_start.append(off)
            ctx.h_ctx_before.append(start)
            if n == 1 and bi == ctx.n_decode:
                ctx.n_decode += 1
            ctx.max_position = max(ctx.max_position, start + n - 1)
            ctx.max_ctx = max(ctx.max_ctx, start + n)
            commits.append((e.request_id, start + n))
            for g in range(len(self.storage.groups)):
                u = self.storage.pending_table_updates(g, slot, start + n)
                if u is not None:
                    upd[g][0].append(u[0]); upd[g][1].append(u[1])
            off += n
        h_qs[len(entries)] = off
        ctx.h_q_start.append(off)
        for key, mixer in self._planners.items():
            ctx.plans[key] = mixer.plan_step(ctx)
        ctx.h_tokens = h_tok[:T].tolist()

        rows: List[int] = []
        for i, e in enumerate(entries):
            rows.extend(starts_sorted[i] + w for w in e.want)
        h_rows = b.host_section("rows")
        h_rows[:len(rows)] = np.asarray(rows, dtype=np.int32) if rows else 0
        n_upd = []
        for g in range(len(self.storage.groups)):
            if upd[g][0]:
                idx = np.concatenate(upd[g][0]); val = np.concatenate(upd[g][1])
                cap = len(b.host_section(f"upd_idx{g}"))
                if len(idx) > cap:
                    # more new table entries than a step's section holds (requests that arrive with long contexts
                    # already in the cache): the surplus goes to the device tables at once, by a copy of its own
                    self._write_table_entries(g, idx[cap:], val[cap:])
                    idx, val = idx[:cap], val[:cap]
                b.host_section(f"upd_idx{g}")[:len(idx)] = idx
                b.host_section(f"upd_val{g}")[:len(val)] = val
                n_upd.append(len(idx))
            else:
                n_upd.append(0)
        return ctx, len(rows), commits, n_upd

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
        for request_id, new_len in commits:
            self.storage.manager.commit(request_id, new_len)
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
        """Queue the copies of :meth:`read_back` behind what has been launched so far and return a ticket;
        work launched after this call does not delay them."""
        n = values.numel()
        k = self._back_turn = (self._back_turn + 1) % len(self._back)
        if self._back[k] is None or self._back[k][0].numel() < n + 1:
            self._back[k] = (torch.empty(max(n + 1, 257), dtype=torch.int32, pin_memory=True), torch.cuda.Event())
        buf, event = self._back[k]
        buf[:n].copy_(values.reshape(-1), non_blocking=True)
        buf[n:n + 1].copy_(self.bufs.status.reshape(-1)[:1], non_blocking=True)
        event.record()
        return k, n

    def finish_read_back(self, ticket) -> List[int]:
        k, n = ticket
        buf, event = self._back[k]
        event.synchronize()
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
