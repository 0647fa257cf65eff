"""The host runtime's layout of a step (csrc/runtime/step_layout.cpp), called as the step function calls it:
order of the sequences, positions, rows of the wanted places, the block-table entries the device lacks,
its refusals, and that a refusal leaves the bookkeeping as it was (no GPU)."""
import ctypes

import numpy as np
import pytest

from carbon_engine_b200.cache.manager import CacheManager, GroupSpec
from carbon_engine_b200.csrc.runtime_lib import StepLayoutArgs, runtime


class Layout:
    """The arrays a caller owns: sections of the (here ordinary) host buffer, staging for table entries, results."""

    def __init__(self, cm: CacheManager, groups: int, max_tokens: int = 64):
        self.cm, self.max_tokens = cm, max_tokens
        n, self.stride = cm.max_requests, cm.max_requests * cm.max_pages_per_request
        i32 = lambda k: np.full(k, -7, dtype=np.int32)
        self.tok, self.pos, self.seq, self.rows = i32(max_tokens), i32(max_tokens), i32(max_tokens), i32(max_tokens)
        self.slot, self.qs, self.ctx = i32(n), i32(n + 1), i32(n)
        self.synced = np.zeros((groups, n), dtype=np.int64)
        self.upd_idx, self.upd_val = np.zeros((groups, self.stride), np.int32), np.zeros((groups, self.stride), np.int32)
        self.n_upd = np.zeros(groups, np.int32)
        self.out_ids, self.out_slot = np.zeros(n, np.int64), i32(n)
        self.out_before, self.out_len, self.out, self.detail = i32(n), i32(n), np.zeros(8, np.int32), np.zeros(3, np.int64)

    def __call__(self, entries):
        """entries: (request, tokens, wanted places).  Returns the status code."""
        ids = np.array([e[0] for e in entries], dtype=np.int64)
        counts = np.array([len(e[1]) for e in entries], dtype=np.int32)
        tokens = np.array([t for e in entries for t in e[1]] or [0], dtype=np.int32)
        wcounts = np.array([len(e[2]) for e in entries], dtype=np.int32)
        wants = np.array([w for e in entries for w in e[2]] or [0], dtype=np.int32)
        a = StepLayoutArgs()
        p = lambda arr: arr.ctypes.data
        a.n, a.ids, a.counts, a.tokens, a.want_counts, a.wants = len(entries), p(ids), p(counts), p(tokens), p(wcounts), p(wants)
        a.max_step_tokens = self.max_tokens
        a.tok, a.pos, a.seq_of_token, a.seq_slot, a.q_start, a.ctx_len, a.rows = map(
            p, (self.tok, self.pos, self.seq, self.slot, self.qs, self.ctx, self.rows))
        a.synced, a.upd_idx, a.upd_val, a.upd_stride, a.n_upd = p(self.synced), p(self.upd_idx), p(self.upd_val), self.stride, p(self.n_upd)
        a.out_ids, a.out_slot, a.out_ctx_before, a.out_new_len, a.out, a.detail = map(
            p, (self.out_ids, self.out_slot, self.out_before, self.out_len, self.out, self.detail))
        return runtime().step_layout(self.cm.handle, ctypes.byref(a))


def make(pages=32, window_pages=16):
    cm = CacheManager([GroupSpec(4, pages), GroupSpec(8, window_pages, window=16)], max_requests=4, max_pages_per_request=16)
    return cm, Layout(cm, 2)


def test_one_token_sequences_come_first_and_everything_is_where_the_kernels_read_it():
    cm, lay = make()
    for rid in (10, 11, 12):
        cm.open(rid)
    cm.reserve(11, 9); cm.commit(11, 9)                      # request 11 holds 9 tokens already
    cm.reserve(12, 30); cm.commit(12, 30)
    code = lay([(10, [5, 6, 7, 8, 9], [0, 4]), (11, [40], [0]), (12, [50, 51], [1])])
    assert code == 0
    T, n_rows, n_decode, max_position, max_ctx = lay.out[:5].tolist()
    assert (T, n_rows, n_decode, max_position, max_ctx) == (8, 4, 1, 31, 32)
    assert lay.out_ids[:3].tolist() == [11, 10, 12]                        # the one-token sequence leads
    assert lay.tok[:8].tolist() == [40, 5, 6, 7, 8, 9, 50, 51]
    assert lay.pos[:8].tolist() == [9, 0, 1, 2, 3, 4, 30, 31]
    assert lay.seq[:8].tolist() == [0, 1, 1, 1, 1, 1, 2, 2]
    assert lay.qs[:4].tolist() == [0, 1, 6, 8] and lay.ctx[:3].tolist() == [10, 5, 32]
    assert lay.slot[:3].tolist() == [cm.slot_of(11), cm.slot_of(10), cm.slot_of(12)] == lay.out_slot[:3].tolist()
    assert lay.out_before[:3].tolist() == [9, 0, 30] and lay.out_len[:3].tolist() == [10, 5, 32]
    assert lay.rows[:4].tolist() == [1, 5, 0, 7]                           # in the order of the entries and their wants
    assert lay.tok[8] == -7 and lay.rows[4] == -7                          # nothing beyond the step is touched
    # pages were reserved (lengths are committed by the step function once the step is on its way)
    assert cm.reserved_of(10) == 5 and cm.reserved_of(11) == 10 and cm.reserved_of(12) == 32 and cm.length_of(10) == 0
    # the device lacks every entry of these rows: group 0 (pages of 4) and group 1 (pages of 8, window 16)
    for g, ps in ((0, 4), (1, 8)):
        got = dict(zip(lay.upd_idx[g, :lay.n_upd[g]].tolist(), lay.upd_val[g, :lay.n_upd[g]].tolist()))
        want = {}
        for rid, length in ((11, 10), (10, 5), (12, 32)):
            slot, row = cm.slot_of(rid), cm.table(g)[cm.slot_of(rid)]
            for p in range((length + ps - 1) // ps):
                want[slot * 16 + p] = int(row[p])
        assert got == want
        assert lay.synced[g].tolist()[cm.slot_of(12)] == (32 + ps - 1) // ps
    assert -1 in lay.upd_val[1, :lay.n_upd[1]].tolist()                    # a page the window has passed is sent as gone
    # the next step of the same requests adds only what is new
    for rid, n in ((10, 5), (11, 10), (12, 32)):
        cm.commit(rid, n)
    assert lay([(10, [1], [0]), (11, [2], [0]), (12, [3], [0])]) == 0
    assert lay.out[:3].tolist() == [3, 3, 3] and lay.out_ids[:3].tolist() == [10, 11, 12]
    assert lay.n_upd.tolist() == [1, 1]                                    # request 12 starts page 8 of group 0 and page 4 of group 1
    assert lay.upd_idx[0, 0] == cm.slot_of(12) * 16 + 8 and lay.upd_idx[1, 0] == cm.slot_of(12) * 16 + 4
    cm.check()


@pytest.mark.parametrize("entries,code,detail", [
    ([], -101, None),
    ([(1, [1], []), (2, [1], []), (3, [1], []), (4, [1], []), (5, [1], [])], -102, [5, 4]),
    ([(1, list(range(40)), []), (2, list(range(30)), [])], -103, [70, 64]),
    ([(1, [1, 2], [0, 1, 1])], -104, None),
    ([(1, [1], [0]), (2, [], [])], -105, [2]),
    ([(1, [1], [0]), (2, [1, 2], []), (1, [3], [])], -106, [1]),
    ([(1, [1, 2, 3], [3])], -107, [1, 3, 3]),
    ([(1, [1], [0]), (9, [1], [0])], -3, [9]),                            # a request the cache does not know
])
def test_refusals_name_the_fault_and_change_nothing(entries, code, detail):
    cm, lay = make()
    for rid in (1, 2, 3, 4):
        cm.open(rid)
    before = (lay.synced.copy(), [cm.reserved_of(r) for r in (1, 2, 3, 4)], cm.free_pages(0), cm.free_pages(1))
    assert lay(entries) == code
    if detail is not None:
        assert lay.detail[:len(detail)].tolist() == detail
    after = (lay.synced, [cm.reserved_of(r) for r in (1, 2, 3, 4)], cm.free_pages(0), cm.free_pages(1))
    assert np.array_equal(before[0], after[0]) and before[1:] == after[1:]
    cm.check()


def test_when_pages_run_out_the_bookkeeping_of_the_table_entries_is_put_back():
    cm, lay = make(pages=6)                                                # group 0: 6 pages of 4 tokens
    for rid in (1, 2):
        cm.open(rid)
    assert lay([(1, list(range(12)), []), (2, list(range(20)), [])]) == -4  # request 1 takes 3 pages, request 2 needs 5
    assert lay.detail[:2].tolist() == [2, 20]
    assert not lay.synced.any()                                            # request 1's entries were never sent: all to do again
    assert cm.reserved_of(1) == 12 and cm.reserved_of(2) == 0             # (its pages stay with it)
    assert lay([(1, list(range(12)), [11])]) == 0
    assert lay.n_upd[0] == 3 and lay.synced[0, cm.slot_of(1)] == 3
    cm.check()
