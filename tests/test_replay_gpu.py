"""Trace replay through bin/trace_run, compared with the plain implementation.

For every tiny configuration and both precisions ONE trace_run process replays the same requests
whole, with the last 32 tokens decoded one by one, in portions of changing size (down to two
tokens, and one-token portions at the very start of a sequence), as a long decode, and mixed: up to
four live requests, portions of some beside single tokens of others, requests left out of steps,
with so few pages that the pages of finished requests are used again.  Fresh pages are filled with
NaN, so a read of a place that was never written shows; reused pages hold another request's keys,
so a read of a stale place shows as a wrong number.

In float32 the rows of every later cut must EQUAL, bit for bit, the rows the whole request gave: the
32-bit kernels take a token's sums in an order that depends on its position only (the reference forces
float32 in its own equivalence suite for the same reason, tests/parallel.rs:125-126).

Configurations D and E have the head sizes of real checkpoints and prompts of several hundred tokens;
their bfloat16 replays must have launched the kernels that serving runs (the report trace_run writes).
"""
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import (TINY, TOL, TOL_MODEL_BF16_MEDIAN, TOL_MODEL_BF16_ROW, TraceRun, make_model_dir,
                     random_tokens)

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [150, 97, 64, 33, 120, 70, 1, 2, 3], "B": [141, 100, 57, 40, 90, 64, 1, 2, 3],
           "C": [170, 101, 64, 35, 128, 77, 1, 2, 3],
           "D": [900, 610, 333, 300, 700, 420, 1, 2, 3], "E": [777, 515, 290, 300, 640, 400, 1, 2, 3]}
# the most tokens live requests hold (each rounded up to 64): four live requests fill the pool exactly
MAX_TOKENS = {"A": 448, "B": 448, "C": 448,           # 192 + 128 + 64 + 64
              "D": 2304, "E": 2048}                     # 960 + 640 + 384 + 320; 832 + 576 + 320 + 320
# the long decode: (prompt tokens, tokens decoded one by one)
LONG = {"A": (8, 260), "B": (8, 260), "C": (8, 260), "D": (560, 230), "E": (600, 180)}
# portion sizes of cut 3, taken in turn; the long ones cross several 128-query tiles over a cached prefix
PORTIONS = {name: [1, 1, 2, 7, 2, 19, 3, 2, 31, 5, 16, 2, 40, 9] for name in "ABC"}
PORTIONS["D"] = PORTIONS["E"] = [1, 1, 2, 130, 7, 300, 2, 257, 64, 19, 128, 3, 40]
# what a mixed step gives a request that is still in its prompt
MIXED_PORTIONS = {name: [2, 3, 5, 8, 13, 30] for name in "ABC"}
MIXED_PORTIONS["D"] = MIXED_PORTIONS["E"] = [2, 3, 9, 14, 70, 130, 260]
# kernels a bfloat16 replay of a configuration must have launched
MUST_LAUNCH = {
    "D": ["attention_decode_tma_kernel (merge in the cluster)", "attention_prefill_tc_kernel", "gemm_tc_pair_kernel",
          "gemm_tc_kernel (split-K)", "gemm_tc_kernel (split-K, splits add together)", "qk_rope_kvwrite_warp_kernel"],
    "E": ["attention_decode_tma_kernel (merge in the cluster)", "attention_prefill_tc_kernel", "gemm_tc_pair_kernel",
          "gemm_tc_kernel (split-K)"],
}


class Case:
    def __init__(self, tmp, name):
        self.name = name
        self.dir = make_model_dir(tmp, name)
        self.cfg, w = plain.read_model(self.dir)
        rng = np.random.default_rng(TINY[name]["seed"])
        self.reqs = [random_tokens(rng, n, self.cfg["vocab_size"]) for n in LENGTHS[name]]
        self.long = random_tokens(rng, sum(LONG[name]), self.cfg["vocab_size"])
        self.want = [plain.forward(self.cfg, w, t).numpy() for t in self.reqs]
        self.want_long = plain.forward(self.cfg, w, self.long).numpy()


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    tmp = str(tmp_path_factory.mktemp("models"))
    return {name: Case(tmp, name) for name in TINY}


class Checker:
    def __init__(self, dtype):
        self.tol = TOL[dtype] if dtype == "float32" else TOL_MODEL_BF16_ROW
        self.median_tol = TOL[dtype] if dtype == "float32" else TOL_MODEL_BF16_MEDIAN
        self.worst = 0.0
        self.rows = []

    def check(self, got, want, what, same_as=None):
        assert got is not None and got.shape == want.shape, what
        assert np.isfinite(got).all(), f"{what}: non-finite logits (a read of a place never written?)"
        if same_as is not None and not np.array_equal(got, same_as):
            rows = np.nonzero((got != same_as).any(axis=1))[0]
            raise AssertionError(f"{what}: float32 rows differ from those of the whole request (first at row {rows[0]} of "
                                 f"{len(got)}, largest difference {np.abs(got - same_as).max():.3e}): a sum depends on the cut")
        scale = np.abs(want).max()
        err = np.abs(got - want).max() / scale
        self.worst = max(self.worst, err)
        self.rows.extend((np.abs(got - want).max(axis=1) / scale).tolist())
        if err > self.tol:
            per_row = np.abs(got - want).max(axis=1) / scale
            first = int(np.argmax(per_row > self.tol))
            raise AssertionError(f"{what}: relative error {err:.3e} > {self.tol:.0e}; first wrong row {first} "
                                 f"of {len(per_row)} (errors {per_row[max(0, first - 2):first + 3]})")


def replay_all(case: Case, dtype: str, out_dir: str):
    max_tokens = max(MAX_TOKENS[case.name], (len(case.long) + 63) // 64 * 64)
    report = out_dir + ".kernels.json"
    tr = TraceRun(case.dir, dtype, out_dir, max_tokens, TINY[case.name]["page_size"],
                  extra=["--poison", "--kernel-report", report])
    ck = Checker(dtype)
    rng = np.random.default_rng(99)
    exact = dtype == "float32"
    whole = {}

    def same(i, lo, hi):
        return whole[i][lo:hi] if exact else None
    try:
        # 1. each request alone and whole
        for i, toks in enumerate(case.reqs):
            got = tr.step([{"id": f"w{i}", "tokens": toks, "want": list(range(len(toks)))}], end=[f"w{i}"])
            ck.check(got, case.want[i], f"whole request {i}")
            whole[i] = got
        got = tr.step([{"id": "wl", "tokens": case.long, "want": list(range(len(case.long)))}], end=["wl"])
        ck.check(got, case.want_long, "whole long request")
        whole["long"] = got
        # 2. most of it in one step, the last 32 tokens one by one
        for i, toks in enumerate(case.reqs[:4]):
            L = len(toks)
            head = max(1, L - 32)
            got = tr.step([{"id": f"t{i}", "tokens": toks[:head], "want": [head - 1]}])
            ck.check(got, case.want[i][head - 1:head], f"tail decode {i}: prompt", same(i, head - 1, head))
            for p in range(head, L):
                got = tr.step([{"id": f"t{i}", "tokens": [toks[p]], "want": [0]}], end=[f"t{i}"] if p == L - 1 else [])
                ck.check(got, case.want[i][p:p + 1], f"tail decode {i}: position {p}", same(i, p, p + 1))
        # 3. portions of changing size, down to two tokens; one-token portions at the very start
        sizes = PORTIONS[case.name]
        for i, toks in enumerate(case.reqs[:6]):
            p, k = 0, i
            while p < len(toks):
                n = min(sizes[k % len(sizes)], len(toks) - p)
                k += 1
                last = p + n == len(toks)
                got = tr.step([{"id": f"p{i}", "tokens": toks[p:p + n], "want": list(range(n))}], end=[f"p{i}"] if last else [])
                ck.check(got, case.want[i][p:p + n], f"portions {i}: positions {p}..{p + n}", same(i, p, p + n))
                p += n
        # 4. long decoding: a prompt, then a few hundred tokens one by one
        n0 = LONG[case.name][0]
        got = tr.step([{"id": "long", "tokens": case.long[:n0], "want": [n0 - 1]}])
        ck.check(got, case.want_long[n0 - 1:n0], "long decode: prompt", same("long", n0 - 1, n0))
        for p in range(n0, len(case.long)):
            got = tr.step([{"id": "long", "tokens": [case.long[p]], "want": [0]}], end=["long"] if p == len(case.long) - 1 else [])
            ck.check(got, case.want_long[p:p + 1], f"long decode: position {p}", same("long", p, p + 1))
        # 5. mixed: up to four live, portions beside single tokens, requests left out, pages used again
        order = [0, 1, 2, 3, 4, 5, 3, 2, 0, 5]
        waiting = list(enumerate(order))
        live = {}        # key -> [request index, position]
        held = 0
        rounded = lambda n: (n + 63) // 64 * 64
        steps = 0
        while waiting or live:
            while waiting and len(live) < 4 and held + rounded(len(case.reqs[waiting[0][1]])) <= MAX_TOKENS[case.name]:
                j, r = waiting.pop(0)
                live[f"m{j}"] = [r, 0]
                held += rounded(len(case.reqs[r]))
            entries, wants, ends = [], [], []
            for key, (r, p) in list(live.items()):
                toks = case.reqs[r]
                if len(live) > 1 and rng.random() < 0.2:
                    continue                                   # left out of this step, goes on later
                decode_from = max(1, len(toks) - 24)
                n = 1 if p >= decode_from else min(int(rng.choice(MIXED_PORTIONS[case.name])), decode_from - p)
                want = sorted(set(rng.integers(0, n, size=min(n, 3)).tolist())) if rng.random() < 0.9 else []
                entries.append({"id": key, "tokens": toks[p:p + n], "want": want})
                wants.append((r, p, want))
                live[key][1] = p + n
                if p + n == len(toks):
                    ends.append(key)
            if not entries:
                continue
            got = tr.step(entries, end=ends)
            steps += 1
            if got is not None:
                expect = np.concatenate([case.want[r][[p + w for w in want]] for r, p, want in wants if want])
                again = np.concatenate([whole[r][[p + w for w in want]] for r, p, want in wants if want]) if exact else None
                ck.check(got, expect, f"mixed step {steps} ({[(e['id'], len(e['tokens'])) for e in entries]})", again)
            for key in ends:
                held -= rounded(len(case.reqs[live[key][0]]))
                del live[key]
        assert tr.close() == 0
    finally:
        if tr.proc.poll() is None:
            tr.proc.kill()
    assert np.median(ck.rows) <= ck.median_tol, f"median row error {np.median(ck.rows):.3e}"
    if dtype == "bfloat16":
        with open(report) as fh:
            launched = json.load(fh)
        missing = [k for k in MUST_LAUNCH.get(case.name, []) if launched.get(k, 0) == 0]
        assert not missing, f"config {case.name}: never launched {missing}; launched {sorted(launched)}"
    return ck.worst, ck.tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_replay_matches_plain_under_every_cut(cases, tmp_path, name, dtype):
    worst, tol = replay_all(cases[name], dtype, str(tmp_path / "out"))
    print(f"config {name} {dtype}: worst relative error {worst:.3e}")
    assert worst <= tol


def test_trace_run_reports_a_full_pool(cases, tmp_path):
    """Asking for more tokens than the pool was made for fails loudly instead of overwriting pages."""
    case = cases["A"]
    tr = TraceRun(case.dir, "float32", str(tmp_path / "o"), 64, 16)
    try:
        tr.step([{"id": "a", "tokens": case.reqs[2][:60], "want": [0]}])
        with pytest.raises(RuntimeError):
            tr.step([{"id": "b", "tokens": case.reqs[3][:20], "want": [0]}])
        assert tr.proc.wait(timeout=60) != 0
    finally:
        if tr.proc.poll() is None:
            tr.proc.kill()
