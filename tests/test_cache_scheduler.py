"""The cache manager and the scheduler's decisions (no GPU)."""
import random

import numpy as np
import pytest

from carbon_engine_b200.cache.manager import CacheError, CacheManager, GroupSpec, OutOfPages
from carbon_engine_b200.engine.scheduler import Scheduler, SubmitError


def held_set(cm, rid, g=0):
    row = cm.table(g)[cm.slot_of(rid)]
    return [int(p) for p in row if p >= 0]


def test_pages_follow_length_and_come_back():
    cm = CacheManager([GroupSpec(8, 10)], max_requests=2, max_pages_per_request=16)
    s = cm.open(7)
    assert s == 0 and cm.free_slots() == 1
    cm.reserve(7, 17)                       # 3 pages
    assert cm.held_pages(7) == 3 and cm.free_pages() == 7
    cm.reserve(7, 17)                       # idempotent
    assert cm.held_pages(7) == 3
    cm.commit(7, 17)
    cm.reserve(7, 24); cm.commit(7, 24)     # still 3 pages
    assert cm.held_pages(7) == 3
    cm.reserve(7, 25)
    assert cm.held_pages(7) == 4
    cm.check()
    cm.close(7)
    assert cm.free_pages() == 10 and cm.free_slots() == 2 and (cm.table() == -1).all()
    cm.check()


def test_refusal_changes_nothing_and_pages_are_reused_low_first():
    cm = CacheManager([GroupSpec(4, 5)], 3, 8)
    cm.open(1); cm.reserve(1, 12); cm.commit(1, 12)          # pages 0,1,2
    cm.open(2)
    with pytest.raises(OutOfPages):
        cm.reserve(2, 12)                                     # needs 3, only 2 free
    assert cm.held_pages(2) == 0 and cm.free_pages() == 2
    cm.check()
    cm.close(1)
    cm.reserve(2, 12)
    assert held_set(cm, 2) == [0, 1, 2]                       # the freed pages are used again, low ids first
    cm.check()


def test_errors():
    cm = CacheManager([GroupSpec(4, 4)], 1, 2)
    cm.open(1)
    with pytest.raises(CacheError, match="already open"):
        cm.open(1)
    with pytest.raises(CacheError, match="slot"):
        cm.open(2)
    with pytest.raises(CacheError, match="more pages than"):
        cm.reserve(1, 9)
    with pytest.raises(CacheError, match="no such"):
        cm.reserve(5, 1)
    with pytest.raises(CacheError):
        cm.commit(1, 3)                                       # beyond what was reserved
    cm.close(1)
    with pytest.raises(CacheError, match="no such"):
        cm.close(1)                                           # freed twice
    cm.check()


def test_window_group_gives_pages_back_once_the_window_has_passed():
    cm = CacheManager([GroupSpec(4, 64, 0), GroupSpec(4, 6, 6)], 2, 64)
    cm.open(1)
    n = 0
    for chunk in (5, 1, 1, 7, 1, 1, 1, 9, 2):
        cm.reserve(1, n + chunk)
        # during the step every position from the first one a query still needs must have a page
        first_needed = max(0, n - 6 + 1)
        row = cm.table(1)[cm.slot_of(1)]
        for pos in range(first_needed, n + chunk):
            assert row[pos // 4] >= 0, (n, chunk, pos)
        n += chunk
        cm.commit(1, n)
        row = cm.table(1)[cm.slot_of(1)]
        keep_from = max(0, n - 6 + 1) // 4
        assert all(row[i] < 0 for i in range(keep_from)) and all(row[i] >= 0 for i in range(keep_from, (n + 3) // 4))
        assert cm.held_pages(1, 0) == (n + 3) // 4            # the full group keeps everything
        cm.check()
    assert cm.pages_for_lifetime(1, 1000, 9) == (6 - 1 + 9 + 3) // 4 + 1
    assert cm.pages_for_lifetime(0, 1000, 9) == 250
    cm.close(1)
    assert cm.free_pages(0) == 64 and cm.free_pages(1) == 6


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_share_a_page(seed):
    rng = random.Random(seed)
    cm = CacheManager([GroupSpec(4, 40, 0), GroupSpec(4, 24, 10)], 5, 32)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and cm.free_slots() > 0:
            cm.open(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = live[rid] + rng.choice([1, 1, 1, 2, 5, 13])
            if n > 120:
                continue
            try:
                cm.reserve(rid, n)
                cm.commit(rid, n)
                live[rid] = n
            except OutOfPages:
                pass
        elif live:
            rid = rng.choice(list(live))
            cm.close(rid); del live[rid]
        cm.check()
        owners = {}
        for g in range(2):
            for rid in live:
                for p in held_set(cm, rid, g):
                    assert (g, p) not in owners, "a page is held twice"
                    owners[(g, p)] = rid
        assert cm.open_requests() == len(live)
    for rid in list(live):
        cm.close(rid)
    cm.check()
    assert cm.free_pages(0) == 40 and cm.free_pages(1) == 24 and cm.free_slots() == 5


# ---- scheduler ------------------------------------------------------------------------------------
def make(pages=16, page_size=4, max_running=4, budget=8, max_seq_len=64, eos=(99,)):
    cm = CacheManager([GroupSpec(page_size, pages)], max_running, max_seq_len // page_size)
    return cm, Scheduler(cm, max_running, budget, max_seq_len, 100, eos)


def run_all(s, token_fn, max_steps=500):
    steps = []
    for _ in range(max_steps):
        if s.idle():
            break
        plan = s.plan()
        steps.append(plan)
        s.commit([token_fn(e) for e in plan if e.sample])
    return steps


def test_prompts_are_cut_under_the_budget_and_decoders_go_first():
    cm, s = make(pages=32, budget=8)
    s.submit(1, list(range(1, 12)), max_tokens=3)            # 11 prompt tokens
    s.submit(2, list(range(20, 25)), max_tokens=2)           # 5 prompt tokens
    p = s.plan()
    assert [(e.request_id, e.start, e.count, e.sample) for e in p] == [(1, 0, 8, False)]
    assert p[0].tokens == list(range(1, 9))
    s.commit([])
    p = s.plan()                                             # rest of 1 (3), then 5 of request 2
    assert [(e.request_id, e.start, e.count, e.sample) for e in p] == [(1, 8, 3, True), (2, 0, 5, True)]
    s.commit([50, 60])
    p = s.plan()                                             # both decode: one token each, their last sampled token
    assert [(e.request_id, e.start, e.count, e.tokens) for e in p] == [(1, 11, 1, [50]), (2, 5, 1, [60])]
    s.commit([51, 61])
    assert s.pop_finished() == [(2, "length")]
    p = s.plan()
    assert [(e.request_id, e.count) for e in p] == [(1, 1)]
    s.commit([52])
    assert s.pop_finished() == [(1, "length")]
    assert s.tokens_of(1)[11:] == [50, 51, 52] and s.idle()
    cm.check()
    assert cm.free_pages() == 32 and cm.free_slots() == 4


def test_a_decoding_request_is_never_starved_by_prompts():
    cm, s = make(pages=64, budget=6, max_seq_len=128)
    s.submit(1, [1, 2], max_tokens=20)
    s.commit([]) if False else None
    s.plan(); s.commit([5])
    s.submit(2, list(range(30)), max_tokens=2)
    for _ in range(5):
        p = s.plan()
        assert p[0].request_id == 1 and p[0].count == 1          # the decoder is in every step, first
        assert sum(e.count for e in p) <= 6
        s.commit([5] * sum(e.sample for e in p))


def test_stop_tokens_and_ignore_eos():
    cm, s = make()
    s.submit(1, [1, 2, 3], max_tokens=10)
    s.submit(2, [1, 2, 3], max_tokens=4, ignore_eos=True)
    s.submit(3, [1, 2, 3], max_tokens=10, stop_token_ids=[42])
    steps = run_all(s, lambda e: {1: 99, 2: 99, 3: 42}[e.request_id])
    fin = dict()
    # finished lists were popped inside run_all? no: collect now
    assert s.tokens_of(1)[3:] == [99]
    assert s.tokens_of(2)[3:] == [99, 99, 99, 99]
    assert s.tokens_of(3)[3:] == [42]
    assert sorted(s.pop_finished()) == [(1, "stop"), (2, "length"), (3, "stop")]
    cm.check()
    assert cm.free_pages() == 16


def test_submit_validation():
    cm, s = make(pages=4, page_size=4, max_seq_len=64)
    for prompt, msg in (([], "empty"), (list(range(64)), "room"), ([1, 100], "vocabulary")):
        with pytest.raises(SubmitError, match=msg):
            s.submit(9, prompt, 4)
    with pytest.raises(SubmitError, match="does not fit"):
        s.submit(9, [1] * 10, max_tokens=20)                  # 29 tokens -> 8 pages > 4
    s.submit(9, [1] * 10, max_tokens=4)
    with pytest.raises(SubmitError, match="already"):
        s.submit(9, [1], 1)
    assert Scheduler(cm, 2, 8, 64, 100).max_step_tokens == 8


def test_max_new_is_clamped_to_the_context():
    cm, s = make(pages=32, max_seq_len=16, budget=16)
    s.submit(1, [1] * 12, max_tokens=100)                     # at most 4 new tokens fit
    run_all(s, lambda e: 5)
    assert len(s.tokens_of(1)) == 16 and s.pop_finished() == [(1, "length")]


def test_when_pages_run_out_the_head_waits_and_running_requests_finish():
    # 8 pages of 4 tokens.  Each request: 9 prompt + 4 new - 1 = 12 tokens = 3 pages for its whole life.
    cm, s = make(pages=8, page_size=4, max_running=4, budget=32)
    for rid in (1, 2, 3):
        s.submit(rid, [1] * 9, max_tokens=4)
    p = s.plan()
    assert sorted(e.request_id for e in p) == [1, 2]           # the third would need pages the first two may still take
    assert s.stats()["waiting"] == 1 and s.stats()["running"] == 2
    s.commit([5, 5])
    order = []
    while not s.idle():
        p = s.plan()
        order.append(sorted(e.request_id for e in p))
        assert all(cm.held_pages(e.request_id) <= 3 for e in p)
        s.commit([5] * sum(e.sample for e in p))
        cm.check()
    assert [3] in order and order[0] == [1, 2]                 # request 3 ran after the others gave pages back
    assert sorted(s.pop_finished()) == [(1, "length"), (2, "length"), (3, "length")]
    assert cm.free_pages() == 8 and cm.free_slots() == 4


def test_a_request_that_can_never_run_ends_with_an_error():
    cm, s = make(pages=8, page_size=4, max_running=2, budget=32)
    cm.open(1000); cm.reserve(1000, 24)                        # somebody else holds 6 of the 8 pages
    s.submit(1, [1] * 9, max_tokens=4)                         # needs 3
    assert s.plan() == []
    assert s.pop_finished() == [(1, "error")] and s.idle()
    cm.close(1000)
    cm.check()


def test_max_running_is_respected_and_slots_are_reused():
    cm, s = make(pages=64, max_running=2, budget=32)
    for rid in range(5):
        s.submit(rid, [1, 2, 3], max_tokens=2)
    seen = []
    while not s.idle():
        p = s.plan()
        assert len(p) <= 2
        seen.append([e.request_id for e in p])
        s.commit([7] * sum(e.sample for e in p))
    assert sorted(r for r, _ in s.pop_finished()) == [0, 1, 2, 3, 4]
    assert seen[0] == [0, 1] and cm.free_slots() == 2


def test_a_failed_step_ends_its_requests_and_frees_their_pages():
    cm, s = make(pages=16, budget=4)
    s.submit(1, [1] * 3, max_tokens=4)
    s.submit(2, [1] * 10, max_tokens=4)
    p = s.plan()                                               # request 1 whole (3), request 2 gets 1 token
    assert [e.request_id for e in p] == [1, 2]
    s.fail_step()
    assert sorted(s.pop_finished()) == [(1, "error"), (2, "error")]
    assert cm.free_pages() == 16 and cm.free_slots() == 4 and s.idle()
    s.submit(3, [1, 2], max_tokens=1)                          # the scheduler keeps serving
    run_all(s, lambda e: 9)
    assert s.pop_finished() == [(3, "length")]
    cm.check()


def test_abort_waiting_and_running():
    cm, s = make(pages=16, max_running=1, budget=8)
    s.submit(1, [1] * 4, max_tokens=8)
    s.submit(2, [1] * 4, max_tokens=8)
    s.plan(); s.commit([5])
    assert s.abort(2) and s.abort(1) and not s.abort(1)
    assert sorted(s.pop_finished()) == [(1, "abort"), (2, "abort")]
    assert s.idle() and cm.free_pages() == 16
    cm.check()


def test_the_step_after_the_last_one_is_planned_for_the_requests_it_was_launched_for():
    """``plan_for``: the engine has put the step after the last one on the device already, for the requests
    that decoded; the scheduler lays out exactly that step for those that still run and admits nothing."""
    cm, s = make(pages=32, max_running=3, budget=8)
    s.submit(1, [1, 2, 3], max_tokens=6)
    s.submit(2, [4, 5], max_tokens=6)
    s.submit(3, [6], max_tokens=3, stop_token_ids=[42])
    assert s.waiting() == 3 and s.remaining(1) == 6 and s.remaining(77) == -1
    s.plan(); s.commit([10, 20, 30])
    assert s.waiting() == 0 and s.running() == 3 and [s.remaining(r) for r in (1, 2, 3)] == [5, 5, 2]
    s.submit(4, [7, 8], max_tokens=2)                         # arrives while two steps are under way
    p = s.plan_for([1, 2, 3])
    assert [(e.request_id, e.start, e.count, e.sample, e.tokens) for e in p] == \
        [(1, 3, 1, True, [10]), (2, 2, 1, True, [20]), (3, 1, 1, True, [30])]
    assert s.waiting() == 1                                   # request 4 was not admitted
    s.commit([11, 21, 42])                                    # request 3 meets its stop token
    assert s.pop_finished() == [(3, "stop")] and s.remaining(3) == -1
    p = s.plan_for([1, 2, 3])                                 # the step launched for all three: 3 has ended
    assert [(e.request_id, e.start, e.tokens) for e in p] == [(1, 4, [11]), (2, 3, [21])]
    s.commit([12, 22])
    assert s.abort(1)
    p = s.plan_for([1, 2])
    assert [(e.request_id, e.start, e.tokens) for e in p] == [(2, 4, [22])]
    s.commit([23])
    assert s.plan_for([1]) == [] and s.plan_for([]) == []
    p = s.plan()                                              # the ordinary plan goes on, and admits request 4
    assert [(e.request_id, e.start, e.count) for e in p] == [(2, 5, 1), (4, 0, 2)]
    s.commit([24, 40])
    run_all(s, lambda e: 5)
    assert s.tokens_of(2)[2:] == [20, 21, 22, 23, 24, 5] and s.idle()
    cm.check()
    assert cm.free_pages() == 32 and cm.free_slots() == 3


def test_stats_count_tokens():
    cm, s = make(pages=32, budget=8)
    s.submit(1, [1] * 11, max_tokens=3)
    run_all(s, lambda e: 5)
    st = s.stats()
    assert st["prefill_tokens"] == 11 and st["decode_tokens"] == 2 and st["steps"] == 4 and st["finished"] == 1


@pytest.mark.parametrize("seed", range(6))
def test_random_workloads_keep_the_schedulers_promises(seed):
    """Random arrivals, prompt lengths, budgets, pool sizes, stop tokens, aborts and failed steps: every step
    keeps the token budget and carries every decoding request once, positions follow on without a gap,
    the pool is never overdrawn, and at the end every request has finished with what it was promised."""
    rng = random.Random(seed)
    page_size = rng.choice([2, 4, 8])
    max_running = rng.randint(1, 5)
    budget = rng.randint(max_running, 12)
    max_seq_len = rng.choice([32, 64])
    pages = rng.randint(max_seq_len // page_size, 3 * max_seq_len // page_size)
    cm, s = make(pages=pages, page_size=page_size, max_running=max_running, budget=budget, max_seq_len=max_seq_len, eos=(99,))
    todo = list(range(1, 25))
    want, stops, aborted, failed = {}, {}, set(), set()
    pos = {}                                   # request -> tokens the scheduler has handed out so far
    decoding = set()
    finished = {}
    for step in range(4000):
        while todo and rng.random() < 0.4:     # arrivals
            rid = todo.pop(0)
            n_prompt = rng.randint(1, max_seq_len - 2)
            max_tokens = rng.randint(1, 12)
            stop = [98] if rng.random() < 0.3 else []
            s.submit(rid, [rng.randrange(90) for _ in range(n_prompt)], max_tokens=max_tokens,
                     ignore_eos=rng.random() < 0.2, stop_token_ids=stop)
            want[rid] = (n_prompt, min(max_tokens, max_seq_len - n_prompt))
            stops[rid] = stop
            pos[rid] = 0
        if s.idle():
            if not todo:
                break
            continue
        if rng.random() < 0.03 and pos:        # an abort now and then
            rid = rng.choice(list(pos))
            if rid not in finished and s.abort(rid):
                aborted.add(rid)
                decoding.discard(rid)
        plan = s.plan()
        assert sum(e.count for e in plan) <= budget
        ids = [e.request_id for e in plan]
        assert len(ids) == len(set(ids)) and len(ids) <= max_running
        assert decoding <= set(ids)            # nobody who decodes is left out of a step
        for e in plan:
            assert e.start == pos[e.request_id] and e.count == len(e.tokens) and e.count >= 1
            if e.request_id in decoding:
                assert e.count == 1 and e.sample
        assert cm.free_pages() >= 0
        cm.check()
        if plan and rng.random() < 0.03:       # the step fails: its requests end with an error, the pool gets their pages back
            s.fail_step()
            for e in plan:
                failed.add(e.request_id)
                decoding.discard(e.request_id)
        elif plan:
            for e in plan:
                pos[e.request_id] += e.count
                if e.sample:
                    decoding.add(e.request_id)
            s.commit([rng.choice([5, 6, 7, 98, 99]) for e in plan if e.sample])
        for rid, reason in s.pop_finished():
            finished[rid] = reason
            decoding.discard(rid)
            toks = s.tokens_of(rid)
            n_prompt, max_new = want[rid]
            gen = toks[n_prompt:]
            if reason == "length":
                assert len(gen) == max_new
            elif reason == "stop":
                assert 1 <= len(gen) <= max_new and (gen[-1] == 99 or gen[-1] in stops[rid])
            elif reason == "abort":
                assert rid in aborted
            else:
                assert reason == "error" and (rid in failed or n_prompt + max_new - 1 > pages * page_size)
            s.forget(rid)
    assert not todo and s.idle()
    assert set(finished) == set(want)
    cm.check()
    assert cm.free_pages() == pages and cm.free_slots() == max_running
