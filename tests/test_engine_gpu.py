"""Generation through the Python entry point, compared with the plain implementation."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import TINY, TOL, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    tmp = str(tmp_path_factory.mktemp("models"))
    out = {}
    for name in TINY:
        d = make_model_dir(tmp, name)
        cfg, w = plain.read_model(d)
        out[name] = (d, cfg, w)
    return out


def make_engine(model_dir, dtype, name, **kw):
    from carbon_engine_b200 import Engine
    args = dict(dtype=dtype, page_size=TINY[name]["page_size"], kv_tokens=2048, max_seq_len=512, poison_cache=True)
    args.update(kw)
    return Engine(model_dir, **args)


# Two logits closer than this (relative to the row's largest) count as a tie: twice what a logit of the
# engine may be off by (float32: the replay's 1e-4; bfloat16: the replay's typical row, 2e-2).
GREEDY_MARGIN = {"float32": 2e-4, "bfloat16": 4e-2}


def check_greedy(cfg, w, prompt, got, dtype):
    """``got`` must be the plain implementation's greedy continuation; a different token is accepted
    only where the plain logits of the two candidates are closer than the precision's tolerance
    (the reference's own comparison treats such margins as ties, scripts/compare_reference.py:43-51),
    and the comparison then goes on from the engine's token."""
    toks = list(prompt)
    for i, t in enumerate(got):
        logits = plain.forward(cfg, w, toks)[-1]
        best = int(logits.argmax())
        if t != best:
            margin = float(logits[best] - logits[t])
            assert margin <= GREEDY_MARGIN[dtype] * float(logits.abs().max()), (i, t, best, margin)
        toks.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_config_a(models, dtype):
    from carbon_engine_b200 import SamplingParams
    d, cfg, w = models["A"]
    rng = np.random.default_rng(1)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (5, 11, 17)]
    eng = make_engine(d, dtype, "A")
    outs = eng.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "length" and len(o.token_ids) == 8 and o.prompt_token_ids == p
        check_greedy(cfg, w, p, o.token_ids, dtype)
        if dtype == "float32":
            assert o.token_ids == plain.greedy_generate(cfg, w, p, 8)
    st = eng.stats()
    assert st["finished"] == 3 and st["running"] == 0 and st["kv_pages_free"] == st["kv_pages_total"]
    eng.storage.manager.check()


def gumbel_pick(logits_row, temperature, seed):
    from carbon_engine_b200.sampling.sampler import mix64
    z = logits_row.astype(np.float64) / temperature
    idx = np.arange(len(z), dtype=np.uint64)
    best, second, best_i = -1e300, -1e300, -1
    for i in range(len(z)):
        h = mix64(seed ^ mix64((i + 0x632BE59BD9B4E019) & ((1 << 64) - 1)))
        u = ((h >> 40) + 0.5) / 16777216.0
        g = z[i] - math.log(-math.log(u))
        if g > best:
            second, best, best_i = best, g, i
        elif g > second:
            second = g
    return best_i, best - second


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_chunked_prefill_mixed_with_decode_and_seeded_temperature_config_b(models, dtype):
    """Prompts 3/9/24/40 under a 7-token step budget, so portions of prompts run beside decoded
    tokens; temperature 0.8 with a fixed seed gives the tokens the same draw gives on plain logits."""
    from carbon_engine_b200 import SamplingParams
    from carbon_engine_b200.sampling.sampler import step_seed
    d, cfg, w = models["B"]
    rng = np.random.default_rng(2)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (3, 9, 24, 40)]
    eng = make_engine(d, dtype, "B", max_prefill_tokens=7, max_running_requests=4)
    params = [SamplingParams(temperature=0.8, seed=100 + i, max_tokens=6, ignore_eos=True) for i in range(4)]
    outs = eng.generate(prompts, params)
    again = make_engine(d, dtype, "B", max_prefill_tokens=512, max_running_requests=4).generate(prompts, params)
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o.token_ids) == 6
        toks = list(p)
        for step, t in enumerate(o.token_ids):
            logits = plain.forward(cfg, w, toks)[-1].numpy().astype(np.float32)
            pick, margin = gumbel_pick(logits, 0.8, step_seed(100 + i, step))
            assert t == pick or margin < 2 * TOL[dtype] * np.abs(logits).max() / 0.8, (i, step, t, pick, margin)
            toks.append(t)
        if dtype == "float32":
            assert again[i].token_ids == o.token_ids           # the cut of the prompt does not change the draw
    assert eng.stats()["steps"] > 10                           # 76 prompt tokens at 7 a step


def test_small_cache_queues_requests_and_gives_the_same_tokens(models):
    """Few pages: requests wait for the pages of finished ones (src/scheduler.rs:636-641;
    tests/parallel.rs:380-392 in the reference).  Tokens equal those of each request run alone."""
    from carbon_engine_b200 import SamplingParams
    d, cfg, w = models["A"]
    rng = np.random.default_rng(3)
    prompts = [random_tokens(rng, int(n), cfg["vocab_size"]) for n in rng.integers(4, 40, size=10)]
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    big = make_engine(d, "float32", "A", kv_tokens=4096).generate(prompts, sp)
    small_eng = make_engine(d, "float32", "A", kv_tokens=112, max_prefill_tokens=16, max_running_requests=3)
    small = small_eng.generate(prompts, sp)
    for a, b in zip(big, small):
        assert a.token_ids == b.token_ids and b.finish_reason == "length"
    assert small_eng.stats()["kv_pages_total"] == 7 and small_eng.stats()["kv_pages_free"] == 7
    small_eng.storage.manager.check()


def test_identical_prompts_in_one_batch_give_identical_outputs(models):
    from carbon_engine_b200 import SamplingParams
    d, cfg, w = models["C"]
    p = random_tokens(np.random.default_rng(4), 50, cfg["vocab_size"])
    for dtype in ("float32", "bfloat16"):
        outs = make_engine(d, dtype, "C").generate([p, p, p], SamplingParams(max_tokens=12, ignore_eos=True))
        assert outs[0].token_ids == outs[1].token_ids == outs[2].token_ids


def test_requests_that_cannot_run_end_with_an_error_and_the_rest_go_on(models):
    from carbon_engine_b200 import SamplingParams
    d, cfg, w = models["A"]
    eng = make_engine(d, "float32", "A", kv_tokens=64, max_seq_len=128)
    ok = random_tokens(np.random.default_rng(5), 10, 256)
    outs = eng.generate([ok, [], list(range(100)), [1, 2, 999], ok],
                        [SamplingParams(max_tokens=4, ignore_eos=True), SamplingParams(), SamplingParams(max_tokens=50),
                         SamplingParams(), SamplingParams(max_tokens=4, ignore_eos=True)])
    assert [o.finish_reason for o in outs] == ["length", "error", "error", "error", "length"]
    assert "empty" in outs[1].error and "fit" in outs[2].error and "vocabulary" in outs[3].error
    assert outs[0].token_ids == outs[4].token_ids == plain.greedy_generate(cfg, w, ok, 4)


@pytest.mark.parametrize("ahead", [True, False])
def test_a_step_that_fails_on_the_device_ends_its_requests_and_the_engine_goes_on(models, ahead):
    """A kernel whose bounded wait gives up leaves a code in the device status word; it comes back with the
    picks.  Here the word is written from the host between two steps (nothing faults), while a step is in
    flight and another has been launched ahead of it: the requests of the failed step end with an error that
    names the code, the step launched ahead is dropped with them, pages and slots come back, the word is
    cleared, and the next request is served as if nothing had happened."""
    from carbon_engine_b200 import SamplingParams
    d, cfg, w = models["A"]
    rng = np.random.default_rng(9)
    prompts = [random_tokens(rng, n, 256) for n in (10, 4, 25)]
    eng = make_engine(d, "float32", "A", max_running_requests=4, run_ahead=ahead)
    ids = [eng.add_request(p, SamplingParams(max_tokens=40, ignore_eos=True)) for p in prompts]
    for _ in range(6):
        assert eng.step() == []
    assert (eng._in_flight is not None) == ahead
    eng.runner.bufs.status.fill_(7)
    outs = []
    for _ in range(4):
        outs += eng.step()
        if len(outs) == 3:
            break
    assert sorted(o.request_id for o in outs) == ids
    for o in outs:
        assert o.finish_reason == "error" and "device status 7" in o.error and "decode attention" in o.error
        assert 4 <= len(o.token_ids) < 40                                    # what it had generated stays with it
    assert eng._in_flight is None and not eng.has_unfinished()
    eng.storage.manager.check()
    st = eng.stats()
    assert eng.storage.manager.free_slots() == 4 and st["kv_pages_free"] == st["kv_pages_total"] and st["failed"] == 3
    assert int(eng.runner.bufs.status.item()) == 0
    again = eng.generate([prompts[2]], SamplingParams(max_tokens=6, ignore_eos=True))[0]
    assert again.finish_reason == "length" and again.token_ids == plain.greedy_generate(cfg, w, prompts[2], 6)


def test_eos_stop_and_sampling_options_through_the_entry_point(models):
    from carbon_engine_b200 import SamplingParams
    d, cfg, w = models["A"]
    p = random_tokens(np.random.default_rng(6), 12, 256)
    free_run = plain.greedy_generate(cfg, w, p, 8)
    eng = make_engine(d, "float32", "A")
    stop_at = free_run[3]
    first = free_run.index(stop_at)
    outs = eng.generate([p, p, p, p], [
        SamplingParams(max_tokens=8, stop_token_ids=[stop_at]),
        SamplingParams(max_tokens=8, stop_token_ids=[stop_at], ignore_eos=True),
        SamplingParams(max_tokens=8, temperature=0.9, top_k=1, seed=1),               # top_k 1 is greedy
        SamplingParams(max_tokens=8, logprobs=3),
    ])
    assert outs[0].finish_reason == "stop" and outs[0].token_ids == free_run[:first + 1]
    assert outs[1].finish_reason == "length" and outs[1].token_ids == free_run
    assert outs[2].token_ids == free_run and outs[3].token_ids == free_run           # logprobs do not change tokens
    lp = outs[3].logprobs
    assert len(lp) == 8 and lp[0]["token"] == free_run[0] and lp[0]["top"][0][0] == free_run[0]
    want = torch.log_softmax(plain.forward(cfg, w, p)[-1], dim=-1)
    assert abs(lp[0]["logprob"] - float(want[free_run[0]])) < 1e-4
    # a repetition penalty large enough forbids repeating the prompt's or the output's tokens
    rep = eng.generate([p], SamplingParams(max_tokens=8, repetition_penalty=1e6, presence_penalty=100.0, ignore_eos=True))[0]
    assert len(set(rep.token_ids)) == 8


def test_dummy_weights_equal_the_written_folder(models, tmp_path):
    """--dummy-weight makes, on the GPU, the same tensors that the random-weights mode writes."""
    from carbon_engine_b200 import Engine, SamplingParams
    d, cfg, w = models["B"]
    # the written folder of this fixture has sharpened q/k norms; compare with an untouched one
    plain_dir = make_model_dir(str(tmp_path), "B", sharpen=1.0)
    p = random_tokens(np.random.default_rng(7), 20, cfg["vocab_size"])
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    a = Engine(plain_dir, dtype="float32", kv_tokens=256, page_size=8).generate([p], sp)[0]
    b = Engine(plain_dir, dtype="float32", kv_tokens=256, page_size=8, dummy_weight=True, seed=TINY["B"]["seed"]).generate([p], sp)[0]
    assert a.token_ids == b.token_ids


def test_no_cpu_path():
    from carbon_engine_b200.engine.engine import require_gpu
    with pytest.raises(RuntimeError, match="CUDA device only"):
        require_gpu("cpu")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_cuda_graphs_give_the_same_tokens_as_eager(models, name, dtype):
    """Decode steps replayed as CUDA graphs (src/model/graph.rs:50-120; tests/parallel.rs:826-868 in the
    reference): same tokens, while batch size and context length change under the captured graphs.
    Configuration D runs the TMA decode kernel, whose grid (the split bound) is part of the graph's key:
    its contexts cross several bounds while the graphs are replayed."""
    from carbon_engine_b200 import SamplingParams, ops
    d, cfg, w = models[name]
    rng = np.random.default_rng(8)
    lengths = (30, 3, 250, 77, 12) if name == "B" else (620, 3, 250, 900, 77)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in lengths]
    sps = [SamplingParams(max_tokens=m, ignore_eos=True) for m in (40, 25, 30, 9, 50)]
    kw = dict(max_seq_len=1024) if name == "B" else dict(max_seq_len=2048, kv_tokens=8192)
    eager = make_engine(d, dtype, name, **kw).generate(prompts, sps)
    eng = make_engine(d, dtype, name, cuda_graphs=True, **kw)
    assert eng.cuda_graphs
    graphed = eng.generate(prompts, sps)
    for p, a, b in zip(prompts, eager, graphed):
        assert a.token_ids == b.token_ids
        check_greedy(cfg, w, p, b.token_ids, dtype)
    assert len(eng.runner._graphs) >= 3            # several batch sizes were captured
    if name == "D":
        assert len({key[1] for key in eng.runner._graphs}) >= 3      # and several split bounds
        if dtype == "bfloat16":
            assert ops.kernel_counts().get("attention_decode_tma_kernel (merge in the cluster)", 0) > 0


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "bfloat16")])
def test_host_lookahead_gives_the_same_tokens(models, graphs, name, dtype):
    """While a decode step runs, the next one is laid out on the host on the guess that the same requests
    go on with one token each.  The guess fails when a request finishes, a queued one is admitted or a
    late one arrives; the step then takes the ordinary way.  Same tokens either way, pages crossed and
    reused in between, no page or slot lost."""
    from carbon_engine_b200 import SamplingParams
    d, cfg, w = models[name]
    rng = np.random.default_rng(21)
    lengths = (20, 5, 61, 33, 9, 47) if name == "A" else (320, 5, 610, 33, 130, 470)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in lengths]
    sps = [SamplingParams(max_tokens=m, ignore_eos=True) for m in (35, 12, 50, 7, 41, 23)]
    kw = {} if name == "A" else dict(max_seq_len=1024, kv_tokens=4096)

    def run(lookahead):
        eng = make_engine(d, dtype, name, max_running_requests=4, cuda_graphs=graphs, host_lookahead=lookahead,
                          run_ahead=False, **kw)
        ids = [eng.add_request(p, s) for p, s in zip(prompts[:5], sps[:5])]
        done, steps, used = {}, 0, 0
        while eng.has_unfinished():
            for out in eng.step():
                done[out.request_id] = out.token_ids
            steps += 1
            if steps == 15:                           # a late arrival, in the middle of the others' decoding
                ids.append(eng.add_request(prompts[5], sps[5]))
            used += eng.runner._ahead is not None
        eng.storage.manager.check()
        assert eng.storage.manager.free_slots() == 4
        return [done[i] for i in ids], used

    plain_way, used_off = run(False)
    ahead_way, used_on = run(True)
    assert used_off == 0 and used_on > 20             # the layout in advance was really taken, many times
    assert plain_way == ahead_way
    for p, s, got in zip(prompts, sps, ahead_way):
        if dtype == "float32":
            assert got == plain.greedy_generate(cfg, w, p, s.max_tokens)
        else:
            check_greedy(cfg, w, p, got, dtype)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("D", "bfloat16"), ("E", "bfloat16")])
def test_a_step_launched_before_the_last_one_is_read_gives_the_same_tokens(models, graphs, name, dtype):
    """While requests only decode, the engine launches the step after the running one before it has read the
    running one's tokens; that step takes its token ids on the device.  What the host could not know then, a
    stop token or an abort, ends a request one computed token late, and that token is dropped.  A request
    that ends by length, or one that waits to be admitted, makes the engine take the ordinary way.  Same
    tokens either way (bit for bit in float32, seeded temperature rows included; bfloat16 against the plain
    implementation, since a late admission pairs other steps with the prompt), no page or slot lost, with
    windows that pages fall out of (B: 37 tokens, E: 200) and pages used again."""
    from carbon_engine_b200 import SamplingParams
    d, cfg, w = models[name]
    rng = np.random.default_rng(33)
    f32 = dtype == "float32"
    lengths = (20, 5, 61, 33, 9, 47) if name == "B" else (320, 5, 410, 33, 130, 270)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in lengths]
    new = (60, 12, 50, 7, 41, 23)
    kw = dict(max_seq_len=512, kv_tokens=1024) if name == "B" else dict(max_seq_len=1024, kv_tokens=2048)
    budget = 48 if name == "B" else 400

    def params(stop_of_0):
        return [SamplingParams(max_tokens=m, ignore_eos=i != 0, stop_token_ids=stop_of_0 if i == 0 else (),
                               temperature=0.7 if f32 and i in (1, 4) else 0.0, seed=50 + i) for i, m in enumerate(new)]

    def run(ahead, sps):
        eng = make_engine(d, dtype, name, max_running_requests=4, cuda_graphs=graphs, run_ahead=ahead,
                          max_prefill_tokens=budget, **kw)
        ids = [eng.add_request(p, s) for p, s in zip(prompts[:5], sps[:5])]
        done, steps = {}, 0
        while eng.has_unfinished():
            for out in eng.step():
                done[out.request_id] = (out.token_ids, out.finish_reason)
            steps += 1
            if steps == 15:                           # a late arrival, in the middle of the others' decoding
                ids.append(eng.add_request(prompts[5], sps[5]))
            if steps == 30:
                assert eng.abort(ids[2])              # ... and an abort while two steps are under way
        eng.storage.manager.check()
        assert eng.storage.manager.free_slots() == 4
        assert eng.stats()["kv_pages_free"] == eng.stats()["kv_pages_total"]
        return [done[i] for i in ids], eng.run_ahead_steps, steps

    free_run, _, _ = run(False, params(()))
    stop = free_run[0][0][17]                             # request 0 shall stop on a token it meets while it decodes
    sps = params([stop])
    one_by_one, used_off, steps_off = run(False, sps)
    ahead, used_on, steps_on = run(True, sps)
    assert used_off == 0 and used_on > 20                 # steps were really launched ahead, many times
    # nobody was kept waiting by it: the prompts, which take several steps under this budget, and the late
    # arrival got their turn as soon (a step later at most) as without it
    assert abs(steps_on - steps_off) <= 3
    cut = free_run[0][0].index(stop) + 1
    assert one_by_one[0] == (free_run[0][0][:cut], "stop") and cut < 60
    assert [r for _, r in ahead] == [r for _, r in one_by_one] == ["stop", "length", "abort", "length", "length", "length"]
    assert len(ahead[2][0]) == len(one_by_one[2][0]) < 50      # the abort took effect after the same step
    if f32:
        assert ahead == one_by_one
    for i, (p, (got, _)) in enumerate(zip(prompts, ahead)):
        if sps[i].temperature == 0.0:
            if f32:
                assert got == plain.greedy_generate(cfg, w, p, len(got))
            else:
                check_greedy(cfg, w, p, got, dtype)


def test_more_new_table_entries_than_a_steps_section_holds(models):
    """Requests that arrive with long contexts already in the cache (as the benchmark's harness makes them) bring
    more new block-table entries in their first step than the step's section of the pinned buffer holds: the
    surplus reaches the device tables by a copy of its own, and the step gives the same logits."""
    from carbon_engine_b200.cache.storage import CacheStorage
    from carbon_engine_b200.engine.batch import StepEntry
    from carbon_engine_b200.engine.engine import build_model
    from carbon_engine_b200.engine.runner import ModelRunner
    d, cfg, w = models["B"]
    dev = torch.device("cuda:0")
    model, _, _ = build_model(d, torch.float32, dev, max_seq_len=1024)
    out = {}
    for step_tokens in (16, 2048):
        storage = CacheStorage(model, torch.float32, dev, 8, 512, 4, 1024)
        g = torch.Generator(device=dev).manual_seed(5)
        for view in storage.paged_views():
            view.k_pool.normal_(0.0, 1.0, generator=g)
            view.v_pool.normal_(0.0, 1.0, generator=g)
        runner = ModelRunner(model, storage, step_tokens)
        for rid, ctx_len in enumerate((700, 90, 512, 333)):
            runner.open_request(rid)
            storage.manager.reserve(rid, ctx_len)
            storage.manager.commit(rid, ctx_len)
        cap = len(runner.bufs.host_section("upd_idx0"))
        assert (cap < 200) == (step_tokens == 16)                       # 205 entries are new in this step
        out[step_tokens] = runner.step([StepEntry(rid, [7 + rid], [0]) for rid in range(4)]).clone()
        runner.check_status()
    assert torch.isfinite(out[16]).all() and torch.equal(out[16], out[2048])
