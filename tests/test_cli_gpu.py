"""The command line as a user runs it (subprocesses of ``bin/carbon``), and the engine on its own thread.

``tiny-model`` writes a folder, ``generate --print-ids`` prints the ids that ``Engine.generate`` and the
plain implementation give, greedy and with a seeded temperature, for one prompt and for a batch, and
``devices --selftest`` checks every kernel and names those it launched (src/main.rs:381-414, 973-1070;
src/device.rs:152-416 in the reference).
"""
import ast
import os
import re
import subprocess
import sys
import time

import numpy as np
import pytest

import plain_qwen3 as plain
from helpers import ROOT, random_tokens

pytestmark = pytest.mark.gpu
CARBON = [sys.executable, os.path.join(ROOT, "bin", "carbon")]


def run_cli(*args, ok=True):
    proc = subprocess.run(CARBON + list(args), capture_output=True, text=True, timeout=600)
    if ok:
        assert proc.returncode == 0, proc.stderr[-2000:]
    return proc


def output_ids(stderr: str):
    return [ast.literal_eval(m) for m in re.findall(r"output_ids: (\[[^\]]*\])", stderr)]


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("cli") / "tiny")
    p = run_cli("tiny-model", "--out", out, "--layers", "2", "--hidden", "64", "--heads", "4", "--kv-heads", "2",
                "--head-dim", "16", "--intermediate", "96", "--vocab", "263", "--seed", "3", "--max-positions", "512")
    assert "wrote" in p.stdout and os.path.exists(os.path.join(out, "model.safetensors"))
    return out


def test_generate_greedy_prints_the_plain_implementations_tokens(folder):
    cfg, w = plain.read_model(folder)
    prompt = random_tokens(np.random.default_rng(1), 14, cfg["vocab_size"])
    p = run_cli("generate", "--model", folder, "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "9",
                "--ignore-eos", "--print-ids", "--dtype", "f32", "--kv-tokens", "512", "--page-size", "16")
    want = plain.greedy_generate(cfg, w, prompt, 9)
    assert output_ids(p.stderr) == [want]
    assert [int(t) for t in p.stdout.split()] == want                      # streamed to standard output as they came
    assert re.search(r"\[Length\] prompt 14 tok, output 9 tok, ttft \d+\.\d+s, decode \d+\.\d tok/s", p.stderr)
    from carbon_engine_b200 import Engine, SamplingParams
    eng = Engine(folder, dtype="float32", kv_tokens=512, page_size=16)
    assert eng.generate([prompt], SamplingParams(max_tokens=9, ignore_eos=True))[0].token_ids == want


def test_generate_a_batch_with_a_seeded_temperature(folder):
    from carbon_engine_b200 import Engine, SamplingParams
    cfg, w = plain.read_model(folder)
    rng = np.random.default_rng(2)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (5, 30, 11)]
    args = ["generate", "--model", folder, "--max-tokens", "7", "--ignore-eos", "--print-ids", "--dtype", "f32",
            "--kv-tokens", "512", "--page-size", "16", "--temperature", "0.8", "--seed", "40"]
    for pr in prompts:
        args += ["--prompt-ids", ",".join(map(str, pr))]
    a, b = run_cli(*args), run_cli(*args)
    ids = output_ids(a.stderr)
    assert len(ids) == 3 and all(len(x) == 7 for x in ids)
    assert ids == output_ids(b.stderr)                                      # seeded: the same again
    eng = Engine(folder, dtype="float32", kv_tokens=512, page_size=16)
    outs = eng.generate(prompts, [SamplingParams(temperature=0.8, seed=40 + i, max_tokens=7, ignore_eos=True) for i in range(3)])
    assert [o.token_ids for o in outs] == ids
    lines = [l for l in a.stdout.splitlines() if l.startswith("[")]
    assert [[int(t) for t in l.split("] ")[1].split()] for l in lines] == ids
    greedy = eng.generate(prompts, SamplingParams(max_tokens=7, ignore_eos=True))
    assert [o.token_ids for o in greedy] != ids                              # the temperature really drew


def test_generate_reports_errors(folder):
    p = run_cli("generate", "--model", folder, "--prompt-ids", "1,2,999999", "--dtype", "f32", "--kv-tokens", "256",
                "--page-size", "16", ok=False)
    assert p.returncode != 0 and "vocabulary" in p.stderr
    p = run_cli("generate", "--model", folder, "--dtype", "f32", ok=False)
    assert p.returncode != 0 and "--prompt-ids" in p.stderr
    p = run_cli("generate", "--model", folder + "_nowhere", "--prompt-ids", "1", ok=False)
    assert p.returncode != 0 and "config.json" in p.stderr


def test_devices_selftest_checks_and_names_the_serving_kernels():
    p = run_cli("devices", "--selftest")
    assert "selftest: all ok" in p.stdout and "FAIL" not in p.stdout
    for name in ("attention_decode_tma_kernel (merge in the cluster)", "attention_prefill_tc_kernel", "gemm_tc_pair_kernel",
                 "gemm_tc_kernel (split-K, splits add together)", "sample_kernel", "argmax_kernel", "qk_rope_kvwrite"):
        assert name in p.stdout, name
    assert re.search(r"cuda:0 .* sm_100 ", p.stdout)


def test_engine_on_its_own_thread_streams_tokens_as_events(folder):
    """Submit returns at once; tokens arrive as events while later steps run; abort ends a request with
    ``Done('abort')``; a bad prompt gets an ``Error``; the tokens are those of ``Engine.generate``."""
    from carbon_engine_b200 import Engine, EngineHandle, SamplingParams
    from carbon_engine_b200.engine.handle import Done, Error, Token
    cfg, w = plain.read_model(folder)
    rng = np.random.default_rng(3)
    prompts = [random_tokens(rng, n, cfg["vocab_size"]) for n in (9, 40, 3, 25)]
    sps = [SamplingParams(max_tokens=m, ignore_eos=True) for m in (12, 30, 5, 300)]
    kw = dict(dtype="float32", kv_tokens=1024, page_size=16, max_running_requests=3, max_prefill_tokens=16)
    want = Engine(folder, **kw).generate(prompts[:3], sps[:3])
    with EngineHandle(Engine(folder, **kw)) as handle:
        t0 = time.perf_counter()
        streams = [handle.submit(p, s) for p, s in zip(prompts, sps)]
        assert time.perf_counter() - t0 < 0.5                                 # nothing ran in the caller's thread
        bad = handle.submit([1, 2, 10 ** 6])
        first = streams[1].get(timeout=120)
        assert isinstance(first, Token) and first.token_id == want[1].token_ids[0]
        st = handle.stats()
        assert st["running"] + st["waiting"] + st["finished"] >= 3
        handle.abort(streams[3].request_id)                                      # the long one, while it runs or waits
        for i in (0, 2):
            toks, end = streams[i].collect(timeout=120)
            assert toks == want[i].token_ids and end == Done("length", {"prompt_tokens": len(prompts[i]), "completion_tokens": len(toks)})
        rest, end = streams[1].collect(timeout=120)
        assert [first.token_id] + rest == want[1].token_ids and end.reason == "length"
        toks, end = streams[3].collect(timeout=120)
        assert isinstance(end, Done) and end.reason == "abort" and len(toks) < 300
        _, err = bad.collect(timeout=120)
        assert isinstance(err, Error) and "vocabulary" in err.message
        again = handle.submit(prompts[0], sps[0])                                # the engine goes on after all that
        assert again.collect(timeout=120)[0] == want[0].token_ids
        final = handle.stats()
        assert final["running"] == 0 and final["waiting"] == 0 and final["kv_pages_free"] == final["kv_pages_total"]
    late = handle.submit(prompts[0], sps[0])                                      # after shutdown
    assert isinstance(late.get(timeout=5), Error)
