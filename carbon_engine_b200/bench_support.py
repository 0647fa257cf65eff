"""What bench.py measures with: an engine at given layer sizes with random weights, decode steps
timed on the device, the same through the public entry point, and a one-step prefill."""
from __future__ import annotations

import time
from typing import Dict, List

import numpy as np
import torch

from . import ops
from .config.qwen3 import Qwen3Config
from .engine.batch import StepEntry
from .engine.engine import Engine
from .sampling.params import SamplingParams


class BenchHarness:
    def __init__(self, cfg: Dict, max_batch: int, context: int, new_tokens: int, graphs: bool = True,
                 page_size: int = 64, seed: int = 0, step_tokens: int = 4096):
        raw = dict(cfg, architectures=["Qwen3ForCausalLM"], model_type="qwen3")
        self.config = Qwen3Config.from_dict(raw)
        self.context, self.new_tokens, self.page_size, self.max_batch = context, new_tokens, page_size, max_batch
        self.seed = seed
        per_seq = (context + new_tokens + page_size - 1) // page_size * page_size
        self.max_seq_len = max(4096, per_seq)
        self.engine = Engine(config=self.config, dtype="bfloat16", dummy_weight=True, seed=seed,
                             kv_tokens=max_batch * per_seq + 4096, page_size=page_size, max_seq_len=max(4096, per_seq),
                             max_running_requests=max_batch, max_prefill_tokens=step_tokens, cuda_graphs=graphs)
        self.graphs = bool(graphs and self.engine.runner.graphs_enabled)
        self.rng = np.random.default_rng(seed)
        self._next = 1 << 40
        g = torch.Generator(device=self.engine.device).manual_seed(seed)
        for view in self.engine.storage.paged_views():          # a cache that holds plausible keys and values
            for pool in (view.k_pool, view.v_pool):
                pool.normal_(0.0, 1.0, generator=g)

    def _tokens(self, n: int) -> List[int]:
        return self.rng.integers(0, self.config.vocab_size, size=n).tolist()

    def _open_with_context(self, batch: int) -> List[int]:
        """Requests whose first ``context`` positions are already in the cache (random keys/values)."""
        runner, mgr = self.engine.runner, self.engine.storage.manager
        ids = []
        for _ in range(batch):
            rid = self._next
            self._next += 1
            runner.open_request(rid)
            mgr.reserve(rid, self.context)
            mgr.commit(rid, self.context)
            ids.append(rid)
        return ids

    def decode(self, batch: int, steps: int, warmup: int, pick: bool = True) -> Dict:
        """``steps`` decode steps of ``batch`` sequences timed on the device; ``pick``: each step ends with the
        greedy pick of every sequence's next token (False: the step ends with the logits)."""
        runner = self.engine.runner
        ids = self._open_with_context(batch)
        out = torch.empty(batch, dtype=torch.int32, device=self.engine.device)
        toks = [self._tokens(batch) for _ in range(steps + warmup)]

        def one(i):
            logits = runner.step([StepEntry(r, [toks[i][j]], [0]) for j, r in enumerate(ids)])
            if pick:
                ops.argmax(logits, out)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = ops.launch_count()
        start.record()
        for i in range(warmup, warmup + steps):
            one(i)
        end.record()
        torch.cuda.synchronize()
        runner.check_status()
        ms = start.elapsed_time(end) / steps
        for r in ids:
            runner.close_request(r)
        return {"ms_per_step": ms, "tokens_per_s": batch / (ms / 1e3), "launches": ops.launch_count() - l0}

    def decode_e2e(self, batch: int, steps: int, warmup: int) -> Dict:
        """Through Engine.add_request / Engine.step: real prompts are prefilled, then ``steps`` decode
        steps are timed on the host clock between two synchronisations."""
        eng = self.engine
        # The prompts' prefill just before draws the most power a step can; the clocks need some tens of
        # milliseconds of decoding to settle again, so at least 32 steps are left untimed.
        warmup = max(warmup, 32)
        # long enough that no request ends inside the timed region: a request whose prompt is done decodes
        # through every step that the later prompts' portions take
        prompt_steps = batch * ((self.context + eng.max_step_tokens - 1) // eng.max_step_tokens + 1)
        if warmup + steps + prompt_steps + 8 > self.new_tokens:
            raise ValueError(f"the harness was sized for {self.new_tokens} new tokens a request; this run needs "
                             f"{warmup + steps + prompt_steps + 8}")
        sp = SamplingParams(max_tokens=warmup + steps + prompt_steps + 8, ignore_eos=True)
        before = eng.scheduler.stats()["prefill_tokens"]
        for _ in range(batch):
            eng.add_request(self._tokens(self.context), sp)
        while eng.scheduler.stats()["prefill_tokens"] - before < batch * self.context:
            for out in eng.step():
                raise RuntimeError(f"a request ended during the prompts ({out.finish_reason}: {out.error})")
            if not eng.has_unfinished():
                raise RuntimeError("the engine ran out of work before the prompts were done")
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        h2d = d2h = 0
        ahead0 = eng.run_ahead_steps
        for _ in range(steps):
            eng.step()
            h2d += eng.runner.h2d_bytes_last
            d2h += eng.d2h_bytes_last
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        ahead = eng.run_ahead_steps - ahead0
        while eng.has_unfinished():
            eng.step()
        return {"ms_per_step": dt / steps * 1e3, "tokens_per_s": batch * steps / dt, "h2d_bytes": h2d // steps,
                "d2h_bytes": d2h // steps, "launched_ahead": ahead}

    def between_steps(self, batch: int, steps: int = 6) -> Dict:
        """What the device does between the last kernel of one decode step and the first of the next, through
        Engine.add_request / Engine.step: device activities (PyTorch profiler, CUDA only) that precede each
        step's first kernel, in microseconds relative to it, and the steps' period."""
        from torch.profiler import ProfilerActivity, profile
        eng = self.engine
        sp = SamplingParams(max_tokens=self.new_tokens - 8, ignore_eos=True)
        for _ in range(batch):
            eng.add_request(self._tokens(self.context), sp)
        for _ in range(batch * ((self.context + eng.max_step_tokens - 1) // eng.max_step_tokens + 1) + 32):
            eng.step()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(steps):
                eng.step()
            torch.cuda.synchronize()
        while eng.has_unfinished():
            eng.step()
        ev = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda e: e.time_range.start)
        rows = [(e.name, e.time_range.start, e.time_range.end) for e in ev]
        firsts = [i for i, r in enumerate(rows) if "embed_kernel" in r[0]]
        out = {"period_us": None, "before_a_step": []}
        if len(firsts) >= 3:
            i = firsts[2]
            out["period_us"] = round(rows[i][1] - rows[firsts[1]][1], 1)
            out["before_a_step"] = [{"activity": n[:60], "start_us": round(s - rows[i][1], 1), "us": round(e - s, 1)}
                                    for n, s, e in rows[max(i - 7, 0):i + 1]]
        return out

    def serve(self, prompt_lens: List[int], new_tokens: int) -> Dict:
        """A whole workload through Engine.add_request / Engine.step: all requests are queued at once, the
        scheduler admits them, cuts their prompts into portions under the step's token budget beside the
        decoding requests, and frees them as they finish.  Timed on the host clock between two
        synchronisations."""
        eng = self.engine
        sp = SamplingParams(max_tokens=new_tokens, ignore_eos=True)
        for n in prompt_lens:
            eng.add_request(self._tokens(n), sp)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        steps, l0 = 0, ops.launch_count()
        while eng.has_unfinished():
            eng.step()
            steps += 1
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        eng.runner.check_status()
        prompt, gen = int(sum(prompt_lens)), len(prompt_lens) * new_tokens
        return {"seconds": dt, "steps": steps, "prompt_tokens": prompt, "generated_tokens": gen,
                "tokens_per_s": (prompt + gen) / dt, "generated_per_s": gen / dt, "launches": ops.launch_count() - l0}

    def profile(self, batch: int, prompt_tokens: int, hbm_gbs: float, tflops: float, repeats: int = 3) -> Dict:
        """Per-kernel times of a decode step at ``batch`` and of a one-prompt prefill, from CUDA events around
        every launch (eager, dependent launches off: kernels run one after another, so the sum is longer than a
        served step; the SHARES and the per-kernel rates are what this is for)."""
        runner = self.engine.runner
        graphs, runner.graphs_enabled = runner.graphs_enabled, False
        try:
            ids = self._open_with_context(batch)
            out = torch.empty(batch, dtype=torch.int32, device=self.engine.device)

            def one():
                logits = runner.step([StepEntry(r, [t], [0]) for r, t in zip(ids, self._tokens(batch))])
                ops.argmax(logits, out)
            for _ in range(3):
                one()
            with ops.KernelProfile() as prof:
                for _ in range(repeats):
                    one()
            decode_rows, decode_us = prof.table(hbm_gbs, tflops, repeats)
            for r in ids:
                runner.close_request(r)
            rid = self._next
            self._next += 1
            prefill_rows, prefill_us = [], 0.0
            for i in range(2):
                runner.open_request(rid + i)
                toks = self._tokens(prompt_tokens)
                if i == 0:
                    runner.step([StepEntry(rid + i, toks, [prompt_tokens - 1])])
                else:
                    with ops.KernelProfile() as prof:
                        runner.step([StepEntry(rid + i, toks, [prompt_tokens - 1])])
                    prefill_rows, prefill_us = prof.table(hbm_gbs, tflops, 1)
                runner.close_request(rid + i)
            self._next += 2
            runner.check_status()
        finally:
            runner.graphs_enabled = graphs
        return {"decode": {"batch": batch, "us": round(decode_us, 1), "kernels": decode_rows},
                "prefill": {"tokens": prompt_tokens, "us": round(prefill_us, 1), "kernels": prefill_rows}}

    def check_against_float32(self, prompt_tokens: int = 192, new_tokens: int = 8, seed: int = 3) -> Dict:
        """Outside any timed region: a short greedy continuation by this (bfloat16) engine, and the same
        tokens fed to a float32 engine of the same sizes and weights.  Every token this engine picked must be
        the float32 logits' first choice or lie within the tie margin of it (two logits closer than 4e-2 of
        the row's largest count as a tie, as in the tests); the largest relative difference between the two
        engines' logits rows is reported too."""
        eng = self.engine
        prompt = np.random.default_rng(seed).integers(0, self.config.vocab_size, size=prompt_tokens).tolist()
        out = eng.generate([prompt], SamplingParams(max_tokens=new_tokens, ignore_eos=True))[0]
        # this engine's own logits at the same places (teacher-forced, one step)
        seq = prompt + out.token_ids[:-1]
        places = list(range(prompt_tokens - 1, len(seq)))
        rid = self._next
        self._next += 1
        eng.runner.open_request(rid)
        mine = eng.runner.step([StepEntry(rid, seq, places)]).clone()
        eng.runner.close_request(rid)
        ref = Engine(config=self.config, dtype="float32", dummy_weight=True, seed=self.seed, kv_tokens=1024,
                     page_size=self.page_size, max_seq_len=1024, max_running_requests=2, max_prefill_tokens=512)
        ref.runner.open_request(0)
        theirs = ref.runner.step([StepEntry(0, seq, places)])
        ref.runner.check_status()
        big = theirs.abs().amax(dim=1)
        err = float(((mine - theirs).abs().amax(dim=1) / big).max())
        picked = torch.tensor(out.token_ids, device=theirs.device)
        gap = (theirs.max(dim=1).values - theirs.gather(1, picked[:, None])[:, 0]) / big
        first = int((theirs.argmax(dim=1) == picked).sum())
        ties = int(((gap > 0) & (gap <= 4e-2)).sum())
        del ref
        torch.cuda.empty_cache()
        return {"prompt_tokens": prompt_tokens, "new_tokens": new_tokens, "first_choice_of_float32": first, "ties": ties,
                "ok": first + ties == new_tokens, "max_logit_diff_rel": round(err, 5)}

    def prefill(self, tokens: int, reps: int, warmup: int) -> Dict:
        runner = self.engine.runner
        times = []
        for i in range(reps + warmup):
            rid = self._next
            self._next += 1
            runner.open_request(rid)
            toks = self._tokens(tokens)
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            logits = runner.step([StepEntry(rid, toks, [tokens - 1])])
            end.record()
            torch.cuda.synchronize()
            if i >= warmup:
                times.append(start.elapsed_time(end))
            runner.close_request(rid)
        runner.check_status()
        return {"ms": float(np.median(times))}
