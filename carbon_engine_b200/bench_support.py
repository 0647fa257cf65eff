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

    def decode(self, batch: int, steps: int, warmup: int) -> Dict:
        runner = self.engine.runner
        ids = self._open_with_context(batch)
        out = torch.empty(batch, dtype=torch.int32, device=self.engine.device)
        toks = [self._tokens(batch) for _ in range(steps + warmup)]

        def one(i):
            logits = runner.step([StepEntry(r, [toks[i][j]], [0]) for j, r in enumerate(ids)])
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
        # long enough that no request ends inside the timed region (requests whose prompts were done
        # first have decoded through the other prompts' steps already)
        sp = SamplingParams(max_tokens=warmup + steps + batch + 8, ignore_eos=True)
        for _ in range(batch):
            eng.add_request(self._tokens(self.context), sp)
        while eng.scheduler.stats()["prefill_tokens"] < batch * self.context:
            eng.step()
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        h2d = d2h = 0
        for _ in range(steps):
            eng.step()
            h2d += eng.runner.h2d_bytes_last
            d2h += eng.d2h_bytes_last
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        while eng.has_unfinished():
            eng.step()
        return {"ms_per_step": dt / steps * 1e3, "tokens_per_s": batch * steps / dt, "h2d_bytes": h2d // steps,
                "d2h_bytes": d2h // steps}

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
