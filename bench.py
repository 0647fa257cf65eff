#!/usr/bin/env python3
"""Benchmark of the engine's decode step (and a 2,048-token prefill) at Qwen3-8B layer sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at the given batch (default 8), each
sequence holding ``context_len`` tokens of context, timed on the device with CUDA events around
exactly K decode steps after W warm-up steps; a step includes the greedy pick of every sequence's
next token on the device.  ``e2e`` is the same measured through the Python entry point (the
scheduler, the step function and the sampler): every step copies its inputs from pinned host memory
to the device and reads the sampled tokens back to the host.  ``prefill`` is one 2,048-token prompt
in one step; ``roofline`` compares the bytes a decode step has to read (every weight once, and the
cache of the live requests) with the measured copy bandwidth; ``points`` holds decode at batch 1 and
64 and the main batch without the pick; ``check`` (outside every timed region) says whether a short greedy
continuation by the timed engine is what a float32 engine of the same weights picks, ties apart.
``--profile`` prints a per-kernel table instead.
Weights are random (seeded), token ids are uniform-random (seeded): no dataset is involved.
The weights alone (over 15 GB) exceed the L2 cache many times over, so no flush is needed between
steps.  Runs on one GPU only.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SIZES_8B = dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                intermediate_size=12288, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                tie_word_embeddings=False, max_position_embeddings=40960)
SIZES_14B = dict(SIZES_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)
SIZES_32B = dict(SIZES_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as fh:
                p = json.load(fh)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def mark(self):
        return time.time()

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, t0, t1):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.samples:
            if not (t0 - 0.05 <= t <= t1 + 0.15):
                continue
            f = [x.strip() for x in line.split(",")]
            try:
                mhz.append(int(f[0])); mx = max(mx, int(f[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, f[2:]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def decode_bytes(cfg, layers, batch, ctx, el=2):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q, kv = cfg["num_attention_heads"] * cfg["head_dim"], cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * H + H * q + 3 * H * I + 2 * H + 2 * cfg["head_dim"]
    weights = layers * per_layer + V * H + H + batch * H            # head, final norm, the embedding rows that are read
    cache = layers * 2 * kv * ctx * batch
    return (weights + cache) * el


def prefill_flops(cfg, layers, T):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, d = cfg["num_attention_heads"], cfg["head_dim"]
    q, kv = nh * d, cfg["num_key_value_heads"] * d
    linear = 2 * T * ((q + 2 * kv) * H + H * q + 3 * H * I)
    attn = 4 * d * nh * T * (T + 1) // 2
    return layers * (linear + attn) + 2 * V * H


def serve_workload(args, BenchHarness) -> int:
    """The two serving workloads of the larger model sizes, through the engine's public entry point."""
    import numpy as np
    if args.workload == "mixed-14b":
        sizes, name, n_req, new_tokens, budget = SIZES_14B, "Qwen3-14B sizes", 32, 128, 2048
        lens = np.random.default_rng(1).integers(128, 3073, size=n_req).tolist()
    else:
        sizes, name, n_req, new_tokens, budget = SIZES_32B, "Qwen3-32B sizes", 16, 256, 4096
        lens = [1024] * n_req
    layers = args.layers if args.layers != SIZES_8B["num_hidden_layers"] else sizes["num_hidden_layers"]
    h = BenchHarness(dict(sizes, num_hidden_layers=layers), max_batch=n_req, context=max(lens), new_tokens=new_tokens,
                     graphs=not args.no_graphs, step_tokens=budget)
    h.serve(lens, new_tokens)                      # once untimed: kernels, graphs and allocations are warm afterwards
    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.3)
    t0 = clocks.mark()
    r = h.serve(lens, new_tokens)
    t1 = clocks.mark()
    clocks.stop()
    print(json.dumps({
        "metric": f"tokens/s (prompt + generated) of the {args.workload} workload ({name}, bf16)", "value": round(r["tokens_per_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "generated_tokens_per_s": round(r["generated_per_s"], 1), "seconds": round(r["seconds"], 3),
        "steps": r["steps"], "ms_per_step": round(r["seconds"] / r["steps"] * 1e3, 3), "prompt_tokens": r["prompt_tokens"],
        "generated_tokens": r["generated_tokens"], "higher_is_better": True, "dtype": "bf16", "impl": "ours",
        "data": "synthetic: seeded random weights, seeded uniform-random token ids",
        "config": {"model": name, "layers": layers, "layers_of_model": sizes["num_hidden_layers"], "hidden_size": sizes["hidden_size"],
                   "heads": sizes["num_attention_heads"], "kv_heads": sizes["num_key_value_heads"], "head_dim": sizes["head_dim"],
                   "intermediate_size": sizes["intermediate_size"], "vocab_size": sizes["vocab_size"], "requests": n_req,
                   "prompt_tokens_min": int(min(lens)), "prompt_tokens_max": int(max(lens)), "new_tokens": new_tokens,
                   "step_token_budget": budget, "page_size": h.page_size, "cuda_graphs": h.graphs},
        "clocks": clocks.summary(t0, t1), "gpu_launches": r["launches"]}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048, help="tokens of context each sequence holds when decoding starts")
    ap.add_argument("--layers", type=int, default=SIZES_8B["num_hidden_layers"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--prefill-only", action="store_true",
                    help="run only the prefill of one prompt (for profiling, and for other prompt lengths) and print its time")
    ap.add_argument("--prefill-tokens", type=int, default=2048, help="with --prefill-only: tokens of the prompt (one step)")
    ap.add_argument("--profile", action="store_true",
                    help="instead of the contract's line: time every kernel of a decode step and of a 2,048-token prefill "
                         "with CUDA events (eager, kernels one after another) and print a table per kernel: launches, "
                         "microseconds, share, GB/s, TFLOP/s and the fraction of the measured peak")
    ap.add_argument("--between-steps", action="store_true",
                    help="instead of the contract's line: the device activities between two decode steps through the entry "
                         "point (pick, read-back copies, upload, token copy) and the steps' period")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of a short greedy continuation with float32")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed-14b", "batch16-32b"],
                    help="decode: the contract's line (default).  mixed-14b: 32 requests with prompts of 128 to 3,072 tokens at "
                         "Qwen3-14B sizes, prompts cut under a 2,048-token step budget beside the decoding requests, 128 new "
                         "tokens each.  batch16-32b: 16 prompts of 1,024 tokens at Qwen3-32B sizes, 256 new tokens each.  Both "
                         "run through the scheduler and print a line of their own")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust crate on the candle library: no "
                          "Python package to install offline, and neither cargo/rustc nor its crates are on this machine"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU only; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from carbon_engine_b200.bench_support import BenchHarness
    pk = peaks()
    if args.workload != "decode":
        return serve_workload(args, BenchHarness)
    cfg = dict(SIZES_8B, num_hidden_layers=args.layers)
    if args.prefill_only:
        T = args.prefill_tokens
        h = BenchHarness(cfg, max_batch=2, context=max(args.context, T), new_tokens=256, graphs=not args.no_graphs,
                         step_tokens=max(4096, T))
        pf = h.prefill(T, 3, 2)
        flops = prefill_flops(cfg, args.layers, T)
        print(json.dumps({"prefill_ms": round(pf["ms"], 3), "tokens": T, "layers": args.layers,
                          "tokens_per_s": round(T / (pf["ms"] / 1e3), 1), "tflops": round(flops / (pf["ms"] / 1e3) / 1e12, 1),
                          "frac": round(flops / (pf["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4), "peaks": pk["source"]}))
        return 0
    h = BenchHarness(cfg, max_batch=max(64 if not args.no_points else args.batch, args.batch),
                     context=args.context,
                     new_tokens=max(256, args.steps + max(args.warmup, 32) + 8 + args.batch * ((args.context + 4095) // 4096 + 1)),
                     graphs=not args.no_graphs)
    if args.between_steps:
        print(json.dumps({"between_steps": h.between_steps(args.batch), "batch": args.batch, "context": args.context,
                          "layers": args.layers}, indent=1))
        return 0
    if args.profile:
        prof = h.profile(args.batch, 2048, pk["hbm_gbs"], pk["bf16_tflops"])
        for part in ("decode", "prefill"):
            p = prof[part]
            what = f"decode step, batch {p['batch']}, {args.context}-token contexts" if part == "decode" else f"prefill of {p['tokens']} tokens"
            print(f"\n{what}, {args.layers} layers: {p['us']:.0f} us with kernels one after another (peaks {pk['source']}: "
                  f"{pk['hbm_gbs']:.0f} GB/s, {pk['bf16_tflops']:.0f} TFLOP/s)", file=sys.stderr)
            print(f"{'kernel':58s} {'launches':>8s} {'us':>10s} {'share':>6s} {'GB/s':>8s} {'TFLOP/s':>8s} {'of peak':>8s}", file=sys.stderr)
            for r in p["kernels"]:
                frac = "" if r["frac_of_peak"] is None else f"{r['frac_of_peak']:.2f}"
                print(f"{r['kernel'][:58]:58s} {r['launches']:8d} {r['us']:10.1f} {r['share']:6.3f} {r['gb_s']:8.0f} {r['tflop_s']:8.0f} {frac:>8s}",
                      file=sys.stderr)
        print(json.dumps({"profile": prof, "layers": args.layers, "peaks": pk["source"]}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.3)

    t0 = clocks.mark()
    main_run = h.decode(args.batch, args.steps, args.warmup)
    t1 = clocks.mark()
    e2e = h.decode_e2e(args.batch, args.steps, args.warmup)
    t2 = clocks.mark()
    points, prefill = {}, None
    if not args.no_points:
        pf = h.prefill(2048, 3, 3)
        flops = prefill_flops(cfg, args.layers, 2048)
        prefill = {"value": round(2048 / (pf["ms"] / 1e3), 1), "tokens": 2048, "ms": round(pf["ms"], 3),
                   "frac": round(flops / (pf["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        for b in (1, 64):
            r = h.decode(b, min(args.steps, 32), 3)
            points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
        # the same step without the greedy pick at its end (the logits are the step's result)
        points[f"decode_b{args.batch}_without_pick"] = round(h.decode(args.batch, min(args.steps, 32), 3, pick=False)["tokens_per_s"], 1)
    clocks.stop()
    check = None if args.no_check else h.check_against_float32()

    ms = main_run["ms_per_step"]
    need = decode_bytes(cfg, args.layers, args.batch, args.context + args.warmup + args.steps // 2)
    achieved = need / (ms / 1e3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-8B sizes, bf16, {args.context}-token contexts)", "value": round(main_run["tokens_per_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights, seeded uniform-random token ids", "impl": "ours",
        "config": {"model": "Qwen3-8B sizes", "layers": args.layers, "layers_of_model": SIZES_8B["num_hidden_layers"],
                   "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate_size": cfg["intermediate_size"], "vocab_size": cfg["vocab_size"],
                   "global_batch": args.batch, "seq_len": args.context, "max_seq_len": h.max_seq_len, "new_tokens": args.steps,
                   "page_size": h.page_size, "parallelism": "single GPU", "cuda_graphs": h.graphs,
                   "l2": "inputs larger than L2 (weights over 15 GB per step)", "peaks": pk["source"]},
        "clocks": clocks.summary(t0, t1),
        "e2e": {"value": round(e2e["tokens_per_s"], 1), "unit": "tokens/s", "ms_per_step": round(e2e["ms_per_step"], 4),
                "h2d_bytes_per_step": e2e["h2d_bytes"], "d2h_bytes_per_step": e2e["d2h_bytes"],
                # timed steps that were launched before the step before them had been read back
                "steps_launched_ahead": e2e["launched_ahead"],
                # over the whole e2e run: its prompts' prefill (which may meet the power cap), warm-up and timed steps
                "clocks": clocks.summary(t1, t2)},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if prefill is not None:
        out["prefill"] = prefill
        out["points"] = points
    if check is not None:
        out["check"] = check
    print(json.dumps(out))
    return 0 if check is None or check["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
