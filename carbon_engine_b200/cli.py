"""Command line of the engine, in the manner of the reference's ``carbon`` binary.

Sub-commands and option names follow the reference where it has them (src/main.rs:103-217 engine
flags, :381-414 ``generate``, :634-661 ``tiny-model``, :51-61 ``devices --selftest``):

    python -m carbon_engine_b200 generate --model DIR --prompt-ids 1,2,3 --max-tokens 16 --print-ids
    python -m carbon_engine_b200 generate --model DIR --prompt-ids 1,2,3 --prompt-ids 7,8 --temperature 0.8 --seed 5
    python -m carbon_engine_b200 tiny-model --out DIR --layers 2 --hidden 64 --seed 1
    python -m carbon_engine_b200 devices --selftest

Prompts are token ids (``--prompt-ids``, as in src/main.rs:385-389); text needs a tokenizer, which is
outside an engine that goes from a request's tokens to its next token.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List, Optional


def _engine_flags(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", "--model-path", required=True, help="model folder: config.json + safetensors")
    p.add_argument("--hf-overrides", default=None, help="JSON merged into config.json before loading")
    p.add_argument("--dummy-weight", action="store_true", help="random weights shaped from config.json")
    p.add_argument("--devices", default="cuda:0", help="one CUDA device (this engine runs on a single GPU)")
    p.add_argument("--dtype", default="auto", help="auto | bf16 | f32")
    p.add_argument("--kv-tokens", "--num-tokens", type=int, default=None, help="KV cache capacity in tokens")
    p.add_argument("--memory-ratio", type=float, default=0.9, help="fraction of free device memory for the KV cache")
    p.add_argument("--max-seq-len", type=int, default=0, help="max context (0: from the checkpoint, capped at 32768)")
    p.add_argument("--max-running-requests", type=int, default=16)
    p.add_argument("--max-prefill-tokens", "--max-prefill-length", type=int, default=4096,
                   help="token budget of one step (portions of prompts fill what decoding leaves)")
    p.add_argument("--cuda-graphs", action="store_true", help="replay decode steps as CUDA graphs")
    p.add_argument("--page-size", type=int, default=64, help="tokens per KV page")
    p.add_argument("--seed-weights", type=int, default=0, help="seed of --dummy-weight")


def _make_engine(a):
    from .engine.engine import Engine
    overrides = json.loads(a.hf_overrides) if a.hf_overrides else None
    dev = a.devices.split(",")[0].strip() or "cuda:0"
    if dev == "cpu":
        raise SystemExit("this engine has no CPU path: --devices must name a CUDA device")
    return Engine(a.model, dtype=a.dtype, device=dev, hf_overrides=overrides, dummy_weight=a.dummy_weight,
                  seed=a.seed_weights, kv_tokens=a.kv_tokens, memory_ratio=a.memory_ratio, page_size=a.page_size,
                  max_seq_len=a.max_seq_len, max_running_requests=a.max_running_requests,
                  max_prefill_tokens=a.max_prefill_tokens, cuda_graphs=a.cuda_graphs)


def _parse_ids(text: str) -> List[int]:
    try:
        return [int(x.strip()) for x in text.split(",") if x.strip() != ""]
    except ValueError:
        raise SystemExit("bad --prompt-ids: comma separated integers expected")


def cmd_generate(a) -> int:
    """Submit the prompt (or prompts) to an engine running on its own thread and print tokens as their
    events arrive, as the reference's ``generate`` consumes its event stream (src/main.rs:1020-1066)."""
    from .engine.handle import Done, EngineHandle, Error, Token
    from .sampling.params import SamplingParams
    if not a.prompt_ids:
        raise SystemExit("--prompt-ids is required (text prompts need a tokenizer, which this engine does not carry)")
    prompts = [_parse_ids(p) for p in a.prompt_ids]
    handle = EngineHandle(_make_engine(a))
    failed = False
    try:
        t0 = time.perf_counter()
        streams = []
        for i, ids in enumerate(prompts):
            # a seeded batch gives every prompt a seed of its own, so that equal prompts differ
            seed = None if a.seed is None else a.seed + i
            sp = SamplingParams(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, min_p=a.min_p,
                                max_tokens=a.max_tokens, seed=seed, ignore_eos=a.ignore_eos)
            streams.append(handle.submit(ids, sp))
        for i, (ids, stream) in enumerate(zip(prompts, streams)):
            first: Optional[float] = None
            out_ids: List[int] = []
            tag = f"[{i}] " if len(prompts) > 1 else ""
            for ev in stream:
                if isinstance(ev, Token):
                    if first is None:
                        first = time.perf_counter() - t0
                    out_ids.append(ev.token_id)
                    if len(prompts) == 1:            # one prompt: its tokens as they come
                        sys.stdout.write(f"{ev.token_id} ")
                        sys.stdout.flush()
                elif isinstance(ev, Error):
                    print(f"\n{tag}generation failed: {ev.message}", file=sys.stderr)
                    failed = True
                elif isinstance(ev, Done):
                    total = time.perf_counter() - t0
                    if len(prompts) > 1:
                        print(f"{tag}" + " ".join(str(t) for t in out_ids))
                    if a.print_ids:
                        print(f"\n{tag}output_ids: {out_ids}", file=sys.stderr)
                    ttft = first if first is not None else total
                    n = ev.usage["completion_tokens"]
                    tps = max(n - 1, 0) / max(total - ttft, 1e-9)
                    # the reference's summary line (src/main.rs:1044-1050)
                    print(f"\n{tag}[{ev.reason.capitalize()}] prompt {ev.usage['prompt_tokens']} tok, output {n} tok, "
                          f"ttft {ttft:.3f}s, decode {tps:.1f} tok/s", file=sys.stderr)
    finally:
        handle.shutdown()
    return 1 if failed else 0


def cmd_tiny_model(a) -> int:
    import torch
    from . import models  # noqa: F401
    from .config.qwen3 import Qwen3Config
    from .weights.loader import write_random_model
    if a.arch != "qwen3":
        raise SystemExit(f"--arch {a.arch}: only qwen3 is built")
    heads = a.heads or 4
    head_dim = a.head_dim or 16
    cfg = Qwen3Config.from_dict(dict(
        architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=a.layers, hidden_size=a.hidden,
        num_attention_heads=heads, num_key_value_heads=a.kv_heads or max(1, heads // 2), head_dim=head_dim,
        intermediate_size=a.intermediate or 2 * a.hidden, vocab_size=a.vocab, rope_theta=a.rope_theta,
        rms_norm_eps=a.rms_norm_eps, tie_word_embeddings=a.tie_word_embeddings, max_position_embeddings=a.max_positions))
    store = {"f32": torch.float32, "bf16": torch.bfloat16}.get(a.dtype)
    if store is None:
        raise SystemExit("--dtype must be f32 or bf16")
    out = write_random_model(cfg, a.out, seed=a.seed, store_dtype=store)
    print(f"wrote {out}")
    return 0


def cmd_devices(a) -> int:
    import torch
    if not torch.cuda.is_available():
        print("no CUDA device")
        return 1
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        print(f"cuda:{i} {p.name} sm_{p.major}{p.minor} {p.total_memory >> 20} MiB {p.multi_processor_count} SMs")
    if a.selftest:
        from .selftest import run
        return run()
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="carbon_engine_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate tokens for a prompt (or, --prompt-ids given several times, a batch)")
    _engine_flags(g)
    g.add_argument("--prompt-ids", action="append", default=None,
                   help="comma separated prompt token ids; may be given more than once: the prompts run as one batch")
    g.add_argument("--print-ids", action="store_true", help="print the generated ids once more at the end")
    g.add_argument("--max-tokens", type=int, default=128)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=-1)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--ignore-eos", action="store_true")
    g.set_defaults(fn=cmd_generate)

    t = sub.add_parser("tiny-model", help="write a small random model folder")
    t.add_argument("--out", required=True)
    t.add_argument("--arch", default="qwen3")
    t.add_argument("--layers", type=int, default=4)
    t.add_argument("--hidden", type=int, default=64)
    t.add_argument("--heads", type=int, default=None)
    t.add_argument("--kv-heads", type=int, default=None)
    t.add_argument("--head-dim", type=int, default=None)
    t.add_argument("--intermediate", type=int, default=None)
    t.add_argument("--vocab", type=int, default=263)
    t.add_argument("--rope-theta", type=float, default=10000.0)
    t.add_argument("--rms-norm-eps", type=float, default=1e-6)
    t.add_argument("--tie-word-embeddings", action="store_true")
    t.add_argument("--max-positions", type=int, default=4096)
    t.add_argument("--seed", type=int, default=0)
    t.add_argument("--dtype", default="bf16", help="stored dtype of the matrices: f32 | bf16")
    t.set_defaults(fn=cmd_tiny_model)

    d = sub.add_parser("devices", help="list devices; --selftest checks every kernel against a plain computation")
    d.add_argument("--selftest", action="store_true")
    d.set_defaults(fn=cmd_devices)

    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
