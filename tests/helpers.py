"""Shared test material: the tiny configurations, model folders in temporary places, and a driver
for bin/trace_run."""
from __future__ import annotations

import json
import os
import struct
import subprocess
import sys
from typing import Dict, List, Optional

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Tiny configurations that differ in every size and option: layers, width, head counts and
# group size, head size (q width == hidden, != hidden), intermediate and vocabulary sizes that are no
# powers of two, rope theta, norm eps, tied or untied head, cache page size, and a window.
# A, B and C have head sizes 16, 32 and 48: in bfloat16 they run the cp.async decode kernel, the
# mma.sync flash kernel and the one-block tcgen05 product.  D (head size 128) and E (head size 64, one
# windowed layer) have the head geometry of the real checkpoints and, with prompts of several hundred
# tokens, run what serving runs: the TMA decode kernel with its merge inside a cluster, the tcgen05
# flash kernel over a cached prefix, the CTA-pair product (more than 256 tokens) and split-K.
TINY = {
    "A": dict(config=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
                          num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128,
                          vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                          max_position_embeddings=1024),
              page_size=16, seed=11),
    "B": dict(config=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
                          num_attention_heads=8, num_key_value_heads=2, head_dim=32, intermediate_size=224,
                          vocab_size=320, rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
                          max_position_embeddings=2048),
              page_size=8, seed=23),
    "C": dict(config=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=4, hidden_size=80,
                          num_attention_heads=6, num_key_value_heads=3, head_dim=48, intermediate_size=112,
                          vocab_size=301, rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
                          max_position_embeddings=768,
                          layer_types=["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
                          sliding_window=37),
              page_size=32, seed=5),
    "D": dict(config=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=512,
                          num_attention_heads=8, num_key_value_heads=2, head_dim=128, intermediate_size=1536,
                          vocab_size=2003, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False,
                          max_position_embeddings=4096),
              page_size=64, seed=41),
    "E": dict(config=dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=384,
                          num_attention_heads=6, num_key_value_heads=3, head_dim=64, intermediate_size=1000,
                          vocab_size=1511, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
                          max_position_embeddings=2048,
                          layer_types=["full_attention", "sliding_attention", "full_attention"], sliding_window=200,
                          rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 512}),
              # (yarn's attention factor of 1.14 on cos and sin already makes the scores 1.3 times larger)
              page_size=16, seed=77, sharpen=1.5),
}
#: the configurations with small head sizes (quick everywhere) and those with the product's head sizes
SMALL_HEADS = ("A", "B", "C")
REAL_HEADS = ("D", "E")

# tolerances, relative to the largest |logit| of the compared rows: the reference's own kernel
# self-test accepts 1e-4 in float32 and 3e-2 in 16-bit (src/device.rs:776-848)
TOL = {"float32": 1e-4, "bfloat16": 3e-2}
# Whole-model logits in bfloat16 pass through 4 roundings of the activations per layer, and the tiny
# models are 64 to 96 wide, so little averages out: measured on these models the typical row is off
# by 1.5e-2 and the worst of some 3000 rows by 3.4e-2.  A row may therefore be off by 5e-2, but the
# median row by no more than 2e-2.  (A cache fault moves a sharpened model's logits by far more, and
# the float32 replay of the same trace, at 1e-4, shares every line of the cache and step code.)
TOL_MODEL_BF16_ROW = 5e-2
TOL_MODEL_BF16_MEDIAN = 2e-2


def write_safetensors_plain(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    names = {torch.float32: "F32", torch.bfloat16: "BF16"}
    header, off, blobs = {}, 0, []
    for n, t in tensors.items():
        t = t.contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bfloat16 else t.view(torch.int16).numpy().tobytes()
        header[n] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hb = json.dumps(header).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(hb)) + hb + b"".join(blobs))


def make_model_dir(tmp_dir: str, name: str, sharpen: Optional[float] = None) -> str:
    """Write tiny model ``name`` with the engine's random-weights mode, then scale the q/k norm weights
    (scores grow by ``sharpen``) so that attention is peaked: a key that is missed or misplaced then moves
    the logits visibly.  Scores much larger than that lose absolute precision in bfloat16 keys and queries."""
    import carbon_engine_b200.models  # noqa: F401
    from carbon_engine_b200.config.qwen3 import Qwen3Config
    from carbon_engine_b200.weights.loader import write_random_model
    from plain_qwen3 import read_safetensors
    spec = TINY[name]
    if sharpen is None:
        sharpen = spec.get("sharpen", 2.0)
    out = os.path.join(tmp_dir, f"tiny_{name}")
    write_random_model(Qwen3Config.from_dict(dict(spec["config"])), out, seed=spec["seed"])
    if sharpen != 1.0:
        path = os.path.join(out, "model.safetensors")
        raw = read_raw_safetensors(path)
        for n in list(raw):
            if n.endswith("q_norm.weight") or n.endswith("k_norm.weight"):
                raw[n] = raw[n] * (sharpen ** 0.5)
        write_safetensors_plain(path, raw)
    return out


def read_raw_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """Tensors in their stored dtypes (bf16 stays bf16)."""
    with open(path, "rb") as fh:
        blob = fh.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode())
    out = {}
    for name, meta in header.items():
        lo, hi = meta["data_offsets"]
        buf = bytearray(blob[8 + n + lo:8 + n + hi])
        dt = {"F32": torch.float32, "BF16": torch.bfloat16}[meta["dtype"]]
        out[name] = torch.frombuffer(buf, dtype=dt).reshape(meta["shape"]).clone()
    return out


def random_tokens(rng: np.random.Generator, n: int, vocab: int) -> List[int]:
    return rng.integers(0, vocab, size=n).tolist()


class TraceRun:
    """Drives bin/trace_run as a user would: a subprocess fed one JSON line per step."""

    def __init__(self, model_dir: str, dtype: str, out_dir: str, max_tokens: int, page_size: int,
                 extra: Optional[List[str]] = None):
        self.out_dir = out_dir
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
               "--out", out_dir, "--max-tokens", str(max_tokens), "--page-size", str(page_size)] + (extra or [])
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)
        self.step_no = 0
        self.vocab = json.load(open(os.path.join(model_dir, "config.json")))["vocab_size"]

    def step(self, entries: List[dict], end: Optional[List[str]] = None) -> Optional[np.ndarray]:
        rec = {"step": self.step_no, "entries": entries, "end": end or []}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if line.strip() != f"done {self.step_no}":
            raise RuntimeError(f"trace_run answered {line!r} (exit {self.proc.poll()})")
        path = os.path.join(self.out_dir, f"{self.step_no}.f32")
        self.step_no += 1
        wanted = sum(len(e.get("want", [])) for e in entries)
        if wanted == 0:
            assert not os.path.exists(path)
            return None
        data = np.fromfile(path, dtype="<f4")
        return data.reshape(wanted, self.vocab)

    def close(self) -> int:
        self.proc.stdin.close()
        return self.proc.wait(timeout=120)
