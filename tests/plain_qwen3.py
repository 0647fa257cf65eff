"""A plain, slow implementation of the Qwen3 dense decoder for tests.

It restates the reference's FORMULAS (each function cites the file and lines it restates).  The
reference's model code is Rust on the candle library and can be neither imported nor compiled on
the machines these tests run on, so there is no golden output of its whole model; but its CUDA
kernel sources for attention, for the sampler's random numbers and for a key norm + rotation do
build for the CPU, and tests/test_reference_anchor.py holds ``causal_attention``, ``rms_norm``,
``apply_rope`` and the sampler's uniforms to their output (tests/golden/).  SwiGLU, the order of a
layer's operations and the head rest on the formulas alone.  This file shares no code
with the engine: it reads config.json and model.safetensors itself, processes whole sequences with
no cache, and has one function per part.  Everything is float64 by default, so that both the
float32 and the bfloat16 engine can be compared with the same numbers.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch


# ---- reading a model folder (no engine code) -----------------------------------------------------
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """8-byte little-endian header length, JSON header, raw data (src/weights.rs:389-423)."""
    with open(path, "rb") as fh:
        blob = fh.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = np.frombuffer(blob, dtype=np.uint8, count=hi - lo, offset=8 + n + lo)
        if meta["dtype"] == "F32":
            t = torch.from_numpy(raw.copy().view(np.float32).copy())
        elif meta["dtype"] == "BF16":
            u16 = raw.copy().view(np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(u16.view(np.float32).copy())
        elif meta["dtype"] == "F16":
            t = torch.from_numpy(raw.copy().view(np.float16).astype(np.float32))
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = t.reshape(meta["shape"])
    return out


def read_model(model_dir: str, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as fh:
        cfg = json.load(fh)
    weights = {k: v.to(dtype) for k, v in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, weights


# ---- one function per part ----------------------------------------------------------------------
def embedding(table: torch.Tensor, tokens: List[int]) -> torch.Tensor:
    """x0[t] = E[token[t]], no scaling (src/model/mod.rs:781-784)."""
    return table[torch.tensor(tokens, dtype=torch.long, device=table.device)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w over the last dimension, the weight as stored
    (src/model/layers.rs:117-146; the same formula spelled out at src/model/hyper.rs:51)."""
    return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def scaled_inv_freq(rotary_dim: int, theta: float, scaling: Optional[dict], max_position_embeddings: int = 4096):
    """Rotary frequencies with the config.json's ``rope_scaling`` applied (src/model/layers.rs:169-223, keys
    and defaults of src/config.rs:483-519); returns (inv_freq float64 [rd/2], cos/sin multiplier)."""
    i = np.arange(0, rotary_dim // 2, dtype=np.float64)
    inv = 1.0 / theta ** (2.0 * i / rotary_dim)
    kind = (scaling or {}).get("rope_type", (scaling or {}).get("type", "default"))
    if not scaling or kind == "default":
        return torch.from_numpy(inv), 1.0
    factor = float(scaling.get("factor", 1.0))
    if kind == "linear":
        return torch.from_numpy(inv / factor), 1.0
    if kind == "llama3":
        lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wl = 2.0 * np.pi / inv
        smooth = (old / wl - lo) / (hi - lo)
        blended = (1.0 - smooth) * inv / factor + smooth * inv
        out = np.where(wl > old / lo, inv / factor, np.where(wl >= old / hi, blended, inv))
        return torch.from_numpy(out), 1.0
    if kind == "yarn":
        old = float(scaling.get("original_max_position_embeddings", max_position_embeddings))
        fast, slow = float(scaling.get("beta_fast", 32.0)), float(scaling.get("beta_slow", 1.0))
        corr = lambda rot: rotary_dim * math.log(old / (rot * 2.0 * math.pi)) / (2.0 * math.log(theta))
        low, high = max(math.floor(corr(fast)), 0.0), min(math.ceil(corr(slow)), rotary_dim - 1.0)
        if high == low:
            high += 0.001
        ramp = np.clip((i - low) / (high - low), 0.0, 1.0)
        out = inv / factor * ramp + inv * (1.0 - ramp)
        mscale = lambda m: 1.0 if factor <= 1.0 else 0.1 * m * math.log(factor) + 1.0      # src/config.rs:108-114
        if "attention_factor" in scaling:
            att = float(scaling["attention_factor"])
        elif "mscale" in scaling and "mscale_all_dim" in scaling:
            att = mscale(float(scaling["mscale"])) / mscale(float(scaling["mscale_all_dim"]))
        else:
            att = mscale(1.0)
        return torch.from_numpy(out), att
    raise ValueError(kind)


def rope_tables(positions: torch.Tensor, rotary_dim: int, theta: float, scaling: Optional[dict] = None,
                max_position_embeddings: int = 4096):
    """inv_freq[i] = theta^(-2i/rd), rescaled if the config says so; angle = pos * inv_freq[i]; cos and sin
    times the scheme's attention factor (src/model/layers.rs:169-173, 237-251)."""
    inv_freq, att = scaled_inv_freq(rotary_dim, theta, scaling, max_position_embeddings)
    ang = positions.to(torch.float64)[:, None] * inv_freq.to(positions.device)[None, :]
    return ang.cos() * att, ang.sin() * att


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half pairing: y[i] = x[i] cos[i] - x[i+h] sin[i]; y[i+h] = x[i+h] cos[i] + x[i] sin[i]
    (src/model/layers.rs:159; src/kernels/qsa.cu:107-116).  x is [T, heads, d]."""
    h = cos.shape[-1]
    c, s = cos[:, None, :].to(x.dtype), sin[:, None, :].to(x.dtype)
    x1, x2, rest = x[..., :h], x[..., h:2 * h], x[..., 2 * h:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: int = 0) -> torch.Tensor:
    """Grouped-query causal attention of one whole sequence.  q [T, nh, d], k and v [T, nkv, d].
    Query head h reads KV head h // (nh / nkv) (src/model/attention.rs:1035); scores are scaled by
    ``scale`` and a query at position i sees keys 0..i (src/model/attention.rs:1038-1066); with a
    window it sees the last ``window`` of them."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    g = nh // nkv
    out = torch.empty_like(q)
    idx = torch.arange(T, device=q.device)
    allowed = idx[None, :] <= idx[:, None]
    if window > 0:
        allowed &= idx[None, :] > idx[:, None] - window
    for h in range(nh):
        kh = h // g
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, kh, :]
    return out


def attention_block(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict, positions: torch.Tensor,
                    window: int = 0) -> torch.Tensor:
    """q/k/v products, per-head q/k RMSNorm before the rotation, rotation, attention, output product
    (src/model/attention.rs:868-914)."""
    nh, nkv = cfg["num_attention_heads"], cfg.get("num_key_value_heads", cfg["num_attention_heads"])
    d = cfg.get("head_dim", cfg["hidden_size"] // nh)
    eps = cfg.get("rms_norm_eps", 1e-6)
    T = h.shape[0]
    q = (h @ w[f"{prefix}.q_proj.weight"].T).view(T, nh, d)
    k = (h @ w[f"{prefix}.k_proj.weight"].T).view(T, nkv, d)
    v = (h @ w[f"{prefix}.v_proj.weight"].T).view(T, nkv, d)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], eps)
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], eps)
    cos, sin = rope_tables(positions, d, float(cfg.get("rope_theta", 10000.0)),
                           cfg.get("rope_scaling") or cfg.get("rope_parameters"), cfg.get("max_position_embeddings", 4096))
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    a = causal_attention(q, k, v, 1.0 / math.sqrt(d), window)
    return a.reshape(T, nh * d) @ w[f"{prefix}.o_proj.weight"].T


def swiglu_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(silu(gate(h)) * up(h)), silu(z) = z * sigmoid(z) (src/model/layers.rs:568, 625-648)."""
    g = h @ w[f"{prefix}.gate_proj.weight"].T
    u = h @ w[f"{prefix}.up_proj.weight"].T
    return (g * torch.sigmoid(g) * u) @ w[f"{prefix}.down_proj.weight"].T


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], layer: int, cfg: dict, positions: torch.Tensor) -> torch.Tensor:
    """x += attn(norm(x)); x += mlp(norm(x)) (src/model/mod.rs:645-650)."""
    p = f"model.layers.{layer}"
    eps = cfg.get("rms_norm_eps", 1e-6)
    types = cfg.get("layer_types")
    window = cfg.get("sliding_window") or 0 if types and types[layer] == "sliding_attention" else 0
    x = x + attention_block(rms_norm(x, w[f"{p}.input_layernorm.weight"], eps), w, f"{p}.self_attn", cfg, positions, window)
    x = x + swiglu_mlp(rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")
    return x


def lm_head(x: torch.Tensor, w: Dict[str, torch.Tensor], cfg: dict) -> torch.Tensor:
    """Final RMSNorm, then the head; tied embeddings share the embedding tensor
    (src/model/mod.rs:723-761, 793-802)."""
    z = rms_norm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return z @ head.T


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int]) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (computed where the weights live: the tests of real layer
    sizes keep them on the GPU, still in float64 and still with these functions only)."""
    x = embedding(w["model.embed_tokens.weight"], tokens)
    positions = torch.arange(len(tokens), device=x.device)
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, w, layer, cfg, positions)
    return lm_head(x, w, cfg)


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


# ---- sampling (src/sampling.rs:137-181) ---------------------------------------------------------
def sample_kept_set(logits: np.ndarray, temperature: float, top_k: int, top_p: float, min_p: float):
    """Indices the reference's host sampler keeps, and their renormalised probabilities."""
    z = logits.astype(np.float64) / max(temperature, 1e-5)
    order = np.argsort(-z, kind="stable")
    if 0 < top_k < len(z):
        order = order[:top_k]
    p = np.exp(z[order] - z[order[0]])
    p /= p.sum()
    keep = len(p)
    if top_p < 1.0:
        keep = int(np.searchsorted(np.cumsum(p), top_p, side="left")) + 1
        keep = min(keep, len(p))
    if min_p > 0.0:
        keep = min(keep, max(1, int((p >= p[0] * min_p).sum())))
    kept = order[:keep]
    return kept, p[:keep] / p[:keep].sum()
