"""Seeded random weights, the same on the CPU and on the GPU.

Every element is a function of (seed, tensor name, element index) alone: a 64-bit hash gives two
uniform numbers, Box-Muller (in float64) turns them into one normal.  So any tensor can be made
anywhere, lazily, without the whole model ever existing on the host; the reference's
``--dummy-weight`` source has the same property (src/dummy.rs:25-90: FNV-1a of the name xor the
seed drives the generator).  Distributions: linear and embedding weights N(0, 0.02), norm weights
1 + N(0, 0.1).
"""
from __future__ import annotations

import math
from typing import Dict, Sequence

import torch

from ..parts.base import INIT_KINDS, TensorSpec

_M64 = (1 << 64) - 1


def _fnv1a(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & _M64
    return h


def _signed(v: int) -> int:
    v &= _M64
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(x: torch.Tensor, n: int) -> torch.Tensor:
    return (x >> n) & ((1 << (64 - n)) - 1)


def _mix(x: torch.Tensor) -> torch.Tensor:
    """splitmix64 finaliser on int64 tensors (arithmetic wraps modulo 2^64)."""
    x = x + _signed(0x9E3779B97F4A7C15)
    x = (x ^ _lsr(x, 30)) * _signed(0xBF58476D1CE4E5B9)
    x = (x ^ _lsr(x, 27)) * _signed(0x94D049BB133111EB)
    return x ^ _lsr(x, 31)


def standard_normal(name: str, numel: int, seed: int, device, start: int = 0) -> torch.Tensor:
    """float64 [numel]: elements start .. start+numel of the tensor's stream."""
    key = _signed(_fnv1a(name) ^ ((seed * 0x9E3779B97F4A7C15) & _M64))
    idx = torch.arange(start, start + numel, dtype=torch.int64, device=device)
    h1 = _mix(idx * 2 + key)
    h2 = _mix(idx * 2 + 1 + key)
    u1 = (_lsr(h1, 11).to(torch.float64) + 0.5) * (1.0 / (1 << 53))
    u2 = (_lsr(h2, 11).to(torch.float64) + 0.5) * (1.0 / (1 << 53))
    return torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u2)


def random_tensor(spec: TensorSpec, seed: int, device, dtype: torch.dtype, chunk: int = 1 << 24) -> torch.Tensor:
    numel = 1
    for s in spec.shape:
        numel *= s
    out = torch.empty(numel, dtype=dtype, device=device)
    try:
        mean, std, _ = INIT_KINDS[spec.init]
    except KeyError:
        raise ValueError(f"{spec.name}: unknown init kind '{spec.init}' (known: {', '.join(sorted(INIT_KINDS))}; "
                         f"parts.base.register_init_kind adds one)") from None
    for lo in range(0, numel, chunk):
        n = min(chunk, numel - lo)
        z = standard_normal(spec.name, n, seed, device, lo)
        out[lo:lo + n] = (mean + std * z).to(dtype)
    return out.view(spec.shape)


class RandomWeights:
    """A name -> tensor function over a model's declared tensors."""

    def __init__(self, specs: Sequence[TensorSpec], seed: int, device, matrix_dtype: torch.dtype = torch.bfloat16):
        self.specs: Dict[str, TensorSpec] = {s.name: s for s in specs}
        self.seed, self.device, self.matrix_dtype = int(seed), device, matrix_dtype

    def __call__(self, name: str) -> torch.Tensor:
        spec = self.specs[name]
        # norm weights are small and are kept in 32-bit; matrices are rounded to the stored dtype
        dt = torch.float32 if INIT_KINDS.get(spec.init, (0, 0, False))[2] else self.matrix_dtype
        return random_tensor(spec, self.seed, self.device, dt)
