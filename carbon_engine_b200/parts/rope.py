"""Rotary position embedding tables.

inv_freq[i] = theta^(-2i/rd), optionally rescaled ("linear", "llama3", "yarn": src/model/layers.rs:169-234),
angle = position * inv_freq[i]; cos and sin are computed in float64 and kept in float32 for both
precisions (src/model/layers.rs:237-251).  The rotation
itself (rotate-half pairing, src/model/layers.rs:159) happens inside the fused q/k kernel, which
reads rows of these tables at each token's position.  Another position encoding is another class
with the same two tables (or with none: ``cos is None`` turns the rotation off).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch


@dataclass(frozen=True)
class RopeScaling:
    """How the rotary frequencies are stretched for contexts longer than the model was trained on
    (src/config.rs:86-106, 483-529).  ``kind``: "linear", "llama3" or "yarn"."""
    kind: str
    factor: float = 1.0
    low_freq_factor: float = 1.0            # llama3
    high_freq_factor: float = 4.0           # llama3
    original_max_position: int = 8192       # llama3, yarn
    beta_fast: float = 32.0                 # yarn
    beta_slow: float = 1.0                  # yarn
    attention_factor: float = 1.0           # yarn: multiplies cos and sin


def yarn_mscale(scale: float, mscale: float) -> float:
    """YaRN's attention temperature (src/config.rs:108-114)."""
    return 1.0 if scale <= 1.0 else 0.1 * mscale * math.log(scale) + 1.0


def rope_inv_freq(rotary_dim: int, theta: float, scaling: Optional[RopeScaling] = None) -> List[float]:
    """The rotary_dim / 2 inverse frequencies in float64 (src/model/layers.rs:169-223): theta^(-2i/rd),
    then divided by ``factor`` ("linear"), divided for long wavelengths only with a smooth band between
    ("llama3"), or blended between divided and untouched along a ramp over the dimensions ("yarn")."""
    inv = [1.0 / theta ** (2.0 * i / rotary_dim) for i in range(rotary_dim // 2)]
    if scaling is None:
        return inv
    if scaling.kind == "linear":
        return [f / scaling.factor for f in inv]
    if scaling.kind == "llama3":
        old = float(scaling.original_max_position)
        low_wl, high_wl = old / scaling.low_freq_factor, old / scaling.high_freq_factor
        out = []
        for f in inv:
            wl = 2.0 * math.pi / f
            if wl > low_wl:
                f = f / scaling.factor
            elif wl >= high_wl:
                smooth = (old / wl - scaling.low_freq_factor) / (scaling.high_freq_factor - scaling.low_freq_factor)
                f = (1.0 - smooth) * f / scaling.factor + smooth * f
            out.append(f)
        return out
    if scaling.kind == "yarn":
        dim = float(rotary_dim)

        def correction(rotations: float) -> float:
            return dim * math.log(scaling.original_max_position / (rotations * 2.0 * math.pi)) / (2.0 * math.log(theta))
        low = max(math.floor(correction(scaling.beta_fast)), 0.0)
        high = min(math.ceil(correction(scaling.beta_slow)), dim - 1.0)
        if high == low:
            high += 0.001
        out = []
        for i, f in enumerate(inv):
            ramp = min(max((i - low) / (high - low), 0.0), 1.0)
            keep = 1.0 - ramp                                   # 1: the frequency stays, 0: it is divided
            out.append(f / scaling.factor * (1.0 - keep) + f * keep)
        return out
    raise ValueError(f"unknown rope scaling '{scaling.kind}' (linear, llama3, yarn)")


class PositionEncoding:
    """What the attention mixer needs from a position encoding."""
    rotary_dim: int = 0
    cos: Optional[torch.Tensor] = None     # float32 [max_positions, rotary_dim / 2]
    sin: Optional[torch.Tensor] = None
    max_positions: int = 0
    #: which elements of a head turn together by angle i: "half" (i and i + rotary_dim/2, the reference's
    #: layout, src/model/layers.rs:159) or "interleaved" (2i and 2i + 1)
    pairing: str = "half"

    def prepare(self, device: torch.device) -> None:
        """Build the tables on ``device``."""


class RotaryEmbedding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_positions: int, rotary_dim: Optional[int] = None,
                 scaling: Optional[RopeScaling] = None, pairing: str = "half"):
        rd = head_dim if rotary_dim is None else rotary_dim
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown pairing '{pairing}' (half, interleaved)")
        self.pairing = pairing
        if rd % 2 or rd > head_dim or rd <= 0:
            raise ValueError(f"rotary_dim {rd} must be even and within head_dim {head_dim}")
        self.head_dim, self.theta, self.max_positions, self.rotary_dim = head_dim, float(theta), int(max_positions), rd
        self.scaling = scaling
        rope_inv_freq(rd, self.theta, scaling)         # refuses an unknown kind here, not at the first step

    def prepare(self, device: torch.device) -> None:
        """cos and sin of position x frequency, computed in float64, times YaRN's attention factor where
        there is one (src/model/layers.rs:237-251), stored in float32."""
        inv_freq = torch.tensor(rope_inv_freq(self.rotary_dim, self.theta, self.scaling), dtype=torch.float64)
        ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        mscale = self.scaling.attention_factor if self.scaling is not None and self.scaling.kind == "yarn" else 1.0
        self.cos = (ang.cos() * mscale).to(torch.float32).to(device).contiguous()
        self.sin = (ang.sin() * mscale).to(torch.float32).to(device).contiguous()


class NoPositionEncoding(PositionEncoding):
    """Attention without any rotation."""
