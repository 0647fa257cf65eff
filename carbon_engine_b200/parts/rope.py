"""Rotary position embedding tables.

inv_freq[i] = theta^(-2i/rd), angle = position * inv_freq[i]; cos and sin are computed in float64
and kept in float32 for both precisions (src/model/layers.rs:169-173, 237-251).  The rotation
itself (rotate-half pairing, src/model/layers.rs:159) happens inside the fused q/k kernel, which
reads rows of these tables at each token's position.  Another position encoding is another class
with the same two tables (or with none: ``cos is None`` turns the rotation off).
"""
from __future__ import annotations

from typing import Optional

import torch


class PositionEncoding:
    """What the attention mixer needs from a position encoding."""
    rotary_dim: int = 0
    cos: Optional[torch.Tensor] = None     # float32 [max_positions, rotary_dim / 2]
    sin: Optional[torch.Tensor] = None
    max_positions: int = 0

    def prepare(self, device: torch.device) -> None:
        """Build the tables on ``device``."""


class RotaryEmbedding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, max_positions: int, rotary_dim: Optional[int] = None):
        rd = head_dim if rotary_dim is None else rotary_dim
        if rd % 2 or rd > head_dim or rd <= 0:
            raise ValueError(f"rotary_dim {rd} must be even and within head_dim {head_dim}")
        self.head_dim, self.theta, self.max_positions, self.rotary_dim = head_dim, float(theta), int(max_positions), rd

    def prepare(self, device: torch.device) -> None:
        half = self.rotary_dim // 2
        inv_freq = self.theta ** (-torch.arange(0, half, dtype=torch.float64) * 2.0 / self.rotary_dim)
        ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.cos = ang.cos().to(torch.float32).to(device).contiguous()
        self.sin = ang.sin().to(torch.float32).to(device).contiguous()


class NoPositionEncoding(PositionEncoding):
    """Attention without any rotation."""
