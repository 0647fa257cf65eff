"""Gated feed-forward: down(act(gate(h)) * up(h)), added into the residual stream
(src/model/layers.rs:568, 625-648; src/model/mod.rs:649).  Only SiLU is built; the gate and up
weights are held as one matrix so that one product with a SwiGLU epilogue serves both."""
from __future__ import annotations

from typing import List

import torch

from .base import FeedForward, Part
from .linear import ACCUM, SWIGLU, Linear


class GatedMLP(FeedForward):
    def __init__(self, hidden: int, intermediate: int, prefix: str, activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"activation '{activation}' is not supported (silu only)")
        self.hidden, self.intermediate, self.prefix = hidden, intermediate, prefix
        self.gate_up = Linear(hidden, [intermediate, intermediate],
                              [f"{prefix}.gate_proj.weight", f"{prefix}.up_proj.weight"])
        self.down = Linear(intermediate, [hidden], [f"{prefix}.down_proj.weight"])

    def children(self) -> List[Part]:
        return [self.gate_up, self.down]

    def step_bytes(self, tokens: int, element_size: int) -> int:
        return tokens * self.intermediate * element_size

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor) -> None:
        act = ctx.buffer((h.shape[0], self.intermediate))
        self.gate_up.forward(h, act, SWIGLU)
        self.down.forward(act, x, ACCUM)
