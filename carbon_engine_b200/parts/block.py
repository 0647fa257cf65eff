"""Arrangements of parts in a layer.  Pre-norm: x += mixer(norm1(x)); x += ffn(norm2(x))
(src/model/mod.rs:645-650)."""
from __future__ import annotations

from typing import List

import torch

from .base import Block, FeedForward, Mixer, Norm, Part


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Norm, ffn: FeedForward):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def children(self) -> List[Part]:
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def step_bytes(self, tokens: int, element_size: int) -> int:
        h = tokens * self.mixer_norm.width * element_size if hasattr(self.mixer_norm, "width") else 0
        return h + max(self.mixer.step_bytes(tokens, element_size), self.ffn.step_bytes(tokens, element_size))

    def forward(self, ctx, x: torch.Tensor, cache) -> None:
        h = ctx.buffer(tuple(x.shape))
        self.mixer_norm.forward(x, h)
        self.mixer.forward(ctx, h, x, cache)
        self.ffn_norm.forward(x, h)
        self.ffn.forward(ctx, h, x)
