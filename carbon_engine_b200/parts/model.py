"""A decoder put together from parts: embedding, blocks, the order the blocks run in, and the head.

The order is data: a list of :class:`LayerCall`.  A call names the block to run and the cache it
uses; a block may be named twice, and a call may read a cache that another call writes
(``writes=False``).  The plain case is one call per block, each with a cache of its own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .base import Block, CacheSpec, Part
from .embedding import Embedding, LMHead


@dataclass(frozen=True)
class LayerCall:
    block: int
    cache: int
    writes: bool = True


def plain_schedule(n_blocks: int) -> List[LayerCall]:
    return [LayerCall(i, i, True) for i in range(n_blocks)]


class DecoderModel(Part):
    def __init__(self, config, embedding: Embedding, blocks: Sequence[Block], head: LMHead,
                 schedule: Optional[Sequence[LayerCall]] = None):
        self.config = config
        self.embedding = embedding
        self.blocks = list(blocks)
        self.head = head
        self.schedule = list(schedule) if schedule is not None else plain_schedule(len(self.blocks))
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None
        writers = {}
        for call in self.schedule:
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"the schedule names block {call.block}, but there are {len(self.blocks)}")
            if call.writes:
                if call.cache in writers:
                    raise ValueError(f"cache {call.cache} is written by two calls")
                writers[call.cache] = call.block
        for call in self.schedule:
            if not call.writes and call.cache not in writers:
                raise ValueError(f"cache {call.cache} is read but never written")
        self._writers = writers

    def children(self) -> List[Part]:
        return [self.embedding, *self.blocks, self.head]

    @property
    def graph_safe(self) -> bool:
        """True if a step of this model can be captured in a CUDA graph: every mixer reads the step
        from device buffers only."""
        return all(getattr(b.mixer, "graph_safe", False) for b in self.blocks)

    def cache_layout(self) -> List[tuple]:
        """(cache id, spec) for every cache of the schedule, taken from the mixer that writes it."""
        out = []
        for cache_id in sorted(self._writers):
            spec: CacheSpec = self.blocks[self._writers[cache_id]].mixer.cache_spec()
            out.append((cache_id, spec))
        return out

    def step_bytes(self, tokens: int, element_size: int, rows: int = 0) -> int:
        """Activations of a step of ``tokens`` tokens with logits at ``rows`` places: the float32 residual
        stream, the largest block's buffers (blocks run one after another), the normed rows and the logits."""
        blocks = max((b.step_bytes(tokens, element_size) for b in self.blocks), default=0)
        return tokens * self.embedding.width * 4 + blocks + rows * (self.head.width * element_size + self.head.vocab * 4)

    def load_weights(self, get, device: torch.device, dtype: torch.dtype) -> None:
        self.device, self.dtype = device, dtype
        self.load_all(get, device, dtype)

    def forward(self, ctx, caches) -> torch.Tensor:
        """Run all tokens of the step through the schedule; returns the residual stream [T, width]."""
        x = torch.empty((ctx.T, self.embedding.width), dtype=torch.float32, device=self.device)
        self.embedding.forward(ctx, x)
        for call in self.schedule:
            self.blocks[call.block].forward(ctx, x, caches.view(call))
        return x

    def logits(self, ctx, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        return self.head.forward(ctx, x, rows)
