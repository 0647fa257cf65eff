"""Token embedding and the language-model head.

x0[t] = E[token[t]], no scaling (src/model/mod.rs:781-784).  The head takes the final norm of the
requested rows only and multiplies by the head matrix into float32 logits
(src/model/mod.rs:793-802); with tied embeddings the head IS the embedding tensor
(src/model/mod.rs:735): the same memory, no copy.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Norm, Part, TensorGetter, TensorSpec, to_device
from .linear import STORE_F32, matmul_nt


class Embedding(Part):
    def __init__(self, vocab: int, width: int, name: str):
        self.vocab, self.width, self.name = vocab, width, name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab, self.width), "embedding")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        self.weight = to_device(get(self.name), device, dtype)

    def forward(self, ctx, x: torch.Tensor) -> None:
        ops.embed(self.weight, ctx.tokens, x, ctx.status)


class LMHead(Part):
    """Final norm + head product for chosen rows.  ``tied_to`` shares an embedding's tensor."""

    def __init__(self, vocab: int, width: int, norm: Norm, name: Optional[str], tied_to: Optional[Embedding] = None,
                 redundant_name: Optional[str] = None):
        """``redundant_name``: with a tied head, the name under which a checkpoint may still store a copy
        of the head; it is ignored, as the reference ignores it (src/model/mod.rs:725)."""
        if (name is None) == (tied_to is None):
            raise ValueError("the head has either a tensor of its own or an embedding it is tied to")
        self.vocab, self.width, self.norm, self.name, self.tied_to = vocab, width, norm, name, tied_to
        self.redundant_name = redundant_name if tied_to is not None else None
        self._weight: Optional[torch.Tensor] = None

    def ignorable_tensors(self) -> List[str]:
        return [self.redundant_name] if self.redundant_name else []

    def children(self) -> List[Part]:
        return [self.norm]

    def tensor_specs(self) -> List[TensorSpec]:
        return [] if self.name is None else [TensorSpec(self.name, (self.vocab, self.width), "linear")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        if self.name is not None:
            self._weight = to_device(get(self.name), device, dtype)

    @property
    def weight(self) -> torch.Tensor:
        return self.tied_to.weight if self.tied_to is not None else self._weight

    def forward(self, ctx, x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        R = rows.shape[0]
        logits = torch.empty((R, self.vocab), dtype=torch.float32, device=x.device)
        if R == 0:
            return logits
        z = ctx.buffer((R, self.width))
        self.norm.forward(x, z, rows)
        matmul_nt(z, self.weight, logits, STORE_F32)
        return logits
