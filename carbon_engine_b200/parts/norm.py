"""RMSNorm: y = x * (1 / sqrt(mean(x^2) + eps)) * weight, the weight used as stored (no "+1")
(src/model/layers.rs:117-146).  The weight is held in float32 whatever it was stored in; the sum of
squares and the scaling are float32."""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from .base import Norm, TensorGetter, TensorSpec


class RMSNorm(Norm):
    def __init__(self, width: int, eps: float, name: str):
        self.width, self.eps, self.name = int(width), float(eps), name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.width,), "norm")]

    def load(self, get: TensorGetter, device, dtype) -> None:
        self.weight = get(self.name).to(device).to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
        ops.rmsnorm(x, self.weight, out, self.eps, rows)
