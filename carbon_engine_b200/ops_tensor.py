"""Tensor-core kernels of the bfloat16 path.  Each function returns False when it does not take
the shape it is given, and the caller then uses the plain kernel."""
from __future__ import annotations

import torch


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int) -> bool:
    return False


def attention_bf16(ctx, qkv, out, cache, table, nh, nkv, d, window, scale) -> bool:
    return False
