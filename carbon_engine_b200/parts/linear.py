"""Linear layers: y = x W^T with W stored [out_features, in_features] (src/model/layers.rs:441).

A :class:`Linear` may be the row-wise concatenation of several stored tensors that share their
input (q|k|v, gate|up), so that one product serves them all; the reference keeps them as separate
products (src/model/attention.rs:871).  The epilogue is part of the product: store in the
activation dtype, store float32 (logits), add into the float32 residual stream, or SwiGLU.

float32 runs the plain FMA kernel only.  bfloat16 runs the tensor-core kernels of
``csrc/kernels`` when they accept the shape and otherwise a library product (cuBLAS through
``torch.matmul``, where the reference also calls a library) followed by the epilogue kernel.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops
from .base import Part, TensorGetter, TensorSpec, to_device

STORE, STORE_F32, ACCUM, SWIGLU = ops.GEMM_STORE, ops.GEMM_STORE_F32, ops.GEMM_ACCUM_F32, ops.GEMM_SWIGLU

#: bfloat16 products go to "tensor" (own tcgen05 kernels), "library" (cuBLAS + epilogue kernel) or
#: "plain" (the FMA kernel); "auto" takes the first that accepts the shape.
BF16_BACKEND = "auto"
#: under "auto", products the tensor-core kernels refuse go to the plain kernel up to this many
#: multiply-adds and to the library above it
PLAIN_MAX_MACS = 1 << 24


def matmul_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, scratch=None) -> None:
    """out (op)= a @ w.T with the epilogue ``mode``; a [M, K], w [N or 2N, K]."""
    if a.shape[0] == 0:
        return
    prof = ops.profiling()
    if prof is not None:
        M, K = a.shape
        R = w.shape[0]          # weight rows: N, or 2N for SwiGLU
        prof.note_work((M * K + R * K) * a.element_size() + M * out.shape[1] * out.element_size(), 2 * M * R * K)
    if a.dtype == torch.float32 or BF16_BACKEND == "plain":
        ops.gemm_plain(a, w, out, mode)
        return
    if BF16_BACKEND in ("auto", "tensor"):
        from .. import ops_tensor
        if ops_tensor.gemm_bf16(a, w, out, mode):
            return
        if BF16_BACKEND == "tensor":
            raise ops.KernelError(f"the tensor-core product refuses a {tuple(a.shape)} x {tuple(w.shape)}^T product")
    if BF16_BACKEND == "auto" and a.shape[0] * w.shape[0] * a.shape[1] <= PLAIN_MAX_MACS:
        ops.gemm_plain(a, w, out, mode)      # small: one fused kernel, float32 accumulators into the epilogue
        return
    # library product, then the epilogue as a kernel of its own
    if mode == STORE:
        torch.matmul(a, w.t(), out=out)
    elif mode == STORE_F32:
        out.copy_(torch.matmul(a, w.t()))
    elif mode == ACCUM:
        ops.add_residual(out, torch.matmul(a, w.t()))
    elif mode == SWIGLU:
        ops.swiglu(torch.matmul(a, w.t()), out)
    else:
        raise ValueError(f"unknown epilogue {mode}")


class Linear(Part):
    def __init__(self, in_features: int, out_features: Sequence[int], names: Sequence[str], init: str = "linear"):
        if len(out_features) != len(names):
            raise ValueError("one name per stored tensor")
        self.in_features = int(in_features)
        self.out_features = [int(o) for o in out_features]
        self.names = list(names)
        self.init = init
        self.weight: Optional[torch.Tensor] = None

    @property
    def total_out(self) -> int:
        return sum(self.out_features)

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(n, (o, self.in_features), self.init) for n, o in zip(self.names, self.out_features)]

    def load(self, get: TensorGetter, device, dtype) -> None:
        parts = [to_device(get(n), device, dtype) for n in self.names]
        self.weight = parts[0] if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def forward(self, a: torch.Tensor, out: torch.Tensor, mode: int = STORE) -> None:
        matmul_nt(a, self.weight, out, mode)
