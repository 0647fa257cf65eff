"""Tensor-core kernels of the bfloat16 path.  Each function returns False when it does not take
the shape it is given, and the caller then uses the plain kernel."""
from __future__ import annotations

import ctypes

import torch

from . import ops
from .csrc import kernel_lib
from .csrc.kernel_lib import kernels

_i, _f, _ll, _p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
kernel_lib.declare("ce_attention_decode_scratch", _ll, [_i, _i, _i, _i])
# q, k_pool, v_pool, out, scratch, counters, n_counters, positions, seq_slot, q_start, ctx_len, block_table, status,
# n_seqs, nh, nkv, d, q_stride, page_size, max_pages, num_pages, window, scale, max_splits, stream
kernel_lib.declare("ce_attention_decode_bf16", _i, [_p] * 6 + [_i] + [_p] * 6 + [_i] * 9 + [_f, _i, _p])
kernel_lib.declare("ce_attention_decode_split", _i, [])
kernel_lib.declare("ce_attention_decode_kernels", _i, [])
# q, k_pool, v_pool, out, positions, seq_slot, q_start, ctx_len, block_table, tiles, status,
# n_tiles, nh, nkv, d, q_stride, page_size, max_pages, num_pages, window, scale, stream
kernel_lib.declare("ce_attention_prefill_bf16", _i, [_p] * 11 + [_i] * 9 + [_f, _p])

kernel_lib.declare("ce_gemm_tc_supported", _i, [_i, _i, _i, _i])
kernel_lib.declare("ce_gemm_tc_scratch", _ll, [_i, _i, _i, _i])
kernel_lib.declare("ce_gemm_tc_splits", _i, [_i, _i, _i])
# A, W, C, M, N, K, lda, ldc, mode, scratch, scratch_floats, counters, n_counters, status, stream
kernel_lib.declare("ce_gemm_tc", _i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _ll, _p, _i, _p, _p])


def decode_split() -> int:
    """Positions per split of the decode attention kernel."""
    return kernels().ce_attention_decode_split()

GEMM_SCRATCH_FLOATS = 16 << 20        # 64 MB of split-K partial sums
GEMM_COUNTERS = 1 << 16

kernel_lib.declare("ce_attention_prefill_tc_supported", _i, [_i, _i, _i])
# q, k_pool, v_pool, out, seq_slot, q_start, ctx_len, block_table, tiles, status,
# n_tiles, total_tokens, nh, nkv, d, q_stride, page_size, max_pages, num_pages, window, scale, stream
kernel_lib.declare("ce_attention_prefill_tc", _i, [_p] * 10 + [_i] * 10 + [_f, _p])

#: set to False to keep portions of prompts off the tcgen05 attention kernel (the mma.sync one takes them)
USE_TENSOR_ATTENTION = True
#: set to False to keep bfloat16 products off the tcgen05 kernel
USE_TENSOR_GEMM = True

_workspaces = {}


class _Workspace:
    def __init__(self, device):
        self.scratch = torch.empty(GEMM_SCRATCH_FLOATS, dtype=torch.float32, device=device)
        self.counters = torch.zeros(GEMM_COUNTERS, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.attn_counters = torch.zeros(GEMM_COUNTERS, dtype=torch.int32, device=device)


def gemm_workspace(device) -> _Workspace:
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    ws = _workspaces.get(device)
    if ws is None:
        ws = _workspaces[device] = _Workspace(device)
    return ws


def reset_counters(device) -> None:
    """Zero the split-K and split-KV counters (after a step that failed: its kernels may have stopped
    half way through a count)."""
    ws = _workspaces.get(torch.device(device))
    if ws is not None:
        ws.counters.zero_()
        ws.attn_counters.zero_()


def gemm_status(device) -> int:
    """0, or the code a tensor-core product left behind (5: a wait inside the kernel timed out)."""
    ws = _workspaces.get(torch.device(device))
    return 0 if ws is None else int(ws.status.item())


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int) -> bool:
    """out (op)= a @ w.T on the tcgen05 kernel; False if the shape is refused."""
    if not USE_TENSOR_GEMM or a.dtype != torch.bfloat16:
        return False
    M, K = a.shape
    N = out.shape[1]
    k = kernels()
    if a.stride(1) != 1 or not w.is_contiguous() or out.stride(1) != 1:
        return False
    if not k.ce_gemm_tc_supported(M, N, K, a.stride(0)) or (a.data_ptr() | w.data_ptr()) & 15:
        return False
    need = k.ce_gemm_tc_scratch(M, N, K, mode)
    ws = gemm_workspace(a.device)
    if need > ws.scratch.numel():
        return False
    ops._ok(k.ce_gemm_tc(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), out.stride(0), mode,
                         ws.scratch.data_ptr(), ws.scratch.numel(), ws.counters.data_ptr(), ws.counters.numel(),
                         ws.status.data_ptr(), ops._stream()))
    return True


def attention_supported(d: int, q_stride: int) -> bool:
    return 16 <= d <= 256 and d % 16 == 0 and q_stride % 2 == 0


def attention_bf16(ctx, plan, qkv, out, cache, table, nh, nkv, d, window, scale) -> bool:
    """Decode kernel for the leading one-token sequences, flash kernel for the portions.  ``plan``: the
    step's tile lists and split bound (``parts.attention.AttentionPlan``)."""
    if not attention_supported(d, qkv.shape[1]):
        return False
    k = kernels()
    stream = ops._stream()
    args = (cache.page_size, table.shape[1], cache.k_pool.shape[0], int(window), float(scale))
    if ctx.n_decode > 0:
        splits = plan.decode_splits
        need = k.ce_attention_decode_scratch(ctx.n_decode, nh, d, splits)
        scratch = ctx.scratch("attention_decode", need)
        ws = gemm_workspace(qkv.device)
        ops._ok(k.ce_attention_decode_bf16(
            qkv.data_ptr(), cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), out.data_ptr(), scratch.data_ptr(),
            ws.attn_counters.data_ptr(), ws.attn_counters.numel(), ctx.positions.data_ptr(), ctx.seq_slot.data_ptr(), ctx.q_start.data_ptr(), ctx.ctx_len.data_ptr(),
            table.data_ptr(), ctx.status.data_ptr(), ctx.n_decode, nh, nkv, d, qkv.shape[1], *args, splits, stream),
                k.ce_attention_decode_kernels())
    if plan.n_tiles > 0 and USE_TENSOR_ATTENTION and plan.n_tiles128 > 0 and \
            k.ce_attention_prefill_tc_supported(d, cache.page_size, qkv.shape[1]):
        ops._ok(k.ce_attention_prefill_tc(
            qkv.data_ptr(), cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), out.data_ptr(), ctx.seq_slot.data_ptr(),
            ctx.q_start.data_ptr(), ctx.ctx_len.data_ptr(), table.data_ptr(), plan.tiles128.data_ptr(),
            ctx.status.data_ptr(), plan.n_tiles128, qkv.shape[0], nh, nkv, d, qkv.shape[1], *args, stream))
    elif plan.n_tiles > 0:
        ops._ok(k.ce_attention_prefill_bf16(
            qkv.data_ptr(), cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), out.data_ptr(),
            ctx.positions.data_ptr(), ctx.seq_slot.data_ptr(), ctx.q_start.data_ptr(), ctx.ctx_len.data_ptr(),
            table.data_ptr(), plan.tiles.data_ptr(), ctx.status.data_ptr(), plan.n_tiles, nh, nkv, d, qkv.shape[1],
            *args, stream))
    return True
