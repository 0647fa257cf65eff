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
# q, k_pool, v_pool, out, scratch, positions, seq_slot, q_start, ctx_len, block_table, status,
# n_seqs, nh, nkv, d, q_stride, page_size, max_pages, num_pages, window, scale, max_splits, stream
kernel_lib.declare("ce_attention_decode_bf16", _i, [_p] * 11 + [_i] * 9 + [_f, _i, _p])
# q, k_pool, v_pool, out, positions, seq_slot, q_start, ctx_len, block_table, tiles, status,
# n_tiles, nh, nkv, d, q_stride, page_size, max_pages, num_pages, window, scale, stream
kernel_lib.declare("ce_attention_prefill_bf16", _i, [_p] * 11 + [_i] * 9 + [_f, _p])

DECODE_SPLIT = 256


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int) -> bool:
    return False


def attention_supported(d: int, q_stride: int) -> bool:
    return 16 <= d <= 256 and d % 16 == 0 and q_stride % 2 == 0


def attention_bf16(ctx, qkv, out, cache, table, nh, nkv, d, window, scale) -> bool:
    """Decode kernel for the leading one-token sequences, flash kernel for the portions."""
    if not attention_supported(d, qkv.shape[1]):
        return False
    k = kernels()
    stream = torch.cuda.current_stream().cuda_stream
    args = (cache.page_size, table.shape[1], cache.k_pool.shape[0], int(window), float(scale))
    if ctx.n_decode > 0:
        splits = ctx.decode_splits
        need = k.ce_attention_decode_scratch(ctx.n_decode, nh, d, splits)
        scratch = ctx.scratch("attention_decode", need)
        ops._ok(k.ce_attention_decode_bf16(
            qkv.data_ptr(), cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), out.data_ptr(), scratch.data_ptr(),
            ctx.positions.data_ptr(), ctx.seq_slot.data_ptr(), ctx.q_start.data_ptr(), ctx.ctx_len.data_ptr(),
            table.data_ptr(), ctx.status.data_ptr(), ctx.n_decode, nh, nkv, d, qkv.shape[1], *args, splits, stream), 2)
    if ctx.n_tiles > 0:
        ops._ok(k.ce_attention_prefill_bf16(
            qkv.data_ptr(), cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), out.data_ptr(),
            ctx.positions.data_ptr(), ctx.seq_slot.data_ptr(), ctx.q_start.data_ptr(), ctx.ctx_len.data_ptr(),
            table.data_ptr(), ctx.tiles.data_ptr(), ctx.status.data_ptr(), ctx.n_tiles, nh, nkv, d, qkv.shape[1],
            *args, stream))
    return True
