"""Grouped-query attention over the paged cache, with optional per-head q/k RMSNorm, optional
rotary embedding and an optional window.

Order of operations, as the reference has it (src/model/attention.rs:868-914): one product for q, k
and v; RMSNorm over each head of q and k with one weight of head_dim shared by all heads, before
the rotation (:884-889); K (normed, rotated) and V are written to the cache before attending (:890),
so new tokens read themselves from the cache; scores scaled by ``scale`` (1/sqrt(head_dim) unless
given, :810); query at absolute position p sees keys up to p (:1038-1063), or the last ``window``
of them; query head h reads KV head h // (heads / kv_heads) (:1035); then the output product, added
into the residual stream (:913, src/model/mod.rs:648).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .. import ops
from .base import Mixer, PagedCacheSpec, Part, TensorGetter, TensorSpec
from .linear import ACCUM, STORE, Linear
from .rope import PositionEncoding


def split_bucket(splits: int) -> int:
    """Round a split count up to the next value with at most three significant bits (1..8, 10, 12, 14,
    16, 20, ...): few distinct grids (a captured graph per bucket), and a grid at most a quarter larger
    than the contexts need."""
    step = 1
    while splits > 8 * step:
        step *= 2
    return (splits + step - 1) // step * step


class AttentionPlan:
    """What the attention kernels need of a step beyond the common tables: the tiles of the sequences
    that bring more than one token, 64 and 128 tokens at a time, as (sequence, first token) pairs on
    the device, and the grid bound of the split-KV decode kernel."""

    def __init__(self, tiles, n_tiles, tiles128, n_tiles128, decode_splits):
        self.tiles, self.n_tiles, self.tiles128, self.n_tiles128 = tiles, n_tiles, tiles128, n_tiles128
        self.decode_splits = decode_splits       # >= ceil(longest one-token sequence's context / positions per split)
        self.graph_key = decode_splits


class PagedAttention(Mixer):
    graph_safe = True       # reads positions, tables and lengths from device buffers only
    plan_key = "paged_attention"
    TILE, TILE_TC = 64, 128         # tokens per tile of the mma.sync and of the tcgen05 flash kernel

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, prefix: str,
                 position: Optional[PositionEncoding] = None, qk_norm_eps: Optional[float] = None,
                 window: int = 0, scale: Optional[float] = None, page_size: Optional[int] = None):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.prefix, self.position, self.qk_norm_eps, self.window = prefix, position, qk_norm_eps, int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.page_size = page_size          # None: the engine's; else this layer's cache has pages of its own size
        self.qkv = Linear(hidden, [heads * head_dim, kv_heads * head_dim, kv_heads * head_dim],
                          [f"{prefix}.q_proj.weight", f"{prefix}.k_proj.weight", f"{prefix}.v_proj.weight"])
        self.o = Linear(heads * head_dim, [hidden], [f"{prefix}.o_proj.weight"])
        self.q_norm_weight: Optional[torch.Tensor] = None
        self.k_norm_weight: Optional[torch.Tensor] = None

    def children(self) -> List[Part]:
        return [self.qkv, self.o]

    def tensor_specs(self) -> List[TensorSpec]:
        if self.qk_norm_eps is None:
            return []
        return [TensorSpec(f"{self.prefix}.q_norm.weight", (self.head_dim,), "norm"),
                TensorSpec(f"{self.prefix}.k_norm.weight", (self.head_dim,), "norm")]

    def ignorable_tensors(self) -> List[str]:
        # older checkpoints store the rotary frequencies, which are recomputed from the configuration
        return [f"{self.prefix}.rotary_emb.inv_freq"] if self.position is not None else []

    def load(self, get: TensorGetter, device, dtype) -> None:
        if self.qk_norm_eps is not None:
            self.q_norm_weight = get(f"{self.prefix}.q_norm.weight").to(device).to(torch.float32).contiguous()
            self.k_norm_weight = get(f"{self.prefix}.k_norm.weight").to(device).to(torch.float32).contiguous()
        if self.position is not None and self.position.cos is None:
            self.position.prepare(device)

    def cache_spec(self) -> PagedCacheSpec:
        return PagedCacheSpec(self.kv_heads, self.head_dim, self.window, self.page_size)

    def step_bytes(self, tokens: int, element_size: int) -> int:
        return tokens * (2 * self.heads + 2 * self.kv_heads) * self.head_dim * element_size      # q|k|v and the heads' outputs

    def step_sections(self, max_tokens: int, max_seqs: int):
        return [("paged_attention.tiles", 2 * (max_seqs + max_tokens // self.TILE + 1)),
                ("paged_attention.tiles_tc", 2 * (max_seqs + max_tokens // self.TILE_TC + 1))]

    def plan_step(self, ctx) -> AttentionPlan:
        """Tile lists for the flash kernels and the decode kernel's split bound.  The bound is rounded up
        to a bucket whether or not the step is replayed as a graph, so that both ways run the same grid."""
        from .. import ops_tensor
        h_tiles = ctx.bufs.host_section("paged_attention.tiles")
        h_tiles_tc = ctx.bufs.host_section("paged_attention.tiles_tc")
        nt = nt_tc = 0
        longest = 1
        for b in range(ctx.B):
            n = ctx.h_q_start[b + 1] - ctx.h_q_start[b]
            if b < ctx.n_decode:
                longest = max(longest, ctx.h_ctx_before[b] + 1)
                continue
            for q0 in range(0, n, self.TILE):
                h_tiles[2 * nt], h_tiles[2 * nt + 1] = b, q0
                nt += 1
            for q0 in range(0, n, self.TILE_TC):
                h_tiles_tc[2 * nt_tc], h_tiles_tc[2 * nt_tc + 1] = b, q0
                nt_tc += 1
        per_split = ops_tensor.decode_split()
        return AttentionPlan(ctx.bufs.dev_section("paged_attention.tiles"), nt,
                             ctx.bufs.dev_section("paged_attention.tiles_tc"), nt_tc,
                             split_bucket((longest + per_split - 1) // per_split))

    def forward(self, ctx, h: torch.Tensor, x: torch.Tensor, cache) -> None:
        T = h.shape[0]
        nh, nkv, d = self.heads, self.kv_heads, self.head_dim
        qkv = ctx.buffer((T, (nh + 2 * nkv) * d))
        self.qkv.forward(h, qkv, STORE)
        pos = self.position
        cos = pos.cos if pos is not None else None
        sin = pos.sin if pos is not None else None
        if cos is not None and ctx.max_position >= cos.shape[0]:
            raise ValueError(f"position {ctx.max_position} is beyond the rotary table ({cos.shape[0]}): raise max_seq_len")
        table = ctx.block_tables[cache.group]
        ops.qk_rope_kvwrite(qkv, cache.k_pool, cache.v_pool, self.q_norm_weight, self.k_norm_weight, cos, sin,
                            ctx.positions, ctx.seq_of_token, ctx.seq_slot, table, ctx.status, nh, nkv, d,
                            pos.rotary_dim if cos is not None else 0, cache.page_size,
                            self.qk_norm_eps if self.qk_norm_eps is not None else 0.0, write_kv=cache.writes,
                            pairing=pos.pairing if pos is not None else "half")
        out = ctx.buffer((T, nh * d))
        self.attend(ctx, qkv, out, cache, table)
        self.o.forward(out, x, ACCUM)

    def attend(self, ctx, qkv: torch.Tensor, out: torch.Tensor, cache, table: torch.Tensor) -> None:
        nh, nkv, d = self.heads, self.kv_heads, self.head_dim
        prof = ops.profiling()
        if prof is not None:         # keys and values of every sequence once, queries and outputs; causal flops
            el, keys, pairs = qkv.element_size(), 0, 0
            for b in range(ctx.B):
                n, before = ctx.h_q_start[b + 1] - ctx.h_q_start[b], ctx.h_ctx_before[b]
                keys += before + n
                pairs += n * before + n * (n + 1) // 2
            prof.note_work((2 * keys * nkv * d + 2 * ctx.T * nh * d) * el, 4 * pairs * nh * d)
        if qkv.dtype == torch.bfloat16 and ctx.fast_attention:
            from .. import ops_tensor
            if ops_tensor.attention_bf16(ctx, ctx.plans[self.plan_key], qkv, out, cache, table, nh, nkv, d, self.window,
                                         self.scale):
                return
        ops.attention_generic(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, out, ctx.positions, ctx.seq_of_token,
                              ctx.seq_slot, table, ctx.status, nh, nkv, d, cache.page_size, self.window, self.scale)
