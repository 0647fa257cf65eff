"""The entry point for callers that cannot allocate device memory (csrc/kernels/no_alloc.h).

Some hosts of these kernels may not call cudaMalloc: a plug-in living in another runtime's memory
arena, a loop that must never wait on the allocator.  For them the library offers the split-KV
decode attention with its scratch memory in a fixed array of its own.  This test calls that entry
point through its exported C symbol, several times in a row with different sizes, on shapes whose
partial results really pass through the scratch memory, and requires each result to equal the
ordinary entry point's (which takes the scratch from the caller) and to be right by the plain
computation.  It is collected
last, so that a run that stops at the first failure has run everything else before.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_fn():
    from carbon_engine_b200.csrc.kernel_lib import kernels
    lib = kernels()
    fn = lib.ce_attention_decode_bf16_static
    p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.restype = i
    fn.argtypes = [p] * 10 + [i] * 9 + [f, i, p]
    lib.ce_attention_decode_tma_supported.restype = i
    lib.ce_attention_decode_tma_supported.argtypes = [i, i]
    lib.ce_attention_decode_scratch.restype = ctypes.c_longlong
    lib.ce_attention_decode_scratch.argtypes = [i, i, i, i]
    lib.ce_attention_decode_bf16.restype = i
    lib.ce_attention_decode_bf16.argtypes = [p] * 6 + [i] + [p] * 6 + [i] * 9 + [f, i, p]
    return lib, fn


def _case(seed, seqs, nh, nkv, d, ps):
    """Inputs of a decode step (one new token per sequence) over a shuffled paged cache, and what plain
    attention gives for them."""
    import plain_qwen3 as plain
    from test_kernels_gpu import FakeCache, FakeCtx, dev, fill_pools, paged_layout
    gen = torch.Generator().manual_seed(seed)
    table, kp, vp = paged_layout([c + 1 for c, _ in seqs], ps, nkv, d, torch.bfloat16, shuffle_seed=seed)
    ctx = FakeCtx(seqs)
    q = torch.zeros(ctx.T, (nh + 2 * nkv) * d, dtype=torch.bfloat16, device=dev())
    plain_out = []
    for b, (c, _) in enumerate(seqs):
        k_all = (torch.randn(c + 1, nkv, d, generator=gen) * 1.5).to(torch.bfloat16)
        v_all = torch.randn(c + 1, nkv, d, generator=gen).to(torch.bfloat16)
        q_b = (torch.randn(nh, d, generator=gen) * 1.5).to(torch.bfloat16)
        fill_pools(kp, vp, table.cpu().numpy(), b, k_all.to(dev()), v_all.to(dev()), ps)
        q[b, :nh * d] = q_b.reshape(-1).to(dev())
        q_all = torch.zeros(c + 1, nh, d, dtype=torch.float64)
        q_all[c] = q_b.double()
        plain_out.append(plain.causal_attention(q_all, k_all.double(), v_all.double(), 1 / math.sqrt(d))[c].reshape(-1))
    return ctx, q, table, FakeCache(kp, vp, ps), torch.stack(plain_out)


def _run_both(fn, lib, seed, seqs, nh, nkv, d, ps):
    """One decode step through the ordinary entry point (scratch and counters from the caller) and through
    the one that allocates nothing; both must have used scratch memory (no merge inside a cluster) and
    must agree bit for bit, and both must be right by the plain computation."""
    from carbon_engine_b200 import ops, ops_tensor
    from test_kernels_gpu import dev
    assert not lib.ce_attention_decode_tma_supported(d, ps), "this shape would merge in a cluster and use no scratch"
    ctx, q, table, cache, plain_out = _case(seed, seqs, nh, nkv, d, ps)
    scale = 1 / math.sqrt(d)
    stream = torch.cuda.current_stream().cuda_stream
    tail = (ctx.n_decode, nh, nkv, d, q.shape[1], ps, table.shape[1], cache.k_pool.shape[0], 0, scale, ctx.decode_splits, stream)
    # the ordinary entry point, with the caller's scratch (NaN: nothing stale may be read) and zeroed counters
    need = lib.ce_attention_decode_scratch(ctx.n_decode, nh, d, ctx.decode_splits)
    scratch = torch.full((need,), float("nan"), device=dev())
    counters = torch.zeros(4096, dtype=torch.int32, device=dev())
    want = torch.full((ctx.T, nh * d), float("nan"), dtype=torch.bfloat16, device=dev())
    before = ops.kernel_counts().get("attention_merge_kernel", 0)
    rc = lib.ce_attention_decode_bf16(
        q.data_ptr(), cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), want.data_ptr(), scratch.data_ptr(),
        counters.data_ptr(), counters.numel(), ctx.positions.data_ptr(), ctx.seq_slot.data_ptr(), ctx.q_start.data_ptr(),
        ctx.ctx_len.data_ptr(), table.data_ptr(), ctx.status.data_ptr(), *tail)
    assert rc == 0, lib.ce_last_error().decode()
    got = torch.full_like(want, float("nan"))
    rc = fn(q.data_ptr(), cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), got.data_ptr(), ctx.positions.data_ptr(),
            ctx.seq_slot.data_ptr(), ctx.q_start.data_ptr(), ctx.ctx_len.data_ptr(), table.data_ptr(),
            ctx.status.data_ptr(), *tail)
    assert rc == 0, lib.ce_last_error().decode()
    torch.cuda.synchronize()
    assert ops.kernel_counts().get("attention_merge_kernel", 0) == before + 2      # both went through scratch + merge
    assert ctx.status.item() == 0
    assert torch.isfinite(got.float()).all()
    assert torch.equal(got, want)                # the same kernels on the same numbers: the same bits
    err = float((got.double().cpu() - plain_out).abs().max() / plain_out.abs().max())
    assert err < 2e-2, err                       # the tolerance of the kernel tests
    return got


def test_decode_attention_without_allocation_matches_the_ordinary_entry_point():
    """Three calls in a row, each with other sizes: the fixed array still holds the partial results of the
    call before, laid out for other head counts and split counts, when the next one starts."""
    lib, fn = _static_fn()
    a = _run_both(fn, lib, 1, [(700, 1), (30, 1), (1500, 1)], 6, 3, 48, 8)
    b = _run_both(fn, lib, 2, [(90, 1), (2047, 1)], 8, 2, 80, 16)
    c = _run_both(fn, lib, 3, [(400, 1), (33, 1), (260, 1), (5, 1)], 4, 4, 64, 4)      # (pages of 4: no TMA)
    assert a.shape == (3, 288) and b.shape == (2, 640) and c.shape == (4, 256)


def test_sizes_beyond_the_fixed_array_are_refused():
    lib, fn = _static_fn()
    # 64 sequences x 64 heads x 64 splits x 130 floats: far more than the 2 Mi floats the library holds
    rc = fn(1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 64, 64, 8, 128, 8192, 64, 64, 64, 0, 0.1, 64, None)
    assert rc != 0 and "scratch" in lib.ce_last_error().decode()
    # 600 sequences x 8 KV heads want 4800 counters, the library holds 4096 (the partial results would fit)
    rc = fn(1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 600, 8, 8, 16, 384, 16, 64, 64, 0, 0.1, 1, None)
    assert rc != 0 and "counters" in lib.ce_last_error().decode()
