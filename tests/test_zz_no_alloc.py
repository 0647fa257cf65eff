"""The entry point for callers that cannot allocate device memory (csrc/kernels/no_alloc.h).

Some hosts of these kernels may not call cudaMalloc: a plug-in living in another runtime's memory
arena, a loop that must never wait on the allocator.  For them the library offers the split-KV
decode attention with its scratch memory in a fixed array of its own.  This test calls that entry
point through its exported C symbol, twice in a row with different inputs, and compares each
result with the ordinary entry point (which takes the scratch from the caller).  It is collected
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
    return lib, fn


def _case(seed, seqs, nh, nkv, d, ps):
    """Inputs of a decode step (one new token per sequence) over a shuffled paged cache."""
    from test_kernels_gpu import FakeCache, FakeCtx, dev, fill_pools, paged_layout
    torch.manual_seed(seed)
    table, kp, vp = paged_layout([c + 1 for c, _ in seqs], ps, nkv, d, torch.bfloat16, shuffle_seed=seed)
    ctx = FakeCtx(seqs)
    q = torch.zeros(ctx.T, (nh + 2 * nkv) * d, dtype=torch.bfloat16, device=dev())
    for b, (c, _) in enumerate(seqs):
        k_all = (torch.randn(c + 1, nkv, d) * 1.5).to(torch.bfloat16)
        v_all = torch.randn(c + 1, nkv, d).to(torch.bfloat16)
        fill_pools(kp, vp, table.cpu().numpy(), b, k_all.to(dev()), v_all.to(dev()), ps)
        q[b, :nh * d] = (torch.randn(nh * d) * 1.5).to(torch.bfloat16).to(dev())
    return ctx, q, table, FakeCache(kp, vp, ps)


def _run_both(fn, lib, seed, seqs, nh, nkv, d, ps, window=0):
    from carbon_engine_b200 import ops_tensor
    from test_kernels_gpu import dev
    ctx, q, table, cache = _case(seed, seqs, nh, nkv, d, ps)
    scale = 1 / math.sqrt(d)
    want = torch.full((ctx.T, nh * d), float("nan"), dtype=torch.bfloat16, device=dev())
    assert ops_tensor.attention_bf16(ctx, q, want, cache, table, nh, nkv, d, window, scale)
    got = torch.full_like(want, float("nan"))
    rc = fn(q.data_ptr(), cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), got.data_ptr(), ctx.positions.data_ptr(),
            ctx.seq_slot.data_ptr(), ctx.q_start.data_ptr(), ctx.ctx_len.data_ptr(), table.data_ptr(),
            ctx.status.data_ptr(), ctx.n_decode, nh, nkv, d, q.shape[1], ps, table.shape[1], cache.k_pool.shape[0],
            window, scale, ctx.decode_splits, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.ce_last_error().decode()
    torch.cuda.synchronize()
    assert ctx.status.item() == 0
    assert torch.isfinite(got.float()).all()
    err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
    assert err < 2e-2, err                       # the tolerance of the kernel tests; in fact the same kernels ran
    return got


def test_decode_attention_without_allocation_matches_the_ordinary_entry_point():
    lib, fn = _static_fn()
    a = _run_both(fn, lib, 1, [(700, 1), (30, 1), (1500, 1)], 8, 2, 64, 16)
    # a second call right after, other sizes and other data: the shared array holds the first call's leftovers
    b = _run_both(fn, lib, 2, [(90, 1), (2047, 1)], 32, 8, 128, 64, window=0)
    c = _run_both(fn, lib, 3, [(400, 1), (33, 1), (260, 1)], 6, 3, 48, 8, window=100)
    assert a.shape == (3, 512) and b.shape == (2, 4096) and c.shape == (3, 288)


def test_sizes_beyond_the_fixed_array_are_refused():
    lib, fn = _static_fn()
    # 64 sequences x 64 heads x 64 splits x 130 floats: far more than the 2 Mi floats the library holds
    rc = fn(1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 64, 64, 8, 128, 8192, 64, 64, 64, 0, 0.1, 64, None)
    assert rc != 0 and "scratch" in lib.ce_last_error().decode()
