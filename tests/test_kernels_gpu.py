"""Each CUDA kernel alone against a plain PyTorch reference, at sizes other than the engine's."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


def dev():
    return torch.device("cuda:0")


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    want = want.to(torch.float64).cpu()
    return float((got.to(torch.float64).cpu() - want).abs().max() / want.abs().max().clamp_min(1e-30))


@pytest.fixture(scope="module")
def ops():
    from carbon_engine_b200 import ops as o
    return o


def status():
    return torch.zeros(1, dtype=torch.int32, device=dev())


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(ops, dtype):
    V, H = 301, 80
    table = torch.randn(V, H, device=dev()).to(dtype)
    toks = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=dev())
    x = torch.empty(5, H, dtype=torch.float32, device=dev())
    st = status()
    ops.embed(table, toks, x, st)
    assert torch.equal(x, table[toks.long()].float()) and st.item() == 0
    bad = torch.tensor([1, 301], dtype=torch.int32, device=dev())
    ops.embed(table, bad, x[:2], st)
    assert st.item() == 1 and torch.equal(x[1], torch.zeros(H, device=dev()))      # flagged, not read


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [48, 80, 1000, 4104])
def test_rmsnorm(ops, dtype, H):
    x = torch.randn(7, H, device=dev()) * 3
    w = 1 + 0.1 * torch.randn(H, device=dev())
    out = torch.empty(7, H, dtype=dtype, device=dev())
    ops.rmsnorm(x, w, out, 1e-5)
    want = plain.rms_norm(x.double().cpu(), w.double().cpu(), 1e-5)
    assert rel_err(out, want) < TOL[dtype]
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=dev())
    out2 = torch.empty(3, H, dtype=dtype, device=dev())
    ops.rmsnorm(x, w, out2, 1e-5, rows)
    assert torch.equal(out2, out[rows.long()])


def paged_layout(seq_lens, page_size, nkv, d, dtype, shuffle_seed=0, extra_pages=3):
    """Block table and empty pools for sequences of the given lengths, pages handed out in a
    shuffled order so that nothing lies where a contiguous layout would put it."""
    need = [(n + page_size - 1) // page_size for n in seq_lens]
    total = sum(need) + extra_pages
    perm = np.random.default_rng(shuffle_seed).permutation(total)
    max_pages = max(need) + 2
    table = np.full((len(seq_lens), max_pages), -1, dtype=np.int32)
    k = 0
    for b, n in enumerate(need):
        table[b, :n] = perm[k:k + n]
        k += n
    pool = lambda: torch.full((total, nkv, page_size, d), float("nan"), dtype=dtype, device=dev())
    return torch.from_numpy(table).to(dev()), pool(), pool()


def fill_pools(kp, vp, table, seq, k, v, page_size, start=0):
    """Write k, v [n, nkv, d] of sequence ``seq`` at positions start.. into the pools (test-side)."""
    for i in range(k.shape[0]):
        pos = start + i
        page = int(table[seq, pos // page_size])
        kp[page, :, pos % page_size, :] = k[i]
        vp[page, :, pos % page_size, :] = v[i]


def step_meta(seqs):
    """seqs: list of (ctx_before, q_len).  Device int32 arrays positions, seq_of_token, seq_slot."""
    pos, sot = [], []
    for b, (c, n) in enumerate(seqs):
        pos += list(range(c, c + n))
        sot += [b] * n
    mk = lambda a: torch.tensor(a, dtype=torch.int32, device=dev())
    return mk(pos), mk(sot), mk(list(range(len(seqs))))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rd,ps", [(6, 3, 48, 48, 8), (4, 1, 16, 16, 16), (5, 5, 80, 32, 4), (2, 2, 256, 256, 64),
                                            (8, 2, 128, 128, 64), (3, 1, 64, 64, 16), (4, 2, 192, 192, 8), (2, 1, 128, 64, 16)])
@pytest.mark.parametrize("first", [9, 270])        # few tokens: a warp a head; from 256 tokens on a warp takes several heads of a token
def test_qk_norm_rope_and_cache_write(ops, dtype, nh, nkv, d, rd, ps, first):
    torch.manual_seed(1)
    seqs = [(5, first), (0, 3), (30, 1)]
    T = sum(n for _, n in seqs)
    table, kp, vp = paged_layout([c + n for c, n in seqs], ps, nkv, d, dtype)
    qkv = (torch.randn(T, (nh + 2 * nkv) * d, device=dev()) * 2).to(dtype)
    qw, kw = 1 + 0.2 * torch.randn(d, device=dev()), 1 + 0.2 * torch.randn(d, device=dev())
    theta, eps = 3000.0, 1e-5
    positions, sot, slots = step_meta(seqs)
    half = rd // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2 / rd)
    ang = torch.arange(320, dtype=torch.float64)[:, None] * inv[None]
    cos, sin = ang.cos().float().to(dev()), ang.sin().float().to(dev())
    src = qkv.clone()
    st = status()
    ops.qk_rope_kvwrite(qkv, kp, vp, qw, kw, cos, sin, positions, sot, slots, table, st, nh, nkv, d, rd, ps, eps)
    assert st.item() == 0
    s64 = src.double().cpu()
    q = s64[:, :nh * d].view(T, nh, d)
    k = s64[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
    v = s64[:, (nh + nkv) * d:].view(T, nkv, d)
    c, s = plain.rope_tables(positions.cpu(), rd, theta)
    q_want = plain.apply_rope(plain.rms_norm(q, qw.double().cpu(), eps), c, s)
    k_want = plain.apply_rope(plain.rms_norm(k, kw.double().cpu(), eps), c, s)
    assert rel_err(qkv[:, :nh * d].view(T, nh, d), q_want) < TOL[dtype]
    t = 0
    for b, (ctx, n) in enumerate(seqs):
        for i in range(n):
            pos = ctx + i
            page = int(table[b, pos // ps])
            assert rel_err(kp[page, :, pos % ps, :], k_want[t]) < TOL[dtype]
            assert torch.equal(vp[page, :, pos % ps, :].double().cpu(), v[t])          # V is copied as it is
            t += 1
    # nothing else was written: all other places still hold the poison
    written = T * nkv * d
    assert int((~torch.isnan(kp.float())).sum()) == written and int((~torch.isnan(vp.float())).sum()) == written


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,rd", [(4, 2, 64, 64), (3, 1, 48, 32), (2, 2, 128, 128)])
def test_qk_rotation_with_interleaved_pairs(ops, dtype, nh, nkv, d, rd):
    """The pairing is a parameter: elements 2i and 2i + 1 turn together by angle i."""
    torch.manual_seed(4)
    seqs, ps = [(7, 5), (0, 1)], 8
    T = 6
    table, kp, vp = paged_layout([c + n for c, n in seqs], ps, nkv, d, dtype)
    qkv = torch.randn(T, (nh + 2 * nkv) * d, device=dev()).to(dtype)
    positions, sot, slots = step_meta(seqs)
    c, s = plain.rope_tables(torch.arange(32), rd, 500.0)
    src = qkv.clone()
    st = status()
    ops.qk_rope_kvwrite(qkv, kp, vp, None, None, c.float().to(dev()), s.float().to(dev()), positions, sot, slots, table, st,
                        nh, nkv, d, rd, ps, 0.0, pairing="interleaved")
    assert st.item() == 0
    q = src.double().cpu()[:, :nh * d].view(T, nh, d)
    cp, sp = c[positions.cpu().long()][:, None, :], s[positions.cpu().long()][:, None, :]
    want = q.clone()
    want[..., 0:rd:2] = q[..., 0:rd:2] * cp - q[..., 1:rd:2] * sp
    want[..., 1:rd:2] = q[..., 1:rd:2] * cp + q[..., 0:rd:2] * sp
    assert rel_err(qkv[:, :nh * d].view(T, nh, d), want) < TOL[dtype]
    halves = plain.apply_rope(q, c[positions.cpu().long()], s[positions.cpu().long()])
    assert rel_err(qkv[:, :nh * d].view(T, nh, d), halves) > 0.1           # and it is not the other pairing
    with pytest.raises(Exception, match="pairing"):
        ops.qk_rope_kvwrite(qkv, kp, vp, None, None, None, None, positions, sot, slots, table, st, nh, nkv, d, 0, ps, 0.0,
                            pairing="pairs")


def test_qk_kernel_flags_a_page_the_request_does_not_hold(ops):
    table, kp, vp = paged_layout([4], 4, 1, 16, torch.float32)
    qkv = torch.randn(1, 3 * 16, device=dev())
    positions, sot, slots = step_meta([(5, 1)])               # position 5 lies in page index 1, which is not held
    st = status()
    ops.qk_rope_kvwrite(qkv, kp, vp, None, None, None, None, positions, sot, slots, table, st, 1, 1, 16, 0, 4, 0.0)
    assert st.item() == 2 and torch.isnan(kp).all()


def reference_attention(q_all, k_all, v_all, ctx, n, scale, window):
    """Rows ctx..ctx+n of the whole-sequence attention."""
    return plain.causal_attention(q_all, k_all, v_all, scale, window)[ctx:ctx + n]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d,ps,window", [(6, 3, 48, 8, 0), (8, 2, 32, 16, 0), (4, 4, 16, 4, 0), (3, 1, 128, 32, 0),
                                                 (6, 2, 64, 8, 37), (2, 1, 16, 16, 130)])
def test_attention_generic_over_pages(ops, dtype, nh, nkv, d, ps, window):
    torch.manual_seed(2)
    seqs = [(0, 19), (140, 1), (257, 1), (61, 7), (0, 2), (126, 5)]       # whole, decode (past a chunk edge), portions
    lens = [c + n for c, n in seqs]
    table, kp, vp = paged_layout(lens, ps, nkv, d, dtype, shuffle_seed=3)
    T = sum(n for _, n in seqs)
    q_step = torch.empty(T, nh * d, dtype=dtype, device=dev())
    want = []
    t = 0
    for b, (ctx, n) in enumerate(seqs):
        L = ctx + n
        q_all = (torch.randn(L, nh, d) * 1.5).to(dtype)
        k_all = (torch.randn(L, nkv, d) * 1.5).to(dtype)
        v_all = torch.randn(L, nkv, d).to(dtype)
        fill_pools(kp, vp, table.cpu().numpy(), b, k_all.to(dev()), v_all.to(dev()), ps)
        q_step[t:t + n] = q_all[ctx:].reshape(n, nh * d).to(dev())
        want.append(reference_attention(q_all.double(), k_all.double(), v_all.double(), ctx, n, 1 / math.sqrt(d), window))
        t += n
    positions, sot, slots = step_meta(seqs)
    out = torch.empty(T, nh * d, dtype=dtype, device=dev())
    st = status()
    ops.attention_generic(q_step, nh * d, kp, vp, out, positions, sot, slots, table, st, nh, nkv, d, ps, window,
                          1 / math.sqrt(d))
    assert st.item() == 0
    assert rel_err(out.view(T, nh, d), torch.cat(want)) < (2e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds_and_respects_the_window_edge(ops, dtype):
    """One key is made to stand out: the output must be that key's value.  It is put at the first
    position, at a page's last place, right at the window's edge and one before it."""
    nh, nkv, d, ps = 2, 1, 32, 16
    L = 700
    torch.manual_seed(3)
    for far, window, visible in ((0, 0, True), (15, 0, True), (699 - 99, 100, True), (699 - 100, 100, False), (383, 0, True)):
        table, kp, vp = paged_layout([L], ps, nkv, d, dtype, shuffle_seed=far)
        k_all = torch.randn(L, nkv, d) * 0.1
        v_all = torch.randn(L, nkv, d)
        q = torch.randn(1, nh, d)
        k_all[far, 0] = q[0, 1] * 4.0              # head 1's score for this key: 4 |q|^2 / sqrt(d), far above the rest
        k_all, v_all, q = k_all.to(dtype), v_all.to(dtype), q.to(dtype)
        fill_pools(kp, vp, table.cpu().numpy(), 0, k_all.to(dev()), v_all.to(dev()), ps)
        positions, sot, slots = step_meta([(L - 1, 1)])
        out = torch.empty(1, nh * d, dtype=dtype, device=dev())
        st = status()
        ops.attention_generic(q.reshape(1, nh * d).to(dev()), nh * d, kp, vp, out, positions, sot, slots, table, st,
                              nh, nkv, d, ps, window, 1.0)
        got = out.view(nh, d)[1].float().cpu()
        hit = (got - v_all[far, 0].float()).abs().max() < 0.05
        assert bool(hit) == visible, (far, window)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (3, 64, 16), (65, 129, 33), (130, 70, 200), (2, 301, 80)])
def test_gemm_plain_all_epilogues(ops, dtype, M, N, K):
    torch.manual_seed(4)
    a = torch.randn(M, K, device=dev()).to(dtype)
    w = torch.randn(N, K, device=dev()).to(dtype)
    ref = a.double().cpu() @ w.double().cpu().T
    c = torch.empty(M, N, dtype=dtype, device=dev())
    ops.gemm_plain(a, w, c, ops.GEMM_STORE)
    assert rel_err(c, ref) < TOL[dtype]
    c32 = torch.empty(M, N, dtype=torch.float32, device=dev())
    ops.gemm_plain(a, w, c32, ops.GEMM_STORE_F32)
    assert rel_err(c32, ref) < 1e-5
    x = torch.randn(M, N, device=dev())
    x0 = x.clone()
    ops.gemm_plain(a, w, x, ops.GEMM_ACCUM_F32)
    assert rel_err(x, x0.double().cpu() + ref) < 1e-5
    w2 = torch.randn(2 * N, K, device=dev()).to(dtype)
    g = a.double().cpu() @ w2[:N].double().cpu().T
    u = a.double().cpu() @ w2[N:].double().cpu().T
    s = torch.empty(M, N, dtype=dtype, device=dev())
    ops.gemm_plain(a, w2, s, ops.GEMM_SWIGLU)
    assert rel_err(s, g * torch.sigmoid(g) * u) < TOL[dtype]


def test_gemm_plain_rows_do_not_depend_on_their_neighbours(ops):
    """The same row gives the same bits whatever else is in the batch."""
    a = torch.randn(77, 96, device=dev())
    w = torch.randn(50, 96, device=dev())
    full = torch.empty(77, 50, device=dev())
    ops.gemm_plain(a, w, full, ops.GEMM_STORE)
    one = torch.empty(1, 50, device=dev())
    ops.gemm_plain(a[70:71].contiguous(), w, one, ops.GEMM_STORE)
    assert torch.equal(one[0], full[70])


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_and_residual_add(ops, dtype):
    gu = torch.randn(5, 2 * 112, device=dev()).to(dtype)
    out = torch.empty(5, 112, dtype=dtype, device=dev())
    ops.swiglu(gu, out)
    g, u = gu[:, :112].double().cpu(), gu[:, 112:].double().cpu()
    assert rel_err(out, g * torch.sigmoid(g) * u) < TOL[dtype]
    x = torch.randn(5, 80, device=dev())
    dlt = torch.randn(5, 80, device=dev()).to(dtype)
    want = x.double().cpu() + dlt.double().cpu()
    ops.add_residual(x, dlt)
    assert rel_err(x, want) < 1e-6


def test_scatter_i32(ops):
    dst = torch.full((4, 5), -1, dtype=torch.int32, device=dev())
    ops.scatter_i32(dst, torch.tensor([0, 7, 19], dtype=torch.int32, device=dev()),
                    torch.tensor([4, 5, 6], dtype=torch.int32, device=dev()))
    want = torch.full((20,), -1, dtype=torch.int32)
    want[[0, 7, 19]] = torch.tensor([4, 5, 6], dtype=torch.int32)
    assert torch.equal(dst.cpu().view(-1), want)


@pytest.mark.parametrize("rows,V", [(3, 151936 // 8 + 3), (8, 151936), (1, 151936), (100, 40009), (5, 1000)])
def test_argmax_takes_the_first_maximum(ops, rows, V):
    """A few rows of a large vocabulary are shared by the blocks of a cluster (8 rows: 8 blocks a row), many rows
    or a small vocabulary take one block a row; the pick is the first maximum either way."""
    torch.manual_seed(rows + V)
    logits = torch.randn(rows, V, device=dev())
    want = []
    for r in range(rows):
        kind = r % 4
        if kind == 0:                           # a tie between places that different blocks and threads hold: the lower index wins
            a, b = 777 % V, (12000 + 1025 * r) % V
            logits[r, a] = logits[r, b] = 50.0
            want.append(min(a, b))
        elif kind == 1:
            logits[r, V - 1] = 60.0             # the very last place
            want.append(V - 1)
        elif kind == 2:
            logits[r] = -1.0                    # all equal: index 0 (src/sampling.rs:96-106)
            want.append(0)
        else:
            want.append(int(logits[r].argmax()))
    out = torch.empty(rows, dtype=torch.int32, device=dev())
    ops.argmax(logits, out)
    assert out.tolist() == want


def run_sampler(ops, logits, rows):
    params = torch.from_numpy(np.frombuffer(ops.pack_sample_rows(rows), dtype=np.uint8).copy()).to(dev())
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=dev())
    ops.sample(logits, params, out)
    return out.tolist()


def gumbel_reference(logits_row, temperature, kept, seed):
    """The draw the kernel makes, from the same counter-based uniforms (src/kernels/sampling.cu:30-42)."""
    from carbon_engine_b200.sampling.sampler import mix64
    best, best_i = -1e300, -1
    for i in sorted(int(k) for k in kept):
        h = mix64(seed ^ mix64((i + 0x632BE59BD9B4E019) & ((1 << 64) - 1)))
        u = ((h >> 40) + 0.5) / 16777216.0
        g = float(logits_row[i]) / max(temperature, 1e-5) - math.log(-math.log(u))
        if g > best:
            best, best_i = g, i
    return best_i


@pytest.mark.parametrize("V,copies", [(1000, 1), (16384 + 37, 1), (40009, 4), (40009, 20)])
def test_sampler_options_follow_the_host_rules(ops, V, copies):
    """Small vocabularies take one block a row; from 16,384 entries on a cluster of up to 8 blocks shares
    a row (8, 4 or 1 blocks a row here, by the number of rows).  The rules and the draws are the same."""
    rng = np.random.default_rng(5)
    base = [(0.0, 1.0, 0.0, 0, 1), (0.8, 1.0, 0.0, 1, 2), (0.8, 1.0, 0.0, 5, 3), (1.3, 0.6, 0.0, 0, 4),
            (0.7, 1.0, 0.2, 0, 5), (1.0, 0.9, 0.05, 50, 6)]
    rows = [(t, p, m, k, seed + 10 * c) for c in range(copies) for (t, p, m, k, seed) in base]
    logits = torch.from_numpy(rng.normal(size=(len(rows), V)).astype(np.float32) * 3).to(dev())
    got = run_sampler(ops, logits, rows)
    host = logits.cpu().numpy()
    for r, (t, p, m, k, seed) in enumerate(rows):
        if r % 6 < 2:                                                              # temperature 0, top_k 1: greedy
            assert got[r] == int(host[r].argmax())
            continue
        if copies > 1 and r >= 12:                                                 # (the host loop is slow: two copies are checked in full)
            continue
        kept, _ = plain.sample_kept_set(host[r], t, k, p, m)
        assert got[r] in set(kept.tolist()), r
        assert got[r] == gumbel_reference(host[r], t, kept, seed), r
    assert run_sampler(ops, logits, rows) == got                                    # same seeds, same tokens
    other = run_sampler(ops, logits, [(t, p, m, k, s + 1000) for (t, p, m, k, s) in rows])
    assert other[:2] == got[:2] and other[2:6] != got[2:6]


def test_sampler_draws_from_the_softmax(ops):
    probs = np.array([0.4, 0.3, 0.15, 0.1, 0.05])
    n = 4000
    logits = torch.from_numpy(np.tile(np.log(probs).astype(np.float32) * 0.7, (n, 1))).to(dev())   # temperature undoes the 0.7
    got = np.array(run_sampler(ops, logits, [(0.7, 1.0, 0.0, 0, 1000 + i) for i in range(n)]))
    freq = np.bincount(got, minlength=5) / n
    assert np.abs(freq - probs).max() < 0.03
    got = np.array(run_sampler(ops, logits, [(0.7, 0.8, 0.0, 0, 5000 + i) for i in range(n)]))    # nucleus: 0.4+0.3+0.15
    freq = np.bincount(got, minlength=5) / n
    assert freq[3] == 0 and freq[4] == 0 and np.abs(freq[:3] - probs[:3] / 0.85).max() < 0.03


def test_penalties(ops):
    logits = torch.tensor([[2.0, -2.0, 1.0, 0.5], [1.0, 1.0, 1.0, 1.0]], device=dev())
    # row 0: token 0 seen in the prompt, token 1 generated twice, token 2 generated once; row 1 has no penalties
    entries = torch.tensor([[0, 0, 1, 0], [0, 1, 1, 2], [0, 2, 1, 1]], dtype=torch.int32, device=dev())
    row_params = torch.tensor([[2.0, 0.5, 0.25], [1.0, 0.0, 0.0]], device=dev())
    ops.apply_penalties(logits, entries, row_params)
    want = [[2.0 / 2, -2.0 * 2 - (0.5 + 0.25 * 2), 1.0 / 2 - (0.5 + 0.25), 0.5], [1.0, 1.0, 1.0, 1.0]]
    assert torch.allclose(logits.cpu(), torch.tensor(want))


def test_kernels_refuse_sizes_they_cannot_take(ops):
    from carbon_engine_b200.csrc.kernel_lib import KernelError
    with pytest.raises(KernelError, match="head_dim"):
        table, kp, vp = paged_layout([4], 4, 1, 2048, torch.float32)
        positions, sot, slots = step_meta([(0, 1)])
        q = torch.zeros(1, 2048, device=dev())
        ops.attention_generic(q, 2048, kp, vp, torch.empty(1, 2048, device=dev()), positions, sot, slots, table,
                              status(), 1, 1, 2048, 4, 0, 1.0)
    with pytest.raises(KernelError, match="CUDA tensor"):
        ops.rmsnorm(torch.zeros(1, 8), torch.ones(8), torch.zeros(1, 8), 1e-6)


# ---- bfloat16 tensor-core attention (decode split-KV + flash prefill) -----------------------------
class FakeCtx:
    """The fields of a step context the attention kernels read."""

    def __init__(self, seqs):
        mk = lambda a: torch.tensor(a, dtype=torch.int32, device=dev())
        order = sorted(range(len(seqs)), key=lambda i: 0 if seqs[i][1] == 1 else 1)
        self.order = order
        pos, qs, ctx, tiles, tiles128 = [], [0], [], [], []
        self.n_decode = sum(1 for c, n in seqs if n == 1)
        dec = 1
        for bi, i in enumerate(order):
            c, n = seqs[i]
            pos += list(range(c, c + n))
            qs.append(qs[-1] + n)
            ctx.append(c + n)
            if n == 1:
                dec = max(dec, c + n)
            else:
                tiles += [[bi, q0] for q0 in range(0, n, 64)]
                tiles128 += [[bi, q0] for q0 in range(0, n, 128)]
        self.T = qs[-1]
        self.positions, self.q_start, self.ctx_len = mk(pos), mk(qs), mk(ctx)
        self.seq_slot = mk(order)                  # sequence bi of the step uses block-table row order[bi]
        self.tiles = mk(tiles if tiles else [[0, 0]])
        self.n_tiles = len(tiles)
        self.tiles128 = mk(tiles128 if tiles128 else [[0, 0]])
        self.n_tiles128 = len(tiles128)
        from carbon_engine_b200 import ops_tensor
        split = ops_tensor.decode_split()
        self.decode_splits = (dec + split - 1) // split
        self.status = status()
        self.device = dev()
        self._s = {}

    def scratch(self, name, numel):
        if name not in self._s or self._s[name].numel() < numel:
            self._s[name] = torch.full((max(numel, 1),), float("nan"), device=dev())
        return self._s[name]


class FakeCache:
    def __init__(self, kp, vp, ps):
        self.k_pool, self.v_pool, self.page_size = kp, vp, ps


def run_mma_attention(seqs, nh, nkv, d, ps, window, scale, seed=0, far=None, extra_splits=0):
    """Returns (got [T, nh, d] in the caller's sequence order, want)."""
    from carbon_engine_b200 import ops_tensor
    lens = [c + n for c, n in seqs]
    table, kp, vp = paged_layout(lens, ps, nkv, d, torch.bfloat16, shuffle_seed=seed + 1)
    ctx = FakeCtx(seqs)
    ctx.decode_splits += extra_splits
    q_step = torch.zeros(ctx.T, nh * d + 2 * nkv * d, dtype=torch.bfloat16, device=dev())    # q inside a wider qkv row
    want = {}
    t = 0
    for bi, i in enumerate(ctx.order):
        c, n = seqs[i]
        L = c + n
        # a sequence's numbers depend on the seed and on its own lengths only, so that the same sequence
        # can be run again in another batch
        gen = torch.Generator().manual_seed(seed * 1000003 + c * 131 + n)
        q_all = (torch.randn(L, nh, d, generator=gen) * 1.5).to(torch.bfloat16)
        k_all = (torch.randn(L, nkv, d, generator=gen) * 1.5).to(torch.bfloat16)
        v_all = torch.randn(L, nkv, d, generator=gen).to(torch.bfloat16)
        if far is not None and i == far[0]:
            k_all[far[1], 0] = (q_all[L - 1, nh - 1].float() * 3.0).to(torch.bfloat16)     # last head's last query loves this key
        fill_pools(kp, vp, table.cpu().numpy(), i, k_all.to(dev()), v_all.to(dev()), ps)
        q_step[t:t + n, :nh * d] = q_all[c:].reshape(n, nh * d).to(dev())
        want[i] = plain.causal_attention(q_all.double(), k_all.double(), v_all.double(), scale, window)[c:]
        t += n
    out = torch.full((ctx.T, nh * d), float("nan"), dtype=torch.bfloat16, device=dev())
    ok = ops_tensor.attention_bf16(ctx, ctx, q_step, out, FakeCache(kp, vp, ps), table, nh, nkv, d, window, scale)
    assert ok and ctx.status.item() == 0
    got, t = {}, 0
    for bi, i in enumerate(ctx.order):
        n = seqs[i][1]
        got[i] = out[t:t + n].view(n, nh, d)
        t += n
    return got, want


@pytest.mark.parametrize("nh,nkv,d,ps,window", [(32, 8, 128, 64, 0), (6, 3, 48, 8, 0), (8, 2, 32, 16, 0), (4, 4, 16, 4, 0),
                                                 (3, 1, 256, 32, 0), (40, 2, 64, 16, 0), (6, 2, 64, 8, 37), (4, 1, 80, 16, 300),
                                                 (4, 2, 192, 16, 0), (2, 1, 128, 128, 150)])
def test_mma_attention_decode_and_prefill_mixed(nh, nkv, d, ps, window):
    # decode rows at contexts around the split (256) and tile (64) edges, portions with and without a cached prefix
    seqs = [(0, 19), (255, 1), (256, 1), (700, 1), (61, 7), (0, 2), (126, 130), (0, 1), (63, 1), (300, 65)]
    got, want = run_mma_attention(seqs, nh, nkv, d, ps, window, 1 / math.sqrt(d))
    for i in range(len(seqs)):
        assert rel_err(got[i], want[i]) < 2e-2, (i, seqs[i])


def test_mma_decode_result_does_not_depend_on_the_grid():
    """The same call twice gives the same bits.  A grid with more splits than the longest context needs
    (as under a captured graph) may cut the positions into splits of another size: the float32 partial
    results are then merged in another grouping, so the bfloat16 outputs may differ in their last bit,
    not more (the plain result is 2e-2 away at most; the two grids are held to a quarter of that)."""
    from carbon_engine_b200 import ops_tensor
    seqs = [(511, 1), (100, 1)]
    a, want = run_mma_attention(seqs, 8, 2, 64, 16, 0, 0.125, seed=7)
    again, _ = run_mma_attention(seqs, 8, 2, 64, 16, 0, 0.125, seed=7)
    assert torch.equal(a[0], again[0]) and torch.equal(a[1], again[1])
    b, _ = run_mma_attention(seqs, 8, 2, 64, 16, 0, 0.125, seed=7, extra_splits=5)
    for i in range(2):
        assert rel_err(b[i], a[i].double()) < 5e-3
        assert rel_err(b[i], want[i]) < 2e-2
    # the second sequence alone (same numbers): another number of sequences and another longest context,
    # so other split sizes; again the last bit at most
    alone, want_alone = run_mma_attention(seqs[1:], 8, 2, 64, 16, 0, 0.125, seed=7)
    assert torch.equal(want_alone[0], want[1])
    assert rel_err(alone[0], a[1].double()) < 5e-3 and rel_err(alone[0], want[1]) < 2e-2


@pytest.mark.parametrize("far,window,visible", [(0, 0, True), (63, 0, True), (64, 0, True), (255, 0, True), (256, 0, True),
                                                 (899 - 99, 100, True), (899 - 100, 100, False), (511, 0, True)])
@pytest.mark.parametrize("n_new", [1, 5])
def test_mma_attention_finds_one_far_key(far, window, visible, n_new):
    """One key among 900 stands out for the last query of the last head: at the first position, at tile
    and split edges, at the window's edge and one before it.  Both the decode and the flash kernel."""
    nh, nkv, d, ps = 4, 1, 64, 16
    L = 900
    seqs = [(L - n_new, n_new)]
    got, want = run_mma_attention(seqs, nh, nkv, d, ps, window, 1.0, seed=far, far=(0, far))
    assert rel_err(got[0], want[0]) < 2e-2
    # the plain result itself shows that the key decides the output when (and only when) it is visible
    _, base = run_mma_attention(seqs, nh, nkv, d, ps, window, 1.0, seed=far, far=None)
    moved = float((want[0][-1, -1] - base[0][-1, -1]).abs().max()) > 0.5
    assert moved == visible


def test_mma_attention_refuses_odd_head_sizes():
    from carbon_engine_b200 import ops_tensor
    assert not ops_tensor.attention_supported(40, 128) and not ops_tensor.attention_supported(272, 1024)
    assert ops_tensor.attention_supported(48, 96)


# ---- bfloat16 products on tcgen05 ------------------------------------------------------------------
def tc_product(a, w, mode, N, x0=None):
    from carbon_engine_b200 import ops_tensor, ops as o
    M = a.shape[0]
    if mode == o.GEMM_STORE_F32:
        out = torch.full((M, N), float("nan"), device=dev())
    elif mode == o.GEMM_ACCUM_F32:
        out = x0.clone()
    else:
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    assert ops_tensor.gemm_bf16(a, w, out, mode), "the tensor-core product refused the shape"
    torch.cuda.synchronize()
    assert ops_tensor.gemm_status(a.device) == 0
    return out


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 256, 4096), (16, 96, 80), (17, 301, 136), (64, 4096, 512), (100, 200, 1000),
                                   (256, 384, 256), (300, 520, 192), (5, 1000, 2048), (2048, 512, 256), (1000, 5120, 128),
                                   (257, 19000, 64), (200, 4096, 512), (130, 3200, 192), (256, 1600, 128)])
def test_tcgen05_product_all_epilogues(ops, M, N, K):
    """The last three sizes have 129 to 256 tokens and at least a dozen tiles of a CTA pair (the third only as a
    SwiGLU product): they go to the pair kernel, with one partly filled tile of tokens."""
    torch.manual_seed(M * 7 + N)
    pairs_before = ops.kernel_counts().get("gemm_tc_pair_kernel", 0)
    a = torch.randn(M, K, device=dev()).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev()) / math.sqrt(K)).to(torch.bfloat16)
    ref = a.double().cpu() @ w.double().cpu().T
    assert rel_err(tc_product(a, w, ops.GEMM_STORE, N), ref) < 1e-2
    assert rel_err(tc_product(a, w, ops.GEMM_STORE_F32, N), ref) < 2e-5
    x0 = torch.randn(M, N, device=dev())
    assert rel_err(tc_product(a, w, ops.GEMM_ACCUM_F32, N, x0), x0.double().cpu() + ref) < 2e-5
    w2 = (torch.randn(2 * N, K, device=dev()) / math.sqrt(K)).to(torch.bfloat16)
    g = a.double().cpu() @ w2[:N].double().cpu().T
    u = a.double().cpu() @ w2[N:].double().cpu().T
    assert rel_err(tc_product(a, w2, ops.GEMM_SWIGLU, N), g * torch.sigmoid(g) * u) < 1e-2
    pair_launches = ops.kernel_counts().get("gemm_tc_pair_kernel", 0) - pairs_before
    want_pairs = {(200, 4096, 512): 4, (130, 3200, 192): 4, (256, 1600, 128): 1, (256, 384, 256): 0, (100, 200, 1000): 0,
                  (64, 4096, 512): 0, (300, 520, 192): 4}
    if (M, N, K) in want_pairs:
        assert pair_launches == want_pairs[(M, N, K)], pair_launches


@pytest.mark.parametrize("M,N,K", [(9, 256, 4096), (48, 520, 4096), (128, 256, 8192), (200, 384, 12288)])
def test_tcgen05_split_k_with_more_than_eight_tokens(ops, M, N, K):
    """Above 8 tokens every split of a tile adds the partial sums for its share of the tokens (the blocks
    wait for one another's partials): all epilogues against float64, at sizes that do split K."""
    from carbon_engine_b200.csrc.kernel_lib import kernels
    assert kernels().ce_gemm_tc_splits(M, N, K) > 1
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=dev()).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev()) / math.sqrt(K)).to(torch.bfloat16)
    ref = a.double().cpu() @ w.double().cpu().T
    for _ in range(3):        # the counters go back to zero after every launch
        assert rel_err(tc_product(a, w, ops.GEMM_STORE_F32, N), ref) < 2e-5
    assert rel_err(tc_product(a, w, ops.GEMM_STORE, N), ref) < 1e-2
    x0 = torch.randn(M, N, device=dev())
    assert rel_err(tc_product(a, w, ops.GEMM_ACCUM_F32, N, x0), x0.double().cpu() + ref) < 2e-5


def test_tcgen05_product_is_repeatable_and_rows_stand_alone(ops):
    """Split-K adds the partial sums in a fixed order: the same bits every time, and a token's row does
    not depend on how many other tokens share the step (while they fit one tile of tokens)."""
    from carbon_engine_b200.csrc.kernel_lib import kernels
    a = torch.randn(16, 4096, device=dev()).to(torch.bfloat16)
    w = (torch.randn(256, 4096, device=dev()) / 64).to(torch.bfloat16)
    assert kernels().ce_gemm_tc_splits(16, 256, 4096) > 1
    first = tc_product(a, w, ops.GEMM_STORE_F32, 256)
    for _ in range(5):
        assert torch.equal(tc_product(a, w, ops.GEMM_STORE_F32, 256), first)
    one = tc_product(a[5:6].contiguous(), w, ops.GEMM_STORE_F32, 256)
    assert torch.equal(one[0], first[5])
    # a larger tile of tokens may split K differently: equal within a tile size, close across tile sizes
    many = torch.cat([a, a, a, a])
    sixty = tc_product(many[:60].contiguous(), w, ops.GEMM_STORE_F32, 256)
    forty = tc_product(many[:40].contiguous(), w, ops.GEMM_STORE_F32, 256)
    assert torch.equal(sixty[21], forty[21])
    assert rel_err(sixty[21], first[5]) < 1e-5


def test_tcgen05_product_refuses_what_tma_cannot_address(ops):
    from carbon_engine_b200 import ops_tensor
    a = torch.randn(4, 100, device=dev()).to(torch.bfloat16)          # K = 100 is no multiple of 8
    w = torch.randn(32, 100, device=dev()).to(torch.bfloat16)
    out = torch.empty(4, 32, dtype=torch.bfloat16, device=dev())
    assert not ops_tensor.gemm_bf16(a, w, out, ops.GEMM_STORE)
    from carbon_engine_b200.parts import linear
    linear.matmul_nt(a, w, out, linear.STORE)                          # the plain kernel takes it
    assert rel_err(out, a.double().cpu() @ w.double().cpu().T) < 1e-2


@pytest.mark.parametrize("nh,nkv,d,ps,window", [(32, 8, 128, 64, 0), (4, 2, 128, 16, 0), (6, 3, 64, 8, 0), (8, 2, 64, 32, 50),
                                                 (4, 1, 128, 128, 200)])
def test_tcgen05_attention_over_long_portions(nh, nkv, d, ps, window):
    """Portions longer than one tile of 128 queries, with and without a cached prefix, next to short ones."""
    from carbon_engine_b200 import ops_tensor
    assert ops_tensor.kernels().ce_attention_prefill_tc_supported(d, ps, (nh + 2 * nkv) * d)
    seqs = [(0, 300), (517, 131), (64, 128), (0, 1), (1000, 3), (127, 2)]
    got, want = run_mma_attention(seqs, nh, nkv, d, ps, window, 1 / math.sqrt(d), seed=11)
    for i in range(len(seqs)):
        assert rel_err(got[i], want[i]) < 2e-2, (i, seqs[i])


def test_tcgen05_attention_agrees_with_the_mma_kernel():
    from carbon_engine_b200 import ops_tensor
    seqs = [(200, 190), (0, 77)]
    a, want = run_mma_attention(seqs, 8, 2, 128, 64, 0, 0.09, seed=5)
    ops_tensor.USE_TENSOR_ATTENTION = False
    try:
        b, _ = run_mma_attention(seqs, 8, 2, 128, 64, 0, 0.09, seed=5)
    finally:
        ops_tensor.USE_TENSOR_ATTENTION = True
    for i in range(2):
        assert rel_err(a[i], b[i]) < 1e-2 and rel_err(a[i], want[i]) < 2e-2
