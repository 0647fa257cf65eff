"""``devices --selftest``: every kernel once on the device against a plain float64 computation with
torch tensor ops, as the reference's self-test checks each of its kernels against a CPU softmax
reference (src/device.rs:152-416; tolerances 1e-4 in float32 and 3e-2 in 16-bit, src/device.rs:776-848)."""
from __future__ import annotations

import math

import torch

from . import ops, ops_tensor


def _rel(got, want) -> float:
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


def _attention_reference(q, k, v, scale):
    """q [L, nh, d], k/v [L, nkv, d]: whole-sequence causal attention in float64."""
    L, nh, d = q.shape
    g = nh // k.shape[1]
    mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
    out = torch.empty_like(q, dtype=torch.float64)
    for h in range(nh):
        s = (q[:, h].double() @ k[:, h // g].double().T) * scale
        out[:, h] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, h // g].double()
    return out


def run() -> int:
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    failures = []

    def check(name, err, tol):
        ok = err <= tol
        print(f"  {name:34s} {'ok  ' if ok else 'FAIL'} error {err:.2e} (tolerance {tol:.0e})")
        if not ok:
            failures.append(name)

    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 3e-2)):
        tag = "f32" if dtype == torch.float32 else "bf16"
        # embedding, norm
        table = torch.randn(97, 80, device=dev).to(dtype)
        toks = torch.tensor([3, 96, 0, 41], dtype=torch.int32, device=dev)
        x = torch.empty(4, 80, device=dev)
        ops.embed(table, toks, x, status)
        check(f"embedding {tag}", _rel(x, table[toks.long()].float()), 1e-7)
        w = 1 + 0.1 * torch.randn(80, device=dev)
        h = torch.empty(4, 80, dtype=dtype, device=dev)
        ops.rmsnorm(x, w, h, 1e-6)
        want = x.double() * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-6) * w.double()
        check(f"rmsnorm {tag}", _rel(h, want), tol)
        # products
        a = torch.randn(20, 96, device=dev).to(dtype)
        wm = (torch.randn(72, 96, device=dev) / 10).to(dtype)
        c = torch.empty(20, 72, dtype=dtype, device=dev)
        ops.gemm_plain(a, wm, c, ops.GEMM_STORE)
        check(f"plain product {tag}", _rel(c, a.double() @ wm.double().T), tol)
        gu = torch.randn(20, 64, device=dev).to(dtype)
        act = torch.empty(20, 32, dtype=dtype, device=dev)
        ops.swiglu(gu, act)
        g, u = gu[:, :32].double(), gu[:, 32:].double()
        check(f"swiglu {tag}", _rel(act, g * torch.sigmoid(g) * u), tol)
        # q/k norm + rotation + cache write, then attention over pages (a prefix, then a portion, then one token)
        nh, nkv, d, ps, L = 4, 2, 32, 8, 45
        qkv_all = torch.randn(L, (nh + 2 * nkv) * d, device=dev).to(dtype)
        kp = torch.full((8, nkv, ps, d), float("nan"), dtype=dtype, device=dev)
        vp = torch.full_like(kp, float("nan"))
        table_bt = torch.tensor([[5, 2, 7, 0, 3, 6, -1, -1]], dtype=torch.int32, device=dev)
        half = d // 2
        inv = 10000.0 ** (-torch.arange(half, dtype=torch.float64) * 2 / d)
        ang = torch.arange(64, dtype=torch.float64)[:, None] * inv[None]
        cos, sin = ang.cos().float().to(dev), ang.sin().float().to(dev)
        qw, kw = 1 + 0.1 * torch.randn(d, device=dev), 1 + 0.1 * torch.randn(d, device=dev)
        outs = []
        for lo, hi in ((0, 30), (30, 44), (44, 45)):
            n = hi - lo
            mk = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
            pos, sot, slot = mk(list(range(lo, hi))), mk([0] * n), mk([0])
            qkv = qkv_all[lo:hi].clone()
            ops.qk_rope_kvwrite(qkv, kp, vp, qw, kw, cos, sin, pos, sot, slot, table_bt, status, nh, nkv, d, d, ps, 1e-6)
            o = torch.empty(n, nh * d, dtype=dtype, device=dev)
            ops.attention_generic(qkv, qkv.shape[1], kp, vp, o, pos, sot, slot, table_bt, status, nh, nkv, d, ps, 0,
                                  1 / math.sqrt(d))
            outs.append(o)
        s64 = qkv_all.double()

        def norm_rope(t, wt):
            t = t * torch.rsqrt((t * t).mean(-1, keepdim=True) + 1e-6) * wt.double()
            c, s = ang[:L, None, :].cos().to(dev), ang[:L, None, :].sin().to(dev)
            t1, t2 = t[..., :half], t[..., half:]
            return torch.cat([t1 * c - t2 * s, t2 * c + t1 * s], -1)
        q = norm_rope(s64[:, :nh * d].view(L, nh, d), qw)
        k = norm_rope(s64[:, nh * d:(nh + nkv) * d].view(L, nkv, d), kw)
        v = s64[:, (nh + nkv) * d:].view(L, nkv, d)
        want = _attention_reference(q, k, v, 1 / math.sqrt(d)).reshape(L, nh * d)
        check(f"norm+rope+cache+attention {tag}", _rel(torch.cat(outs), want), tol)
    # sampling
    logits = torch.randn(3, 5000, device=dev)
    logits[1, 77] = logits[1, 4000] = 30.0
    out = torch.empty(3, dtype=torch.int32, device=dev)
    ops.argmax(logits, out)
    want = [int(logits[0].argmax()), 77, int(logits[2].argmax())]
    check("greedy pick (first maximum)", 0.0 if out.tolist() == want else 1.0, 0.0)
    # tensor-core kernels
    a = torch.randn(24, 512, device=dev).to(torch.bfloat16)
    wm = (torch.randn(300, 512, device=dev) / 20).to(torch.bfloat16)
    c = torch.empty(24, 300, dtype=torch.float32, device=dev)
    if ops_tensor.gemm_bf16(a, wm, c, ops.GEMM_STORE_F32):
        torch.cuda.synchronize()
        check("tcgen05 product bf16", _rel(c, a.double() @ wm.double().T), 1e-4)
    else:
        failures.append("tcgen05 product refused")
    # the product of more than 256 tokens (CTA pairs) and a split-K product whose splits add together
    a = torch.randn(300, 512, device=dev).to(torch.bfloat16)
    wm = (torch.randn(640, 512, device=dev) / 20).to(torch.bfloat16)
    c = torch.empty(300, 640, dtype=torch.bfloat16, device=dev)
    if ops_tensor.gemm_bf16(a, wm, c, ops.GEMM_STORE):
        check("tcgen05 product, CTA pairs bf16", _rel(c, a.double() @ wm.double().T), 3e-2)
    else:
        failures.append("tcgen05 pair product refused")
    a = torch.randn(12, 4096, device=dev).to(torch.bfloat16)
    wm = (torch.randn(512, 4096, device=dev) / 60).to(torch.bfloat16)
    x = torch.randn(12, 512, device=dev)
    want = x.double() + a.double() @ wm.double().T
    if ops_tensor.gemm_bf16(a, wm, x, ops.GEMM_ACCUM_F32):
        check("tcgen05 product, split-K bf16", _rel(x, want), 1e-4)
    else:
        failures.append("tcgen05 split-K product refused")
    _attention_tensor_core(dev, check, status)
    _sampler(dev, check)
    torch.cuda.synchronize()
    check("tcgen05 and TMA waits completed", float(ops_tensor.gemm_status(dev)), 0.0)
    check("device status word", float(status.item()), 0.0)
    launched = ops.kernel_counts()
    print("kernels launched:")
    for name in sorted(launched):
        print(f"  {name}: {launched[name]}")
    for name in ("attention_decode_tma_kernel (merge in the cluster)", "attention_prefill_tc_kernel", "gemm_tc_pair_kernel",
                 "gemm_tc_kernel (split-K, splits add together)", "sample_kernel"):
        if launched.get(name, 0) == 0:
            failures.append(f"{name} was never launched")
    print("selftest:", "all ok" if not failures else f"FAILED: {', '.join(failures)}")
    return 0 if not failures else 1


class _Step:
    """The tables of a step for the attention kernels, made by hand: sequences of (cached before, new)
    tokens, the one-token sequences first."""

    def __init__(self, seqs, dev, status):
        from .parts.attention import AttentionPlan, PagedAttention, split_bucket
        mk = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        pos, qs, ctx, tiles, tiles_tc, longest = [], [0], [], [], [], 1
        self.n_decode = sum(1 for _, n in seqs if n == 1)
        for b, (c, n) in enumerate(seqs):
            pos += list(range(c, c + n))
            qs.append(qs[-1] + n)
            ctx.append(c + n)
            if n == 1:
                longest = max(longest, c + 1)
            else:
                tiles += [[b, q0] for q0 in range(0, n, PagedAttention.TILE)]
                tiles_tc += [[b, q0] for q0 in range(0, n, PagedAttention.TILE_TC)]
        self.T, self.device, self.status = qs[-1], dev, status
        self.positions, self.q_start, self.ctx_len, self.seq_slot = mk(pos), mk(qs), mk(ctx), mk(list(range(len(seqs))))
        per = ops_tensor.decode_split()
        self.plan = AttentionPlan(mk(tiles or [[0, 0]]), len(tiles), mk(tiles_tc or [[0, 0]]), len(tiles_tc),
                                  split_bucket((longest + per - 1) // per))
        self._scratch = {}

    def scratch(self, name, numel):
        t = self._scratch.get(name)
        if t is None or t.numel() < numel:
            t = self._scratch[name] = torch.empty(max(numel, 1), dtype=torch.float32, device=self.device)
        return t


def _attention_tensor_core(dev, check, status) -> None:
    """The decode kernel that stages by TMA and merges inside a cluster, and the tcgen05 flash kernel, on
    the reference's self-test geometry and beyond (src/device.rs:776-848, 963-1023): grouped heads 8/2 of
    128, shuffled pages, ragged contexts, a portion over a cached prefix."""
    nh, nkv, d, ps = 8, 2, 128, 16
    seqs = [(16, 1), (599, 1), (1336, 1), (5, 37), (0, 20), (130, 300)]
    lens = [c + n for c, n in seqs]
    need = [(n + ps - 1) // ps for n in lens]
    perm = torch.randperm(sum(need) + 3).tolist()
    table = torch.full((len(seqs), max(need) + 1), -1, dtype=torch.int32)
    kp = torch.full((sum(need) + 3, nkv, ps, d), float("nan"), dtype=torch.bfloat16, device=dev)
    vp = torch.full_like(kp, float("nan"))
    step = _Step(seqs, dev, status)
    qkv = torch.zeros(step.T, (nh + 2 * nkv) * d, dtype=torch.bfloat16, device=dev)
    want, t, k_at = [], 0, 0
    for b, (c, n) in enumerate(seqs):
        L = c + n
        pages = perm[k_at:k_at + need[b]]
        k_at += need[b]
        table[b, :need[b]] = torch.tensor(pages, dtype=torch.int32)
        q = (torch.randn(L, nh, d, device=dev) * 1.5).to(torch.bfloat16)
        k = (torch.randn(L, nkv, d, device=dev) * 1.5).to(torch.bfloat16)
        v = torch.randn(L, nkv, d, device=dev).to(torch.bfloat16)
        pad = need[b] * ps - L
        kp[pages] = torch.cat([k, k.new_zeros(pad, nkv, d)]).view(need[b], ps, nkv, d).transpose(1, 2)
        vp[pages] = torch.cat([v, v.new_zeros(pad, nkv, d)]).view(need[b], ps, nkv, d).transpose(1, 2)
        qkv[t:t + n, :nh * d] = q[c:].reshape(n, nh * d)
        want.append(_attention_reference(q, k, v, 1 / math.sqrt(d))[c:].reshape(n, nh * d))
        t += n
    out = torch.full((step.T, nh * d), float("nan"), dtype=torch.bfloat16, device=dev)

    class Cache:
        k_pool, v_pool, page_size = kp, vp, ps
    ok = ops_tensor.attention_bf16(step, step.plan, qkv, out, Cache, table.to(dev), nh, nkv, d, 0, 1 / math.sqrt(d))
    check("attention over pages, tensor cores bf16", _rel(out, torch.cat(want)) if ok else 1.0, 3e-2)


def _sampler(dev, check) -> None:
    """Temperature sampling: the kernel's pick is the Gumbel-max over the row with the counter-based
    uniforms of the reference's sampler (src/kernels/sampling.cu:30-42, 161-182)."""
    import numpy as np
    from .sampling.params import SamplingParams
    from .sampling.sampler import Sampler, step_seed
    V, T = 5000, 0.7
    logits = torch.randn(4, V, device=dev) * 3
    seeds, steps = [11, 12, 13, 14], [0, 5, 1, 9]
    got = Sampler(dev).sample(logits.clone(), [SamplingParams(temperature=T)] * 4, seeds, steps).tolist()
    m = np.uint64((1 << 64) - 1)

    def mix(x):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & m
        x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & m
        x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & m
        return x ^ (x >> np.uint64(31))
    bad = 0
    with np.errstate(over="ignore"):
        for r in range(4):
            h = mix(np.uint64(step_seed(seeds[r], steps[r])) ^ mix(np.arange(V, dtype=np.uint64) + np.uint64(0x632BE59BD9B4E019)))
            u = ((h >> np.uint64(40)).astype(np.float64) + 0.5) / 16777216.0
            g = logits[r].double().cpu().numpy() / T - np.log(-np.log(u))
            order = np.argsort(-g)
            if got[r] != order[0] and g[order[0]] - g[got[r]] > 1e-4:
                bad += 1
    check("temperature sampling (Gumbel-max)", float(bad), 0.0)
