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
        check("tcgen05 waits completed", float(ops_tensor.gemm_status(dev)), 0.0)
    else:
        failures.append("tcgen05 product refused")
    torch.cuda.synchronize()
    check("device status word", float(status.item()), 0.0)
    print("selftest:", "all ok" if not failures else f"FAILED: {', '.join(failures)}")
    return 0 if not failures else 1
