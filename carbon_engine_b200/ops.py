"""Thin, checked Python wrappers around the CUDA launchers of libcarbon_kernels.so.

Each wrapper takes torch tensors that live on the GPU, validates dtype and layout, and launches on
the current CUDA stream.  Nothing here computes on the CPU and nothing falls back to a library:
if the kernel library is missing or refuses a size, the call raises.
"""
from __future__ import annotations

import struct
from typing import Optional, Sequence

import torch

from .csrc.kernel_lib import KernelError, kernels

F32, BF16 = 0, 1
GEMM_STORE, GEMM_STORE_F32, GEMM_ACCUM_F32, GEMM_SWIGLU = 0, 1, 2, 3
ROPE_PAIRINGS = {"half": 0, "interleaved": 1}


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {dt} (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream() -> int:
    """The current stream's handle (of the current device), the short way: this runs at every launch."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


def _need(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


_launches = 0


def launch_count() -> int:
    """Kernels launched through this module so far (replays of captured graphs included)."""
    return _launches


def add_launches(n: int) -> None:
    global _launches
    _launches += n


class KernelProfile:
    """Times every launch that goes through this module with CUDA events, one after each launch on the
    launching stream, while dependent launches are switched off so that kernels do not overlap: the time
    between two events is then the time of the kernel between them (plus its launch gap).  ``work`` that a
    caller notes before a launch (bytes it has to move, floating-point operations) is kept with it, so that
    :meth:`table` can set each kernel against the memory or arithmetic peak.  For measurement only: a
    profiled step is slower than a served one."""

    def __init__(self):
        self.records = []            # (kernel name, event after it, bytes, flops)
        self._work = (0, 0)
        self._start = None

    def __enter__(self):
        global _profile
        import torch
        self._pdl_before = _pdl_on
        set_dependent_launches(False)
        torch.cuda.synchronize()
        self._start = torch.cuda.Event(enable_timing=True)
        self._start.record()
        _profile = self
        return self

    def __exit__(self, *exc):
        global _profile
        import torch
        _profile = None
        torch.cuda.synchronize()
        set_dependent_launches(self._pdl_before)

    def note_work(self, nbytes: int, flops: int) -> None:
        self._work = (int(nbytes), int(flops))

    def mark(self) -> None:
        """The next launch's time counts from here (the step function marks the point where a step's host
        work and upload are done, so that they are not charged to the step's first kernel)."""
        import torch
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.records.append((None, ev, 0, 0))

    def _launched(self, n: int) -> None:
        import torch
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        name = kernels().ce_last_kernel().decode() or "?"
        self.records.append((name if n == 1 else f"{name} (+{n - 1})", ev, *self._work))
        self._work = (0, 0)

    def table(self, hbm_gbs: float, tflops: float, repeats: int = 1):
        """Rows (name, launches, microseconds per repeat, share, GB/s, TFLOP/s, fraction of the nearer
        peak) by kernel name, slowest first."""
        agg, prev, total = {}, self._start, 0.0
        for name, ev, nbytes, flops in self.records:
            us = prev.elapsed_time(ev) * 1e3
            prev = ev
            if name is None:             # a mark: what came before it is nobody's
                continue
            a = agg.setdefault(name, [0, 0.0, 0, 0])
            a[0] += 1; a[1] += us; a[2] += nbytes; a[3] += flops
            total += us
        rows = []
        for name, (n, us, nbytes, flops) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
            gbs = nbytes / us / 1e3 if us > 0 else 0.0
            tf = flops / us / 1e6 if us > 0 else 0.0
            frac = max(gbs / hbm_gbs, tf / tflops) if (nbytes or flops) else None
            rows.append({"kernel": name, "launches": n // repeats, "us": round(us / repeats, 1), "share": round(us / total, 4),
                         "gb_s": round(gbs, 1), "tflop_s": round(tf, 1), "frac_of_peak": None if frac is None else round(frac, 3)})
        return rows, total / repeats


_profile: Optional[KernelProfile] = None


def profiling() -> Optional[KernelProfile]:
    return _profile


def _ok(code: int, n: int = 1) -> None:
    global _launches
    if code != 0:
        raise KernelError(kernels().ce_last_error().decode())
    _launches += n
    if _profile is not None:
        _profile._launched(n)


_pdl_on = True


def set_dependent_launches(on: bool) -> None:
    """Whether kernels launched from now on may start while the kernel before them still runs (programmatic
    dependent launch).  The step function turns it off for steps of many tokens, see ``ModelRunner.step``."""
    global _pdl_on
    if bool(on) != _pdl_on:
        kernels().ce_set_pdl(1 if on else 0)
        _pdl_on = bool(on)


def kernel_counts() -> dict:
    """Launches so far by kernel name (a launch captured in a CUDA graph counts once, at capture): shows
    WHICH kernel took each shape."""
    import ctypes
    k = kernels()
    need = k.ce_kernel_counts(None, 0)
    buf = ctypes.create_string_buffer(need + 64)
    k.ce_kernel_counts(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, _, n = line.rpartition("=")
        out[name] = int(n)
    return out


def reset_kernel_counts() -> None:
    kernels().ce_kernel_counts_reset()


def embed(table: torch.Tensor, tokens: torch.Tensor, x: torch.Tensor, status: torch.Tensor) -> None:
    """x[t, :] = table[tokens[t], :] as float32."""
    _need(table, "table"); _need(tokens, "tokens", torch.int32); _need(x, "x", torch.float32)
    T, H = x.shape
    _ok(kernels().ce_embed(_ptr(table), dtype_code(table.dtype), _ptr(tokens), _ptr(x), T, H, table.shape[0],
                           _ptr(status), _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight; x float32, out float32 or bfloat16."""
    _need(x, "x", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    R, H = out.shape
    if x.shape[1] != H or weight.numel() != H:
        raise KernelError(f"rmsnorm: widths differ: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    _ok(kernels().ce_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), dtype_code(out.dtype), _ptr(rows), R, H, float(eps),
                             _stream()))


def qk_rope_kvwrite(qkv, k_pool, v_pool, q_weight, k_weight, cos, sin, positions, seq_of_token, seq_slot,
                    block_table, status, nh: int, nkv: int, d: int, rotary_dim: int, page_size: int,
                    eps: float, write_kv: bool = True, pairing: str = "half") -> None:
    """Per-head q/k RMSNorm, rotation, and the write of K and V into the pages.  ``pairing``: which elements
    of a head turn together, "half" (i with i + rotary_dim/2) or "interleaved" (2i with 2i + 1)."""
    _need(qkv, "qkv")
    if pairing not in ROPE_PAIRINGS:
        raise KernelError(f"qk_rope_kvwrite: unknown pairing '{pairing}' (half, interleaved)")
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * d:
        raise KernelError(f"qk_rope_kvwrite: qkv width {qkv.shape[1]} != (nh + 2 nkv) d = {(nh + 2 * nkv) * d}")
    for name, t in (("q_weight", q_weight), ("k_weight", k_weight), ("cos", cos), ("sin", sin)):
        if t is not None:
            _need(t, name, torch.float32)
    max_pos = cos.shape[0] if cos is not None else 0
    if cos is not None and cos.shape[1] != rotary_dim // 2:
        raise KernelError("qk_rope_kvwrite: rotary table width is not rotary_dim / 2")
    if write_kv:
        _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype)
        if tuple(k_pool.shape[1:]) != (nkv, page_size, d):
            raise KernelError(f"qk_rope_kvwrite: pool shape {tuple(k_pool.shape)} is not [pages, {nkv}, {page_size}, {d}]")
    num_pages = k_pool.shape[0] if k_pool is not None else 0
    max_pages = block_table.shape[1] if block_table is not None else 0
    _ok(kernels().ce_qk_rope_kvwrite(
        _ptr(qkv), _ptr(k_pool), _ptr(v_pool), dtype_code(qkv.dtype), _ptr(q_weight), _ptr(k_weight), _ptr(cos),
        _ptr(sin), _ptr(positions), _ptr(seq_of_token), _ptr(seq_slot), _ptr(block_table), _ptr(status),
        T, nh, nkv, d, rotary_dim, page_size, max_pages, num_pages, max_pos, 1 if write_kv else 0, float(eps),
        ROPE_PAIRINGS[pairing], _stream()))


def add_residual(x: torch.Tensor, delta: torch.Tensor) -> None:
    _need(x, "x", torch.float32); _need(delta, "delta")
    if x.numel() != delta.numel():
        raise KernelError("add_residual: sizes differ")
    _ok(kernels().ce_add_residual(_ptr(x), _ptr(delta), dtype_code(delta.dtype), x.numel(), _stream()))


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    T, I = out.shape
    if gate_up.shape != (T, 2 * I):
        raise KernelError("swiglu: gate_up must be [T, 2I]")
    _ok(kernels().ce_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), T, I, _stream()))


def attention_generic(q, q_stride: int, k_pool, v_pool, out, positions, seq_of_token, seq_slot, block_table,
                      status, nh: int, nkv: int, d: int, page_size: int, window: int, scale: float,
                      T: Optional[int] = None) -> None:
    _need(k_pool, "k_pool"); _need(v_pool, "v_pool", k_pool.dtype); _need(out, "out", k_pool.dtype)
    if q.dtype != k_pool.dtype:
        raise KernelError("attention: q and the cache differ in dtype")
    T = out.shape[0] if T is None else T
    _ok(kernels().ce_attention_generic(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(out), dtype_code(out.dtype), _ptr(positions), _ptr(seq_of_token),
        _ptr(seq_slot), _ptr(block_table), _ptr(status), T, nh, nkv, d, q_stride, page_size, block_table.shape[1],
        k_pool.shape[0], int(window), float(scale), _stream()))


def gemm_plain(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, mode: int) -> None:
    """c = a @ w.T with float32 FMA arithmetic; see csrc/kernels/gemm_plain.cu for the epilogues."""
    _need(w, "w", a.dtype); _need(c, "c")
    if a.stride(-1) != 1 or c.stride(-1) != 1:
        raise KernelError("gemm_plain: rows must be contiguous")
    M, K = a.shape
    N = c.shape[1]
    rows = 2 * N if mode == GEMM_SWIGLU else N
    if w.shape != (rows, K) or c.shape[0] != M:
        raise KernelError(f"gemm_plain: shapes a {tuple(a.shape)}, w {tuple(w.shape)}, c {tuple(c.shape)} do not fit")
    want = torch.float32 if mode in (GEMM_STORE_F32, GEMM_ACCUM_F32) else a.dtype
    if c.dtype != want:
        raise KernelError(f"gemm_plain: output must be {want}")
    _ok(kernels().ce_gemm_plain(_ptr(a), _ptr(w), _ptr(c), dtype_code(a.dtype), M, N, K, a.stride(0), c.stride(0),
                                mode, _stream()))


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    R, V = logits.shape
    _ok(kernels().ce_argmax(_ptr(logits), R, V, _ptr(out), _stream()))


SAMPLE_ROW = struct.Struct("<fffiQ")     # temperature, top_p, min_p, top_k, seed


def pack_sample_rows(rows: Sequence[tuple]) -> bytes:
    return b"".join(SAMPLE_ROW.pack(float(t), float(p), float(m), int(k), int(s) & 0xFFFFFFFFFFFFFFFF)
                    for (t, p, m, k, s) in rows)


def sample(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor) -> None:
    """params: uint8 [rows, 24] holding SAMPLE_ROW records."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32); _need(params, "params", torch.uint8)
    R, V = logits.shape
    if params.numel() != R * SAMPLE_ROW.size:
        raise KernelError("sample: params must hold one 24-byte record per row")
    _ok(kernels().ce_sample(_ptr(logits), R, V, _ptr(params), _ptr(out), _stream()))


def apply_penalties(logits: torch.Tensor, entries: torch.Tensor, row_params: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32); _need(entries, "entries", torch.int32)
    _need(row_params, "row_params", torch.float32)
    _ok(kernels().ce_apply_penalties(_ptr(logits), logits.shape[1], _ptr(entries), entries.shape[0],
                                     _ptr(row_params), _stream()))


def scatter_i32(dst: torch.Tensor, idx: torch.Tensor, val: torch.Tensor) -> None:
    """dst.view(-1)[idx[i]] = val[i]"""
    _need(dst, "dst", torch.int32); _need(idx, "idx", torch.int32); _need(val, "val", torch.int32)
    _ok(kernels().ce_scatter_i32(_ptr(dst), _ptr(idx), _ptr(val), idx.numel(), dst.numel(), _stream()))
