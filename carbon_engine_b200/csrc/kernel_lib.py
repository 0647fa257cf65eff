"""Loads libcarbon_kernels.so (built on first use) and declares the launchers' C interface.

There is no fallback: if the library cannot be built or loaded, importing an op raises.
"""
from __future__ import annotations

import ctypes
import threading

from . import build

_lib = None
_lock = threading.Lock()

_i, _f, _ll, _p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p

_SIGNATURES = {
    "ce_last_error": (ctypes.c_char_p, []),
    "ce_build_arch": (_i, []),
    "ce_kernel_counts": (_i, [ctypes.c_char_p, _i]),
    "ce_kernel_counts_reset": (None, []),
    "ce_last_kernel": (ctypes.c_char_p, []),
    "ce_set_pdl": (None, [_i]),
    # table, dtype, tokens, x, T, H, V, status, stream
    "ce_embed": (_i, [_p, _i, _p, _p, _i, _i, _i, _p, _p]),
    # x, w, out, out_dtype, rows, R, H, eps, stream
    "ce_rmsnorm": (_i, [_p, _p, _p, _i, _p, _i, _i, _f, _p]),
    # qkv, k_pool, v_pool, dtype, qw, kw, cos, sin, positions, seq_of_token, seq_slot, block_table, status,
    # T, nh, nkv, d, rd, page_size, max_pages, num_pages, max_pos, write_kv, eps, pairing, stream
    "ce_qk_rope_kvwrite": (_i, [_p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p,
                                _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p]),
    "ce_add_residual": (_i, [_p, _p, _i, _ll, _p]),
    "ce_swiglu": (_i, [_p, _p, _i, _i, _i, _p]),
    # q, k_pool, v_pool, out, dtype, positions, seq_of_token, seq_slot, block_table, status,
    # T, nh, nkv, d, q_stride, page_size, max_pages, num_pages, window, scale, stream
    "ce_attention_generic": (_i, [_p, _p, _p, _p, _i, _p, _p, _p, _p, _p,
                                  _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _p]),
    # A, W, C, dtype, M, N, K, lda, ldc, mode, stream
    "ce_gemm_plain": (_i, [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i, _p]),
    "ce_sample": (_i, [_p, _i, _i, _p, _p, _p]),
    "ce_argmax": (_i, [_p, _i, _i, _p, _p]),
    "ce_apply_penalties": (_i, [_p, _i, _p, _i, _p, _p]),
    "ce_scatter_i32": (_i, [_p, _p, _p, _i, _ll, _p]),
}


class KernelError(RuntimeError):
    pass


def kernels() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is None:
            path = build.build_kernels()
            try:
                lib = ctypes.CDLL(path)
            except OSError as exc:
                raise KernelError(f"cannot load the CUDA kernel library {path}: {exc}") from None
            for name, (res, args) in _SIGNATURES.items():
                try:
                    fn = getattr(lib, name)
                except AttributeError:
                    raise KernelError(f"{path} lacks the symbol {name}: rebuild the kernels") from None
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def declare(name: str, restype, argtypes) -> None:
    """Declare a launcher added by a later source file."""
    _SIGNATURES[name] = (restype, argtypes)
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
