"""ctypes loader for ``tile_oracle.c`` (builds it with gcc on first use)."""

from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = _HERE / "_build" / "libtile_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    src = _HERE / "tile_oracle.c"
    if force or not _LIB.exists() or _LIB.stat().st_mtime < src.stat().st_mtime:
        _LIB.parent.mkdir(exist_ok=True)
        # -march=native is avoided here: the library is built on one machine and may be
        # loaded on another (the GPU box) whose host cores differ.
        cmd = ["gcc", "-O3", "-mavx2", "-mfma", "-mf16c", "-fopenmp", "-fPIC", "-std=c11", "-shared",
               "-o", str(_LIB), str(src), "-lm"]
        subprocess.run(cmd, check=True)
    return _LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB.exists() or _LIB.stat().st_mtime < (_HERE / "tile_oracle.c").stat().st_mtime:
            build()
        _lib = ctypes.CDLL(str(_LIB))
    return _lib


def _p(a: np.ndarray | None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.c_void_p)


def contract(desc, srcs, init, out: np.ndarray) -> np.ndarray:
    """Runs the definition-order contraction walker.  ``desc`` is any ctypes structure with the
    layout of ``pmlb_contract_desc``."""
    ptrs = [_p(s) for s in srcs] + [None] * (3 - len(srcs))
    rc = lib().orc_contract(ctypes.byref(desc), ptrs[0], ptrs[1], ptrs[2], _p(init), _p(out))
    assert rc == 0
    return out


def _gemm_args(a, b, b_is_nk):
    a3 = a if a.ndim == 3 else a[None]
    b3 = b if b.ndim == 3 else b[None]
    batch = max(a3.shape[0], b3.shape[0])
    m, k = a3.shape[1], a3.shape[2]
    n = b3.shape[1] if b_is_nk else b3.shape[2]
    sa = 0 if a3.shape[0] == 1 and batch > 1 else m * k
    sb = 0 if b3.shape[0] == 1 and batch > 1 else b3.shape[1] * b3.shape[2]
    return a3, b3, batch, m, n, k, sa, sb


def _call_gemm(fn, a, b, out_dtype, b_is_nk, extra=()):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    a3, b3, batch, m, n, k, sa, sb = _gemm_args(a, b, b_is_nk)
    c = np.empty((batch, m, n), dtype=out_dtype)
    i64 = ctypes.c_int64
    fn(_p(a3), _p(b3), _p(c), *extra, batch, m, n, k, i64(k), i64(b3.shape[2]), i64(n), i64(sa), i64(sb),
       i64(m * n), int(b_is_nk))
    return c if (a.ndim == 3 or b.ndim == 3) else c[0]


def gemm_f32(a, b, b_is_nk=False):
    return _call_gemm(lib().orc_gemm_f32, a.astype(np.float32, copy=False), b.astype(np.float32, copy=False),
                      np.float32, b_is_nk)


def gemm_f32_acc64(a, b, b_is_nk=False):
    return _call_gemm(lib().orc_gemm_f32_acc64, a.astype(np.float32, copy=False),
                      b.astype(np.float32, copy=False), np.float64, b_is_nk)


def gemm_i8_i32(a, b, b_is_nk=False):
    assert a.dtype == np.int8 and b.dtype == np.int8
    return _call_gemm(lib().orc_gemm_i8_i32, a, b, np.int32, b_is_nk)


def gemm_h16_f32(a_bits, b_bits, is_f16, b_is_nk=False):
    """``a_bits`` / ``b_bits`` are uint16 views of bf16 (or f16) data."""
    assert a_bits.dtype == np.uint16 and b_bits.dtype == np.uint16
    a = np.ascontiguousarray(a_bits)
    b = np.ascontiguousarray(b_bits)
    a3, b3, batch, m, n, k, sa, sb = _gemm_args(a, b, b_is_nk)
    c = np.empty((batch, m, n), dtype=np.float32)
    i64 = ctypes.c_int64
    lib().orc_gemm_h16_f32(_p(a3), _p(b3), _p(c), int(is_f16), batch, m, n, k, i64(k), i64(b3.shape[2]), i64(n),
                           i64(sa), i64(sb), i64(m * n), int(b_is_nk))
    return c if (a.ndim == 3 or b.ndim == 3) else c[0]


def conv2d_nhwc_f32(x, f, bias=None, residual=None, stride=(1, 1), pad=(0, 0), dilation=(1, 1), relu=False,
                    out_hw=None):
    x = np.ascontiguousarray(x, dtype=np.float32)
    f = np.ascontiguousarray(f, dtype=np.float32)
    n, h, w, c = x.shape
    r, s, c2, k = f.shape
    assert c == c2
    if out_hw is None:
        p = (h + 2 * pad[0] - dilation[0] * (r - 1) - 1) // stride[0] + 1
        q = (w + 2 * pad[1] - dilation[1] * (s - 1) - 1) // stride[1] + 1
    else:
        p, q = out_hw
    out = np.empty((n, p, q, k), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    res = None if residual is None else np.ascontiguousarray(residual, dtype=np.float32)
    lib().orc_conv2d_nhwc_f32(_p(x), _p(f), _p(b), _p(res), _p(out), n, h, w, c, r, s, k, p, q, stride[0],
                              stride[1], pad[0], pad[1], dilation[0], dilation[1], int(relu))
    return out


_AGG = {"sum": 1, "max": 2, "min": 3}


def pool2d_nhwc_f32(x, agg, window, stride, pad, out_hw, average=False, include_padding=False):
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, h, w, c = x.shape
    p, q = out_hw
    out = np.empty((n, p, q, c), dtype=np.float32)
    lib().orc_pool2d_nhwc_f32(_p(x), _p(out), _AGG[agg], n, h, w, c, window[0], window[1], p, q, stride[0],
                              stride[1], pad[0], pad[1], int(average), int(include_padding))
    return out


def reduce_f32(x, agg):
    """x is [outer, reduce, inner]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    outer, red, inner = x.shape
    out = np.empty((outer, inner), dtype=np.float32)
    i64 = ctypes.c_int64
    lib().orc_reduce_f32(_p(x), _p(out), _AGG[agg], i64(outer), i64(red), i64(inner))
    return out


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_p(x), _p(out), ctypes.c_int64(x.size))
    return out
