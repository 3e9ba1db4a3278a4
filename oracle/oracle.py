"""ctypes front end of libvortx_oracle.so (see vortx_oracle.h for what each function restates).

PARITY STATUS: the f32 GEMM restatement is pinned only by replaying the property the
reference's own test checks (src/linalg/gemm.rs:365-444); the reference holds no golden
vectors.  The Q8_0 / Q4_0 functions are PARITY UNPINNED: the reference has no such code.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_SO = _DIR / "libvortx_oracle.so"

__all__ = [
    "Shape", "build", "lib", "shape_contiguous", "gemm_naive", "gemm_tiled", "gemm_dispatch", "gemm_f64",
    "quantize", "dequantize", "gemv", "gemv_f64", "f32_to_f16", "f16_to_f32", "reduce", "hardware_threads",
    "Q8_0", "Q4_0", "BLOCK_BYTES", "op_assign", "contiguous", "repeat",
]

Q8_0, Q4_0 = 0, 1
BLOCK_BYTES = {Q8_0: 34, Q4_0: 18}


class Shape(C.Structure):
    """vortx-shaders/src/linalg/shape.rs:9-29"""

    _fields_ = [(n, C.c_uint32) for n in
                ("n", "c", "h", "w", "n_stride", "c_stride", "h_stride", "w_stride")]

    @classmethod
    def of(cls, sizes, strides):
        return cls(*sizes, *strides)


def build(force: bool = False) -> Path:
    """Compiles the oracle with the Makefile beside it (g++, -ffp-contract=off)."""
    src_m = max((_DIR / f).stat().st_mtime for f in ("vortx_oracle.cpp", "vortx_oracle.h", "Makefile"))
    if force or not _SO.exists() or _SO.stat().st_mtime < src_m:
        subprocess.run(["make", "-C", str(_DIR), "-B", "libvortx_oracle.so"], check=True,
                       capture_output=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_SO))
        P, S = C.c_void_p, C.POINTER(Shape)
        L.orc_shape_it.restype = C.c_uint32
        L.orc_shape_it.argtypes = [S] + [C.c_uint32] * 4
        L.orc_gemm_naive.argtypes = [P, P, P, S, S, S]
        L.orc_gemm_tiled.argtypes = [P, P, P, S, S, S, C.c_int]
        L.orc_gemm_dispatch.argtypes = [P, P, P, S, S, S, C.c_int]
        L.orc_gemm_f64.argtypes = [P, P, P, C.c_uint32, C.c_uint32, C.c_uint32]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        for n in ("orc_quantize_q8_0", "orc_quantize_q4_0"):
            getattr(L, n).argtypes = [P, C.c_size_t, C.c_size_t, P]
        for n in ("orc_dequantize_q8_0", "orc_dequantize_q4_0"):
            getattr(L, n).argtypes = [P, C.c_size_t, C.c_size_t, P]
        for n in ("orc_gemv_q8_0", "orc_gemv_q4_0"):
            getattr(L, n).argtypes = [P, C.c_size_t, C.c_size_t, P, C.c_size_t, P, C.c_int]
        for n in ("orc_gemv_q8_0_f64", "orc_gemv_q4_0_f64"):
            getattr(L, n).argtypes = [P, C.c_size_t, C.c_size_t, P, C.c_size_t, P, P]
        L.orc_reduce_f32.restype = C.c_float
        L.orc_reduce_f32.argtypes = [P, S, C.c_int]
        L.orc_reduce_u32.restype = C.c_uint32
        L.orc_reduce_u32.argtypes = [P, S, C.c_int]
        L.orc_reduce_i32.restype = C.c_int32
        L.orc_reduce_i32.argtypes = [P, S, C.c_int]
        L.orc_op_assign.argtypes = [C.c_int, P, S, P, S, C.c_uint32, C.c_uint32]
        L.orc_contiguous.argtypes = [P, P, S, C.c_uint32]
        L.orc_repeat.argtypes = [P, S, P, S]
        L.orc_hardware_threads.restype = C.c_int
        _lib = L
    return _lib


def hardware_threads() -> int:
    return lib().orc_hardware_threads()


def shape_contiguous(n, c, h, w) -> Shape:
    return Shape(n, c, h, w, c * h * w, h * w, w, 1)


def _span(s: Shape) -> int:
    if 0 in (s.n, s.c, s.h, s.w):
        return 0
    return ((s.n - 1) * s.n_stride + (s.c - 1) * s.c_stride + (s.h - 1) * s.h_stride
            + (s.w - 1) * s.w_stride + 1)


def _gemm(fn, out, lhs, rhs, so, sl, sr, *extra):
    for a in (out, lhs, rhs):
        assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    assert _span(so) <= out.size and _span(sl) <= max(lhs.size, 1) and _span(sr) <= max(rhs.size, 1)
    fn(out.ctypes.data, lhs.ctypes.data, rhs.ctypes.data, C.byref(so), C.byref(sl), C.byref(sr), *extra)
    return out


def gemm_naive(out, lhs, rhs, so, sl, sr):
    """Flat f32 buffers indexed through the three shapes; writes into `out`."""
    return _gemm(lib().orc_gemm_naive, out, lhs, rhs, so, sl, sr)


def gemm_tiled(out, lhs, rhs, so, sl, sr, nthreads=1):
    return _gemm(lib().orc_gemm_tiled, out, lhs, rhs, so, sl, sr, nthreads)


def gemm_dispatch(out, lhs, rhs, so, sl, sr, nthreads=1):
    return _gemm(lib().orc_gemm_dispatch, out, lhs, rhs, so, sl, sr, nthreads)


def gemm_f64(lhs, rhs):
    lhs = np.ascontiguousarray(lhs, np.float32)
    rhs = np.ascontiguousarray(rhs, np.float32)
    m, k = lhs.shape
    k2, n = rhs.shape
    assert k == k2
    out = np.empty((m, n), np.float64)
    lib().orc_gemm_f64(out.ctypes.data, lhs.ctypes.data, rhs.ctypes.data, m, n, k)
    return out


def f32_to_f16(f: float) -> int:
    return lib().orc_f32_to_f16(f)


def f16_to_f32(h: int) -> float:
    return lib().orc_f16_to_f32(h)


def quantize(qtype, w):
    w = np.ascontiguousarray(w, np.float32)
    rows, cols = w.shape
    assert cols % 32 == 0
    out = np.empty(rows * (cols // 32) * BLOCK_BYTES[qtype], np.uint8)
    fn = lib().orc_quantize_q8_0 if qtype == Q8_0 else lib().orc_quantize_q4_0
    fn(w.ctypes.data, rows, cols, out.ctypes.data)
    return out


def dequantize(qtype, blocks, rows, cols):
    blocks = np.ascontiguousarray(blocks, np.uint8)
    assert blocks.size == rows * (cols // 32) * BLOCK_BYTES[qtype]
    out = np.empty((rows, cols), np.float32)
    fn = lib().orc_dequantize_q8_0 if qtype == Q8_0 else lib().orc_dequantize_q4_0
    fn(blocks.ctypes.data, rows, cols, out.ctypes.data)
    return out


def gemv(qtype, blocks, rows, cols, x, nthreads=1):
    """x: [batch, cols] (or [cols]); returns y [batch, rows] f32, summed in the stated f32 order."""
    blocks = np.ascontiguousarray(blocks, np.uint8)
    x2 = np.ascontiguousarray(np.atleast_2d(x), np.float32)
    assert x2.shape[1] == cols and blocks.size == rows * (cols // 32) * BLOCK_BYTES[qtype]
    y = np.empty((x2.shape[0], rows), np.float32)
    fn = lib().orc_gemv_q8_0 if qtype == Q8_0 else lib().orc_gemv_q4_0
    fn(blocks.ctypes.data, rows, cols, x2.ctypes.data, x2.shape[0], y.ctypes.data, nthreads)
    return y if np.ndim(x) == 2 else y[0]


def gemv_f64(qtype, blocks, rows, cols, x):
    """Returns (y, absdot) in f64: the exact-ish product and sum |w x| per output."""
    blocks = np.ascontiguousarray(blocks, np.uint8)
    x2 = np.ascontiguousarray(np.atleast_2d(x), np.float32)
    assert x2.shape[1] == cols and blocks.size == rows * (cols // 32) * BLOCK_BYTES[qtype]
    y = np.empty((x2.shape[0], rows), np.float64)
    a = np.empty((x2.shape[0], rows), np.float64)
    fn = lib().orc_gemv_q8_0_f64 if qtype == Q8_0 else lib().orc_gemv_q4_0_f64
    fn(blocks.ctypes.data, rows, cols, x2.ctypes.data, x2.shape[0], y.ctypes.data, a.ctypes.data)
    return (y, a) if np.ndim(x) == 2 else (y[0], a[0])


_REDUCE_OPS = {"sum": 0, "prod": 1, "min": 2, "max": 3, "sqnorm": 4}


def reduce(v, op: str, stride: int = 1, length=None):
    """128-lane workgroup reduction of v[0], v[stride], ... (length elements)."""
    v = np.ascontiguousarray(v)
    n = (v.size + stride - 1) // stride if length is None else length
    s = Shape(1, 1, 1, n, 1, 1, 1, stride)
    code = _REDUCE_OPS[op]
    if v.dtype == np.float32:
        return np.float32(lib().orc_reduce_f32(v.ctypes.data, C.byref(s), code))
    if v.dtype == np.uint32:
        return np.uint32(lib().orc_reduce_u32(v.ctypes.data, C.byref(s), code))
    if v.dtype == np.int32:
        return np.int32(lib().orc_reduce_i32(v.ctypes.data, C.byref(s), code))
    raise TypeError(v.dtype)


def op_assign(op: int, a, sa: Shape, b, sb: Shape, off_a: int = 0, off_b: int = 0):
    """In place on the flat f32 buffer `a`; op: 0 add, 1 sub, 2 mul, 3 div, 4 copy."""
    assert a.dtype == np.float32 and b.dtype == np.float32 and a.flags["C_CONTIGUOUS"] and b.flags["C_CONTIGUOUS"]
    lib().orc_op_assign(op, a.ctypes.data, C.byref(sa), b.ctypes.data, C.byref(sb), off_a, off_b)
    return a


def contiguous(src, s: Shape, offset: int = 0):
    """Row-major gather of the 4-byte elements that `s` addresses in the flat buffer `src`."""
    src = np.ascontiguousarray(src)
    assert src.dtype.itemsize == 4
    out = np.empty(s.n * s.c * s.h * s.w, src.dtype)
    lib().orc_contiguous(out.ctypes.data, src.ctypes.data, C.byref(s), offset)
    return out


def repeat(result, sr: Shape, source, ss: Shape):
    assert result.dtype == np.float32 and source.dtype == np.float32
    lib().orc_repeat(result.ctypes.data, C.byref(sr), source.ctypes.data, C.byref(ss))
    return result
