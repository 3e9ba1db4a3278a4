"""Gemm and the quantised GEMV — vortx's src/linalg/gemm.rs entry points over the CUDA kernels.

`Gemm.dispatch / dispatch_naive / dispatch_tiled` keep the reference's argument order
(backend, shapes, pass, out, lhs, rhs).  A shape mismatch raises ShapeMismatch (an
AssertionError) where the reference's assert_eq! panics.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib
from .backend import Backend, GpuBuffer, GpuPass
from .shapes import TensorLayoutBuffers


class MatrixMode:
    """src/linalg/gemm.rs:11-32 (unused by dispatch, kept for call sites)."""

    Normal = 0
    Transposed = 1


N = MatrixMode.Normal
T = MatrixMode.Transposed

_KERNEL_NAMES = {0: "none", 1: "naive", 2: "simt_tiled_vec", 3: "tcgen05_tf32", 4: "simt_tiled_generic"}


class Gemm:
    """src/linalg/gemm.rs:34-41.  `from_backend` mirrors khal's Shader derive."""

    def __init__(self, backend: Optional[Backend] = None):
        self.backend = backend

    @classmethod
    def from_backend(cls, backend: Backend) -> "Gemm":
        return cls(backend)

    def _go(self, kind: int, backend: Backend, out, lhs, rhs) -> None:
        o = out.as_tensor_mut()
        l = lhs.as_tensor_ref()
        r = rhs.as_tensor_ref()
        ob, lb, rb = o.raw_buffer(), l.raw_buffer(), r.raw_buffer()
        for b in (ob, lb, rb):
            if b.dtype != np.float32:
                raise TypeError("Gemm takes f32 tensors")
        st = _lib.load().vx_gemm_dispatch(
            backend._ctx, kind,
            ob.ptr, C.byref(o.layout()._c), ob.len(),
            lb.ptr, C.byref(l.layout()._c), lb.len(),
            rb.ptr, C.byref(r.layout()._c), rb.len())
        _lib.check(st)

    def dispatch(self, backend: Backend, shapes: TensorLayoutBuffers, pass_: GpuPass, out, lhs, rhs) -> None:
        """src/linalg/gemm.rs:47-187"""
        self._go(_lib.VX_DISPATCH, backend, out, lhs, rhs)

    def dispatch_naive(self, backend, shapes, pass_, out, lhs, rhs) -> None:
        """src/linalg/gemm.rs:190-246"""
        self._go(_lib.VX_DISPATCH_NAIVE, backend, out, lhs, rhs)

    def dispatch_tiled(self, backend, shapes, pass_, out, lhs, rhs) -> None:
        """src/linalg/gemm.rs:249-305"""
        self._go(_lib.VX_DISPATCH_TILED, backend, out, lhs, rhs)

    def dispatch_tf32(self, backend, shapes, pass_, out, lhs, rhs) -> None:
        """Same checks as dispatch, then the tcgen05 TF32 kernel (no reference counterpart)."""
        self._go(_lib.VX_DISPATCH_TF32, backend, out, lhs, rhs)

    @staticmethod
    def last_kernel(backend: Backend) -> str:
        k = C.c_int32()
        _lib.check(_lib.load().vx_gemm_last_kernel(backend._ctx, C.byref(k)))
        return _KERNEL_NAMES.get(k.value, str(k.value))


class ReduceVariant:
    """src/linalg/reduce.rs:16-30"""

    Min = 2
    Max = 3
    Sum = 0
    Prod = 1
    SqNorm = 4


_DTYPE_CODES = {np.dtype(np.float32): 0, np.dtype(np.uint32): 1, np.dtype(np.int32): 2}


class Reduce:
    """src/linalg/reduce.rs:44-207.  `launch` keeps the reference's argument order; the reference's host
    type takes f32 tensors only, u32 / i32 tensors are accepted here because their kernels exist
    (vortx-shaders/src/linalg/reduce.rs:301-308)."""

    ORDERED, WIDE = 0, 1

    def __init__(self, backend: Optional[Backend] = None, mode: int = 0):
        self.backend = backend
        self.mode = mode

    @classmethod
    def from_backend(cls, backend: Backend) -> "Reduce":
        return cls(backend)

    def launch(self, backend: Backend, shapes, pass_, variant: int, input_, output, mode: Optional[int] = None) -> None:
        i = input_.as_tensor_ref()
        o = output.as_tensor_mut()
        ib, ob = i.raw_buffer(), o.raw_buffer()
        if ib.dtype != ob.dtype or ib.dtype not in _DTYPE_CODES:
            raise TypeError("Reduce takes f32, u32 or i32 tensors of one type")
        shape = i.layout().canonicalize().into_gpu()
        isz = ib.dtype.itemsize
        st = _lib.load().vx_reduce(backend._ctx, variant, _DTYPE_CODES[ib.dtype], self.mode if mode is None else mode,
                                   ib.ptr + i.layout().offset * isz, C.byref(shape), ib.len() - i.layout().offset,
                                   ob.ptr + o.layout().offset * isz)
        _lib.check(st)


class OpAssignVariant:
    """src/linalg/op_assign.rs:12-24"""

    Add, Sub, Mul, Div, Copy = 0, 1, 2, 3, 4


class OpAssign:
    """src/linalg/op_assign.rs:26-143: a op= b with b broadcast to a."""

    @classmethod
    def from_backend(cls, backend: Backend) -> "OpAssign":
        return cls()

    def launch(self, backend: Backend, shapes, pass_, variant: int, a, b, _repeat: int = 0) -> None:
        am, br = a.as_tensor_mut(), b.as_tensor_ref()
        ab, bb = am.raw_buffer(), br.raw_buffer()
        if ab.dtype != np.float32 or bb.dtype != np.float32:
            raise TypeError("OpAssign / Repeat take f32 tensors")
        _lib.check(_lib.load().vx_op_assign_dispatch(backend._ctx, variant, _repeat, ab.ptr, C.byref(am.layout()._c),
                                                     ab.len(), bb.ptr, C.byref(br.layout()._c), bb.len()))


class Repeat:
    """src/linalg/repeat.rs:16-88: tiles `source` into `destination` by wrapping indices."""

    @classmethod
    def from_backend(cls, backend: Backend) -> "Repeat":
        return cls()

    def launch(self, backend: Backend, shapes, pass_, destination, source) -> None:
        OpAssign().launch(backend, shapes, pass_, OpAssignVariant.Copy, destination, source, _repeat=1)


class Contiguous:
    """src/linalg/contiguous.rs:13-129: gathers a strided view of 4-byte elements into a row-major tensor."""

    @classmethod
    def from_backend(cls, backend: Backend) -> "Contiguous":
        return cls()

    def launch(self, backend: Backend, shapes, pass_, out, tensor, offset: Optional[int] = None) -> None:
        o, t = out.as_tensor_mut(), tensor.as_tensor_ref()
        ob, tb = o.raw_buffer(), t.raw_buffer()
        if ob.dtype.itemsize != 4 or tb.dtype.itemsize != 4:
            raise TypeError("Contiguous only supports tensors with 4-bytes elements.")
        if tuple(t.layout().size) != tuple(o.layout().size):
            raise _lib.ShapeMismatch(_lib.VX_ERR_SHAPE, f"{t.layout()} vs {o.layout()}")
        if not o.is_contiguous():
            raise ValueError(f"Output tensor must be contiguous: {o.layout()}.")
        shape = t.layout().canonicalize().into_gpu()
        # with an explicit offset the reference binds the raw buffer and adds the offset in the kernel
        off = t.layout().offset if offset is None else offset
        _lib.check(_lib.load().vx_contiguous(backend._ctx, ob.ptr + o.layout().offset * 4, ob.len() - o.layout().offset,
                                             tb.ptr, C.byref(shape), tb.len(), off))


# --------------------------------------------------------------------- quantised --------

Q8_0 = _lib.VX_Q8_0
Q4_0 = _lib.VX_Q4_0


def quantize(qtype: int, w: np.ndarray) -> np.ndarray:
    """Host quantiser: f32 [rows, cols] -> block stream (uint8)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    lib = _lib.load()
    out = np.empty(rows * (cols // 32) * lib.vx_qblock_bytes(qtype), dtype=np.uint8)
    _lib.check(lib.vx_quantize(qtype, w.ctypes.data, rows, cols, out.ctypes.data))
    return out


def dequantize_host(qtype: int, blocks: np.ndarray, rows: int, cols: int) -> np.ndarray:
    out = np.empty((rows, cols), dtype=np.float32)
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    _lib.check(_lib.load().vx_dequantize_host(qtype, blocks.ctypes.data, rows, cols, out.ctypes.data))
    return out


class QuantizedMatrix:
    """Device-resident Q8_0 / Q4_0 weights (vx_qweights)."""

    def __init__(self, backend: Backend, qtype: int, blocks: np.ndarray, rows: int, cols: int):
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        lib = _lib.load()
        expect = rows * (cols // 32) * lib.vx_qblock_bytes(qtype)
        if blocks.size != expect:
            raise ValueError(f"block stream has {blocks.size} bytes, expected {expect}")
        h = C.c_void_p()
        _lib.check(lib.vx_qweights_upload(backend._ctx, qtype, blocks.ctypes.data, rows, cols, C.byref(h)))
        self.backend, self.qtype, self.rows, self.cols = backend, qtype, rows, cols
        self._h = h

    @classmethod
    def from_f32(cls, backend: Backend, qtype: int, w: np.ndarray) -> "QuantizedMatrix":
        return cls(backend, qtype, quantize(qtype, w), w.shape[0], w.shape[1])

    @classmethod
    def from_device_f32(cls, backend: Backend, qtype: int, w_ptr: int, rows: int, cols: int,
                        row_stride: Optional[int] = None) -> "QuantizedMatrix":
        """Quantises an f32 matrix that already lives on the device (vx_qweights_from_device)."""
        h = C.c_void_p()
        _lib.check(_lib.load().vx_qweights_from_device(backend._ctx, qtype, w_ptr, rows, cols,
                                                       cols if row_stride is None else row_stride, C.byref(h)))
        self = cls.__new__(cls)
        self.backend, self.qtype, self.rows, self.cols = backend, qtype, rows, cols
        self._h = h
        return self

    def stream_bytes(self) -> int:
        return self.rows * (self.cols // 32) * _lib.load().vx_qblock_bytes(self.qtype)

    def device_bytes(self) -> int:
        """Bytes the weights occupy on the device (both planes with their padding)."""
        n = C.c_size_t()
        _lib.check(_lib.load().vx_qweights_info(self._h, None, None, None, C.byref(n)))
        return int(n.value)

    def checksum(self) -> int:
        """vx_qweights_checksum: one read-only pass over the device form; blocks until done."""
        out = self.backend.uninit_buffer(1, dtype=np.uint32)
        _lib.check(_lib.load().vx_qweights_checksum(self.backend._ctx, self._h, out.ptr))
        v = np.zeros(1, np.uint32)
        self.backend.slow_read_buffer(out, v)
        out.free()
        return int(v[0])

    def free(self) -> None:
        if self._h and self.backend._ctx:
            _lib.check(_lib.load().vx_qweights_free(self.backend._ctx, self._h))
        self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def dequantize(self, out: GpuBuffer) -> None:
        if out.len() < self.rows * self.cols:
            raise ValueError("dequantize destination too small")
        _lib.check(_lib.load().vx_dequantize(self.backend._ctx, self._h, out.ptr))


class Gemv:
    """y = W x for block-quantised W; x and y are device vectors (batch of them, contiguous by default)."""

    @classmethod
    def from_backend(cls, backend: Backend) -> "Gemv":
        return cls()

    def dispatch(self, backend: Backend, pass_: Optional[GpuPass], y, w: QuantizedMatrix, x, batch: int = 1,
                 x_stride: Optional[int] = None, y_stride: Optional[int] = None,
                 row0: int = 0, nrows: Optional[int] = None) -> None:
        nrows = w.rows - row0 if nrows is None else nrows
        xs = w.cols if x_stride is None else x_stride
        ys = nrows if y_stride is None else y_stride
        xp, xl = _ptr_len(x)
        yp, yl = _ptr_len(y)
        if xl is not None and batch and (batch - 1) * xs + w.cols > xl:
            raise IndexError("x is shorter than batch * cols")
        if yl is not None and batch and (batch - 1) * ys + nrows > yl:
            raise IndexError("y is shorter than batch * rows")
        _lib.check(_lib.load().vx_gemv_q_rows(backend._ctx, w._h, row0, nrows, xp, xs, yp, ys, batch))

    def dispatch_multi(self, backend: Backend, pass_: Optional[GpuPass], ys, ws, x, batch: int = 1,
                       x_stride: Optional[int] = None, y_stride: Optional[int] = None) -> None:
        """Several matrices (one type, one column count) times the same vectors in one pass (vx_gemv_q_multi):
        ys[i] = ws[i] x.  y_stride (elements between the vectors of every y) defaults to the largest row count."""
        n = len(ws)
        if n != len(ys):
            raise ValueError("as many outputs as matrices")
        if n == 0:
            return
        xs = ws[0].cols if x_stride is None else x_stride
        yst = max(w.rows for w in ws) if y_stride is None else y_stride
        xp, xl = _ptr_len(x)
        if xl is not None and batch and (batch - 1) * xs + ws[0].cols > xl:
            raise IndexError("x is shorter than batch * cols")
        yps = []
        for w, y in zip(ws, ys):
            yp, yl = _ptr_len(y)
            if yl is not None and batch and (batch - 1) * yst + w.rows > yl:
                raise IndexError("a y is shorter than batch * rows")
            yps.append(yp)
        wa = (C.c_void_p * n)(*[w._h.value if hasattr(w._h, "value") else w._h for w in ws])
        ya = (C.c_void_p * n)(*yps)
        _lib.check(_lib.load().vx_gemv_q_multi(backend._ctx, wa, n, xp, xs, ya, yst, batch))


class GemvBatch:
    """A fixed list of GEMVs run by ONE persistent launch (vx_gemv_batch): one weight stream, one prologue.

    Each entry is a dict: w (QuantizedMatrix), and optionally row0, nrows, x (plain device pointer), x_xvec
    (exchange vector to read x from), y (plain rows), y_xvec (exchange vector to write), peers (the same
    vector on the peer GPUs), y_row0, y_stride, peer_y (peer buffers that receive the plain rows as well),
    x_seg_len / x_seg_stride / x_seg_first (x is a window: that many elements, from that offset, out of every
    stride of x_xvec).  Entries may depend on each other only through exchange
    vectors.  Pointers are captured at construction."""

    def __init__(self, backend: Backend, entries):
        lib = _lib.load()
        n = len(entries)
        arr = (_lib.VxGemvOp * n)()
        self._keep = []
        for i, e in enumerate(entries):
            w = e["w"]
            row0 = e.get("row0", 0)
            nrows = e.get("nrows")
            peers = list(e.get("peers") or [])
            pa = (C.c_void_p * max(1, len(peers)))(*peers)
            plain = list(e.get("peer_y") or [])
            pp = (C.c_void_p * max(1, len(plain)))(*plain)
            self._keep.append((w, pa, pp))
            arr[i].peer_y = pp
            arr[i].n_peer_y = len(plain)
            arr[i].x_seg_len = e.get("x_seg_len", 0)
            arr[i].x_seg_stride = e.get("x_seg_stride", 0)
            arr[i].x_seg_first = e.get("x_seg_first", 0)
            arr[i].w = w._h
            arr[i].row0 = row0
            arr[i].nrows = w.rows - row0 if nrows is None else nrows
            arr[i].x_xvec = e.get("x_xvec") or None
            arr[i].x = e.get("x") or None
            arr[i].y = e.get("y") or None
            arr[i].y_xvec = e.get("y_xvec") or None
            arr[i].peer_y_xvec = pa
            arr[i].n_peers = len(peers)
            arr[i].y_row0 = e.get("y_row0", 0)
            arr[i].y_stride = e.get("y_stride", 1)
        h = C.c_void_p()
        _lib.check(lib.vx_gemv_batch_create(backend._ctx, arr, n, C.byref(h)))
        self.backend, self._h, self.n = backend, h, n

    def launch(self) -> None:
        _lib.check(_lib.load().vx_gemv_batch_launch(self.backend._ctx, self._h))

    def free(self) -> None:
        if self._h and self.backend._ctx:
            _lib.check(_lib.load().vx_gemv_batch_free(self.backend._ctx, self._h))
        self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class HostStages:
    """A step with HOST buffers cut into stages whose copies hide behind the kernels (vx_gemv_batch_run_host).

    Each stage is a dict: batch (GemvBatch) and optionally up = (device_ptr, host_ptr, bytes), down =
    (host_ptr, host_pitch, device_ptr, device_pitch, width_bytes, rows), barrier = (flag pointers of every rank,
    rank): a peer barrier between the list and the copy down.  Host pointers should be page-locked.  Pointers
    are captured at construction; `run()` returns when every stage's results are in host memory.  With
    `recorded=True` the step is recorded once as a CUDA graph (vx_host_pipeline: the step runs once at
    construction, the host buffers must be page-locked) and `run()` replays it with one runtime call."""

    def __init__(self, backend: Backend, stages, recorded: bool = False):
        n = len(stages)
        self._arr = (_lib.VxHostStage * max(1, n))()
        self._keep = []
        for i, s in enumerate(stages):
            a = self._arr[i]
            a.batch = s["batch"]._h
            self._keep.append(s["batch"])
            up = s.get("up")
            if up:
                a.up_device, a.up_host, a.up_bytes = up
            down = s.get("down")
            if down:
                (a.down_host, a.down_host_pitch, a.down_device, a.down_device_pitch, a.down_width_bytes,
                 a.down_rows) = down
            bar = s.get("barrier")
            if bar:
                flags, rank = bar
                fa = (C.c_void_p * len(flags))(*flags)
                self._keep.append(fa)
                a.barrier_flags, a.world, a.rank = fa, len(flags), rank
        self.backend, self.n = backend, n
        self._pipe = None
        if recorded:
            h = C.c_void_p()
            _lib.check(_lib.load().vx_host_pipeline_create(backend._ctx, self._arr, n, C.byref(h)))
            self._pipe = h

    def run(self) -> None:
        lib = _lib.load()
        if self._pipe:
            _lib.check(lib.vx_host_pipeline_run(self._pipe))
        else:
            _lib.check(lib.vx_gemv_batch_run_host(self.backend._ctx, self._arr, self.n))

    def free(self) -> None:
        if self._pipe and self.backend._ctx:
            _lib.check(_lib.load().vx_host_pipeline_free(self._pipe))
        self._pipe = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _ptr_len(t):
    """Device pointer (with view offset) and remaining length of a Tensor / view / buffer / raw int."""
    if isinstance(t, int):
        return t, None
    if isinstance(t, GpuBuffer):
        return t.ptr, t.len()
    if hasattr(t, "as_tensor_ref"):
        v = t.as_tensor_ref()
        sl = v.buffer()
        return sl.ptr, sl.len()
    raise TypeError(f"cannot take a device pointer from {type(t)!r}")
