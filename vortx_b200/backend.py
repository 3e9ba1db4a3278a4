"""Backend, buffers, encoder and pass — the slice of khal's surface that vortx's matmul
path touches (src/tensor/tensor_impl.rs:6-9, src/linalg/gemm.rs:397-426), served by the
CUDA context of libvortx_b200.

Work is ordered on the context's stream the moment it is recorded, so `submit` has nothing
left to do and `synchronize` is the only blocking call besides `slow_read_buffer`.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib


class BufferUsages:
    """khal::BufferUsages bit flags; kept for call-site compatibility (CUDA memory has no usage classes)."""

    STORAGE = 1
    COPY_SRC = 2
    COPY_DST = 4
    UNIFORM = 8


class GpuBuffer:
    """A device allocation of `len` elements of `dtype` (khal's GpuBuffer<T>); freed on drop."""

    def __init__(self, backend: "Backend", ptr: int, length: int, dtype, usage: int = BufferUsages.STORAGE,
                 owned: bool = True):
        self.backend = backend
        self.ptr = ptr
        self._len = length
        self.dtype = np.dtype(dtype)
        self._usage = usage
        self._owned = owned

    def len(self) -> int:
        return self._len

    def __len__(self):
        return self._len

    def usage(self) -> int:
        return self._usage

    def slice(self, start: int = 0) -> "GpuBufferSlice":
        if start > self._len:
            raise IndexError(f"slice start {start} beyond buffer of {self._len} elements")
        return GpuBufferSlice(self, start)

    slice_mut = slice

    def as_slice(self) -> "GpuBufferSlice":
        return GpuBufferSlice(self, 0)

    def free(self) -> None:
        if self._owned and self.ptr and self.backend._ctx:
            _lib.check(_lib.load().vx_free(self.backend._ctx, self.ptr))
        self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class GpuBufferSlice:
    """buffer.slice(offset..): a base pointer advanced by `start` elements."""

    def __init__(self, buffer: GpuBuffer, start: int):
        self.buffer = buffer
        self.start = start

    @property
    def ptr(self) -> int:
        return self.buffer.ptr + self.start * self.buffer.dtype.itemsize

    def len(self) -> int:
        return self.buffer.len() - self.start


class GpuPass:
    """encoder.begin_pass(label, None) — a label only; kernels go straight to the stream."""

    def __init__(self, encoder: "GpuEncoder", label: str):
        self.encoder = encoder
        self.label = label


class GpuEncoder:
    def __init__(self, backend: "Backend"):
        self.backend = backend

    def begin_pass(self, label: str, timestamps=None) -> GpuPass:
        return GpuPass(self, label)

    def copy_buffer_to_buffer(self, src: GpuBuffer, src_offset: int, dst: GpuBuffer, dst_offset: int,
                              length: int) -> None:
        """src/tensor/tensor_impl.rs:207-213 — offsets and length in elements."""
        if src.dtype != dst.dtype:
            raise TypeError("copy_buffer_to_buffer between different element types")
        if src_offset + length > src.len() or dst_offset + length > dst.len():
            raise IndexError("copy_buffer_to_buffer range out of bounds")
        isz = src.dtype.itemsize
        _lib.check(_lib.load().vx_copy(self.backend._ctx, dst.ptr + dst_offset * isz,
                                       src.ptr + src_offset * isz, length * isz))


class Backend:
    """GpuBackend::Cuda(Cuda::new(device)) — src/linalg/gemm.rs:353.

    `stream` (a raw cudaStream_t value) makes the context record onto a stream the caller
    owns, e.g. torch.cuda.current_stream().cuda_stream.
    """

    def __init__(self, device: int = 0, stream: Optional[int] = None):
        lib = _lib.load()
        ctx = C.c_void_p()
        if stream is None:
            _lib.check(lib.vx_context_create(device, C.byref(ctx)))
        else:
            _lib.check(lib.vx_context_create_on_stream(device, C.c_void_p(stream), C.byref(ctx)))
        self._ctx = ctx
        self.device = device

    # -- lifetime ---------------------------------------------------------------------
    def close(self) -> None:
        if self._ctx:
            _lib.load().vx_context_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- recording ----------------------------------------------------------------------
    def begin_encoding(self) -> GpuEncoder:
        return GpuEncoder(self)

    def submit(self, encoder: GpuEncoder) -> None:
        return None

    def synchronize(self) -> None:
        _lib.check(_lib.load().vx_synchronize(self._ctx))

    @property
    def stream(self) -> int:
        s = C.c_void_p()
        _lib.check(_lib.load().vx_context_stream(self._ctx, C.byref(s)))
        return s.value or 0

    def launch_count(self) -> int:
        n = C.c_uint64()
        _lib.check(_lib.load().vx_context_launch_count(self._ctx, C.byref(n)))
        return n.value

    def set_option(self, key: str, value: int) -> None:
        _lib.check(_lib.load().vx_set_option(self._ctx, key.encode(), value))

    # -- memory -----------------------------------------------------------------------------
    def uninit_buffer(self, length: int, usage: int = BufferUsages.STORAGE, dtype=np.float32) -> GpuBuffer:
        """src/tensor/tensor_impl.rs:69"""
        dt = np.dtype(dtype)
        p = C.c_void_p()
        _lib.check(_lib.load().vx_alloc(self._ctx, length * dt.itemsize, C.byref(p)))
        return GpuBuffer(self, p.value, length, dt, usage)

    def init_buffer(self, data, usage: int = BufferUsages.STORAGE) -> GpuBuffer:
        """src/tensor/tensor_impl.rs:105"""
        arr = np.ascontiguousarray(data)
        buf = self.uninit_buffer(arr.size, usage, arr.dtype)
        _lib.check(_lib.load().vx_upload(self._ctx, buf.ptr, arr.ctypes.data, arr.nbytes))
        # The source array may be a temporary: finish the copy before it can be collected.
        self.synchronize()
        return buf

    def write_buffer(self, buffer: GpuBuffer, offset: int, data) -> None:
        """src/tensor/tensor_impl.rs:715 — offset in elements."""
        arr = np.ascontiguousarray(data, dtype=buffer.dtype)
        if offset + arr.size > buffer.len():
            raise IndexError("write_buffer range out of bounds")
        _lib.check(_lib.load().vx_upload(self._ctx, buffer.ptr + offset * buffer.dtype.itemsize,
                                         arr.ctypes.data, arr.nbytes))
        self.synchronize()

    def slow_read_buffer(self, src, out: np.ndarray) -> None:
        """src/linalg/gemm.rs:423-426 — fills `out` (its length decides how much is read)."""
        sl = src if isinstance(src, GpuBufferSlice) else src.as_slice()
        if out.size > sl.len():
            raise IndexError("slow_read_buffer: destination longer than the source slice")
        if not out.flags["C_CONTIGUOUS"]:
            raise ValueError("slow_read_buffer needs a contiguous destination")
        _lib.check(_lib.load().vx_download(self._ctx, out.ctypes.data, sl.ptr, out.nbytes))
