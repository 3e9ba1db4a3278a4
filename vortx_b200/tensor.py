"""Tensor, TensorRef, TensorMut and TensorBuilder — vortx's src/tensor/*.rs over CUDA memory.

A Tensor owns a device buffer plus shape[4] and rank (src/tensor/tensor_impl.rs:117-121);
views borrow the buffer and carry a TensorLayout (src/tensor/tensor_ref.rs:11-14).  Matrices
are row-major.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from .backend import Backend, BufferUsages, GpuBuffer, GpuBufferSlice, GpuEncoder
from .shapes import GGML_IDS, TensorLayout


def _append_ones(shape: Sequence[int]):
    if len(shape) > 4:
        raise ValueError("tensors of ranks > 4 not supported")
    return list(shape) + [1] * (4 - len(shape)), len(shape)


class _LayoutModifiers:
    """The view methods shared by TensorRef and TensorMut (src/tensor/tensor_macro.rs:1-125)."""

    layout_: TensorLayout

    def _with_layout(self, layout: TensorLayout):
        raise NotImplementedError

    def index(self, i):
        return self._with_layout(self.layout_.index(i))

    def transpose(self, axis_a, axis_b):
        return self._with_layout(self.layout_.transpose(axis_a, axis_b))

    def transpose_last_dims(self):
        return self._with_layout(self.layout_.transpose_last_dims())

    def permute(self, permutations):
        return self._with_layout(self.layout_.permute(permutations))

    def permute_ggml(self, permutations):
        return self._with_layout(self.layout_.permute_ggml(permutations))

    def canonicalize(self):
        return self._with_layout(self.layout_.canonicalize())

    def unsqueeze(self, axis):
        l = self.layout_.unsqueeze(axis)
        if l is None:
            raise ValueError("Not enough rank available for unsqueezing.")
        return self._with_layout(l)

    def reshape(self, shape):
        return self._with_layout(self.layout_.reshape(shape))

    def reshape_ggml(self, shape):
        raise NotImplementedError("todo!() in the reference (src/tensor/tensor_macro.rs:54-58)")

    def view(self, offset, shape, stride=()):
        return self._with_layout(self.layout_.view(offset, shape, stride))

    def view_ggml(self, offset, shape, stride=()):
        raise NotImplementedError("todo!() in the reference (src/tensor/tensor_macro.rs:67-72)")

    def narrow(self, axis, first_elt, new_nelts):
        return self._with_layout(self.layout_.narrow(axis, first_elt, new_nelts))

    def matrix(self, matrix_id):
        return self._with_layout(self.layout_.matrix(matrix_id))

    def columns(self, first_col, new_ncols):
        return self._with_layout(self.layout_.columns(first_col, new_ncols))

    def column(self, col):
        return self._with_layout(self.layout_.column(col))

    def rows(self, first_row, new_nrows):
        return self._with_layout(self.layout_.rows(first_row, new_nrows))

    def row(self, row):
        return self._with_layout(self.layout_.row(row))

    def squeeze_axis(self, axis):
        return self._with_layout(self.layout_.squeeze_axis(axis))

    def squeeze(self):
        return self._with_layout(self.layout_.squeeze())

    # -- accessors (src/tensor/tensor_ref.rs:74-137) -------------------------------------
    def is_contiguous(self) -> bool:
        return self.layout_.is_contiguous()

    def is_entire_tensor(self) -> bool:
        return (self.buffer_.len() == self.len() and self.layout_.offset == 0
                and self.is_contiguous())

    def rank(self) -> int:
        return self.layout_.rank

    def layout(self) -> TensorLayout:
        return self.layout_

    def buffer(self) -> GpuBufferSlice:
        """The buffer advanced by the view offset (src/tensor/tensor_ref.rs:101-103)."""
        return self.buffer_.slice(self.layout_.offset)

    def raw_buffer(self) -> GpuBuffer:
        return self.buffer_

    def len(self) -> int:
        return self.layout_.len()

    def is_empty(self) -> bool:
        return self.len() == 0

    def size(self, i: int) -> int:
        return self.layout_.size[i]

    def size_ggml(self, i: int) -> int:
        return self.layout_.size[GGML_IDS[i]]

    def stride(self, i: int) -> int:
        return self.layout_.stride[i]

    def stride_ggml(self, i: int) -> int:
        return self.layout_.stride[GGML_IDS[i]]

    def as_tensor_ref(self) -> "TensorRef":
        return TensorRef(self.layout_, self.buffer_)


class TensorRef(_LayoutModifiers):
    """src/tensor/tensor_ref.rs:11-14"""

    def __init__(self, layout: TensorLayout, buffer: GpuBuffer):
        self.layout_ = layout
        self.buffer_ = buffer

    def _with_layout(self, layout):
        return TensorRef(layout, self.buffer_)


class TensorMut(_LayoutModifiers):
    """src/tensor/tensor_mut.rs:10-13"""

    def __init__(self, layout: TensorLayout, buffer: GpuBuffer):
        self.layout_ = layout
        self.buffer_ = buffer

    def _with_layout(self, layout):
        return TensorMut(layout, self.buffer_)

    def as_ref(self) -> TensorRef:
        return TensorRef(self.layout_, self.buffer_)

    def buffer_mut(self) -> GpuBufferSlice:
        return self.buffer_.slice(self.layout_.offset)

    def as_tensor_mut(self) -> "TensorMut":
        return self


class TensorBuilder:
    """src/tensor/tensor_impl.rs:18-112"""

    def __init__(self, shape: Sequence[int], usage: int):
        self.shape, self.rank = _append_ones(shape)
        self.usage = usage
        self.label_: Optional[str] = None

    @classmethod
    def scalar(cls, usage):
        return cls([], usage)

    @classmethod
    def vector(cls, dim, usage):
        return cls([dim], usage)

    @classmethod
    def matrix(cls, nrows, ncols, usage):
        return cls([nrows, ncols], usage)

    @classmethod
    def tensor(cls, shape, usage):
        return cls(shape, usage)

    def len(self) -> int:
        return int(np.prod(self.shape, dtype=np.uint64))

    def label(self, label: str):
        self.label_ = label
        return self

    def build_uninit(self, backend: Backend, dtype=np.float32) -> "Tensor":
        buf = backend.uninit_buffer(self.len(), self.usage, dtype)
        return Tensor(self.shape, self.rank, buf)

    def build_init(self, backend: Backend, data) -> "Tensor":
        arr = np.ascontiguousarray(data)
        if arr.size < self.len():
            raise ValueError("Incorrect number of elements provided for initializing Tensor. "
                             f"Expected at least {self.len()}, found {arr.size}")
        return Tensor(self.shape, self.rank, backend.init_buffer(arr.reshape(-1), self.usage))


class Tensor:
    """src/tensor/tensor_impl.rs:117-121 — owns shape[4], rank and a device buffer."""

    def __init__(self, shape, rank: int, buffer: GpuBuffer):
        self.shape_ = list(shape)
        self.rank_ = rank
        self.buffer_ = buffer

    # -- constructors (src/tensor/tensor_impl.rs:500-640) ---------------------------------
    @classmethod
    def matrix_uninit(cls, backend, nrows, ncols, usage=BufferUsages.STORAGE, dtype=np.float32):
        return TensorBuilder.matrix(nrows, ncols, usage).build_uninit(backend, dtype)

    @classmethod
    def matrix(cls, backend, nrows, ncols, data, usage=BufferUsages.STORAGE):
        """Row-major `data` of exactly nrows*ncols elements (:543-555)."""
        arr = np.ascontiguousarray(data)
        if arr.size != nrows * ncols:
            raise ValueError(f"matrix data has {arr.size} elements, expected {nrows * ncols}")
        return TensorBuilder.matrix(nrows, ncols, usage).build_init(backend, arr)

    @classmethod
    def matrix_from_na(cls, backend, matrix: np.ndarray, usage=BufferUsages.STORAGE):
        """:522-540 takes a column-major nalgebra matrix and uploads it row-major.  A 2-D numpy
        array of any memory order plays the nalgebra matrix here; the upload is row-major."""
        m = np.asarray(matrix)
        if m.ndim != 2:
            raise ValueError("matrix_from_na needs a 2-D array")
        return cls.matrix(backend, m.shape[0], m.shape[1], np.ascontiguousarray(m), usage)

    @classmethod
    def with_capacity(cls, backend, capacity, usage=BufferUsages.STORAGE, dtype=np.float32):
        t = cls.vector_uninit(backend, capacity, usage, dtype)
        t.shape_ = [0, 1, 1, 1]
        return t

    @classmethod
    def vector_uninit(cls, backend, length, usage=BufferUsages.STORAGE, dtype=np.float32):
        return TensorBuilder.vector(length, usage).build_uninit(backend, dtype)

    @classmethod
    def vector(cls, backend, vector, usage=BufferUsages.STORAGE):
        v = np.ascontiguousarray(vector).reshape(-1)
        return TensorBuilder.vector(v.size, usage).build_init(backend, v)

    @classmethod
    def scalar_uninit(cls, backend, usage=BufferUsages.STORAGE, dtype=np.float32):
        return TensorBuilder.scalar(usage).build_uninit(backend, dtype)

    @classmethod
    def scalar(cls, backend, value, usage=BufferUsages.STORAGE, dtype=np.float32):
        return TensorBuilder.scalar(usage).build_init(backend, np.array([value], dtype=dtype))

    # -- accessors (:123-262) ----------------------------------------------------------------
    def is_empty(self):
        return self.len() == 0

    def len(self) -> int:
        return int(np.prod(self.shape_, dtype=np.uint64))

    def capacity(self) -> int:
        return self.buffer_.len()

    def order(self) -> int:
        return sum(1 for s in self.shape_ if s > 1)

    def size(self, i):
        return self.shape_[i]

    def size_ggml(self, i):
        return self.size(GGML_IDS[i])

    def stride(self, i):
        return self.layout().stride[i]

    def stride_ggml(self, i):
        return self.stride(GGML_IDS[i])

    def bytes_len(self) -> int:
        return self.buffer_.dtype.itemsize * self.len()

    def shape(self):
        return list(self.shape_)

    def rank(self):
        return self.rank_

    def buffer(self) -> GpuBuffer:
        return self.buffer_

    buffer_mut = buffer

    def buffer_slice(self) -> GpuBufferSlice:
        return self.buffer_.slice(0)

    def into_inner(self) -> GpuBuffer:
        return self.buffer_

    def dims(self):
        return self.shape_[: self.rank_]

    def layout(self) -> TensorLayout:
        return TensorLayout.contiguous(self.dims())

    def as_view(self) -> TensorRef:
        return TensorRef(self.layout(), self.buffer_)

    def as_view_mut(self) -> TensorMut:
        return TensorMut(self.layout(), self.buffer_)

    as_tensor_ref = as_view
    as_tensor_mut = as_view_mut

    def copy_from_view(self, encoder: GpuEncoder, source) -> None:
        """:193-214"""
        src = source.as_tensor_ref()
        if self.len() > src.len():
            raise ValueError("copy_from_view: source shorter than destination")
        encoder.copy_buffer_to_buffer(src.raw_buffer(), src.layout().offset, self.buffer_, 0, self.len())

    # -- in-place shape edits (:331-352) --------------------------------------------------------
    def squeeze(self):
        l = self.layout().squeeze()
        self.shape_, self.rank_ = list(l.size), l.rank

    def unsqueeze(self, axis):
        if axis > self.rank_:
            raise ValueError("unsqueeze axis out of bounds")
        if self.rank_ >= 4:
            raise ValueError("unsqueezing would exceed the max supported tensor rank")
        l = self.layout().unsqueeze(axis)
        self.shape_, self.rank_ = list(l.size), l.rank

    # -- views (:355-498) ----------------------------------------------------------------------------
    def reshape(self, shape): return self.as_view().reshape(shape)
    def permute(self, p): return self.as_view().permute(p)
    def permute_ggml(self, p): return self.as_view().permute_ggml(p)
    def view(self, offset, shape, stride=()): return self.as_view().view(offset, shape, stride)
    def transpose(self, a, b): return self.as_view().transpose(a, b)
    def transpose_last_dims(self): return self.as_view().transpose_last_dims()
    def narrow(self, axis, first, n): return self.as_view().narrow(axis, first, n)
    def column(self, i): return self.as_view().column(i)
    def columns(self, first, n): return self.as_view().columns(first, n)
    def row(self, i): return self.as_view().row(i)
    def rows(self, first, n): return self.as_view().rows(first, n)
    def reshape_mut(self, shape): return self.as_view_mut().reshape(shape)
    def permute_mut(self, p): return self.as_view_mut().permute(p)
    def view_mut(self, offset, shape, stride=()): return self.as_view_mut().view(offset, shape, stride)
    def transpose_mut(self, a, b): return self.as_view_mut().transpose(a, b)
    def transpose_last_dims_mut(self): return self.as_view_mut().transpose_last_dims()
    def narrow_mut(self, axis, first, n): return self.as_view_mut().narrow(axis, first, n)
    def column_mut(self, i): return self.as_view_mut().column(i)
    def columns_mut(self, first, n): return self.as_view_mut().columns(first, n)
    def row_mut(self, i): return self.as_view_mut().row(i)
    def rows_mut(self, first, n): return self.as_view_mut().rows(first, n)

    # -- growth (:673-815) ---------------------------------------------------------------------------
    def append(self, backend: Backend, data) -> None:
        """Appends to a rank-1 tensor, growing the buffer to the next power of two when full."""
        if self.rank_ != 1:
            raise ValueError("Appending is currently only supported on rank-1 tensors.")
        arr = np.ascontiguousarray(data, dtype=self.buffer_.dtype).reshape(-1)
        curr = self.shape_[0]
        new_len = curr + arr.size
        if new_len >= self.capacity():
            cap = 1 if new_len <= 1 else 1 << (new_len - 1).bit_length()  # u32::next_power_of_two
            new_buf = backend.uninit_buffer(cap, self.buffer_.usage() | BufferUsages.COPY_DST,
                                            self.buffer_.dtype)
            enc = backend.begin_encoding()
            enc.copy_buffer_to_buffer(self.buffer_, 0, new_buf, 0, curr)
            backend.submit(enc)
            old = self.buffer_
            self.buffer_ = new_buf
            old.free()
        if arr.size:
            backend.write_buffer(self.buffer_, curr, arr)
        self.shape_[0] = new_len

    def shift_remove(self, backend: Backend, start: int, end: Optional[int] = None) -> int:
        """Removes [start, end) from a rank-1 tensor, shifting the tail back (through a staging buffer)."""
        if self.rank_ != 1:
            raise ValueError("Remove is currently only supported on rank-1 tensors.")
        curr = self.shape_[0]
        end = curr if end is None else end
        if end <= start:
            return 0
        if end > curr:
            raise IndexError("Range index out of bounds.")
        moved = curr - end
        if moved > 0:
            staging = backend.uninit_buffer(moved, BufferUsages.STORAGE | BufferUsages.COPY_DST
                                            | BufferUsages.COPY_SRC, self.buffer_.dtype)
            enc = backend.begin_encoding()
            enc.copy_buffer_to_buffer(self.buffer_, end, staging, 0, moved)
            enc.copy_buffer_to_buffer(staging, 0, self.buffer_, start, moved)
            backend.submit(enc)
            staging.free()
        self.shape_[0] -= end - start
        return end - start

    # -- convenience for tests and examples ------------------------------------------------------------
    def read(self, backend: Backend) -> np.ndarray:
        out = np.empty(self.len(), dtype=self.buffer_.dtype)
        if out.size:
            backend.slow_read_buffer(self.buffer_, out)
        return out.reshape(self.dims() or [1])


def as_tensor_ref(x) -> TensorRef:
    return x.as_tensor_ref()


def as_tensor_mut(x) -> TensorMut:
    return x.as_tensor_mut()
