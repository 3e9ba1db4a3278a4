"""TensorLayout — the view/stride algebra of vortx's src/shapes.rs, served by the C
host layer (vx_layout_* in include/vortx_b200_host.h).

Same method names and argument meaning as the reference.  Where the reference panics this
raises LayoutError; where it returns None (broadcast) this returns None.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence, Tuple

from . import _lib
from ._lib import LayoutError, VxLayout, VxShape

# src/shapes.rs:15-18
GGML_IDS = (1, 0, 2, 3)


def _u32(values: Sequence[int]):
    return (C.c_uint32 * max(1, len(values)))(*values)


class TensorLayout:
    """src/shapes.rs:49-60: size[4], stride[4] (elements), rank, offset."""

    __slots__ = ("_c",)

    def __init__(self, size, stride, rank: int, offset: int = 0):
        c = VxLayout()
        for k in range(4):
            c.size[k] = size[k]
            c.stride[k] = stride[k]
        c.rank = rank
        c.offset = offset
        self._c = c

    # -- plumbing ---------------------------------------------------------------
    @classmethod
    def _from_c(cls, c: VxLayout) -> "TensorLayout":
        obj = cls.__new__(cls)
        obj._c = c
        return obj

    def _call(self, name: str, *args) -> "TensorLayout":
        out = VxLayout()
        st = getattr(_lib.load(), name)(C.byref(self._c), *args, C.byref(out))
        if st == _lib.VX_ERR_INVALID_ARGUMENT:
            raise LayoutError(st, _lib.last_error())
        _lib.check(st)
        return TensorLayout._from_c(out)

    @property
    def size(self) -> Tuple[int, int, int, int]:
        return tuple(self._c.size)

    @property
    def stride(self) -> Tuple[int, int, int, int]:
        return tuple(self._c.stride)

    @property
    def rank(self) -> int:
        return self._c.rank

    @property
    def offset(self) -> int:
        return self._c.offset

    def dims(self):
        return self.size[: self.rank]

    def strides(self):
        return self.stride[: self.rank]

    def __eq__(self, other):
        return (isinstance(other, TensorLayout) and self.size == other.size
                and self.stride == other.stride and self.rank == other.rank
                and self.offset == other.offset)

    def __hash__(self):
        return hash((self.size, self.stride, self.rank, self.offset))

    def __repr__(self):
        return (f"TensorLayout(size={list(self.size)}, stride={list(self.stride)}, "
                f"rank={self.rank}, offset={self.offset})")

    # -- constructors -------------------------------------------------------------
    @classmethod
    def contiguous(cls, size: Sequence[int]) -> "TensorLayout":
        """src/shapes.rs:85-99"""
        out = VxLayout()
        st = _lib.load().vx_layout_contiguous(_u32(size), len(size), C.byref(out))
        if st == _lib.VX_ERR_INVALID_ARGUMENT:
            raise LayoutError(st, _lib.last_error())
        _lib.check(st)
        return cls._from_c(out)

    # -- conversions ----------------------------------------------------------------
    def into_gpu(self) -> VxShape:
        """src/shapes.rs:20-47, :71-73"""
        s = VxShape()
        _lib.check(_lib.load().vx_layout_to_shape(C.byref(self._c), C.byref(s)))
        return s

    def canonicalize(self) -> "TensorLayout":
        return self._call("vx_layout_canonicalize")

    def _call_optional(self, name: str, *args) -> Optional["TensorLayout"]:
        """For the reference functions that return Option: None on VX_ERR_UNSUPPORTED."""
        try:
            return self._call(name, *args)
        except _lib.VortxError as e:
            if e.status == _lib.VX_ERR_UNSUPPORTED:
                return None
            raise

    def unsqueeze_to_rank(self, rank: int) -> Optional["TensorLayout"]:
        return self._call_optional("vx_layout_unsqueeze_to_rank", rank)

    def unsqueeze(self, axis: int) -> Optional["TensorLayout"]:
        return self._call_optional("vx_layout_unsqueeze", axis)

    def squeeze_axis(self, axis: int) -> "TensorLayout":
        return self._call("vx_layout_squeeze_axis", axis)

    def squeeze(self) -> "TensorLayout":
        return self._call("vx_layout_squeeze")

    def index(self, i: int) -> "TensorLayout":
        return self._call("vx_layout_index", i)

    def transpose(self, axis_a: int, axis_b: int) -> "TensorLayout":
        return self._call("vx_layout_transpose", axis_a, axis_b)

    def transpose_last_dims(self) -> "TensorLayout":
        return self._call("vx_layout_transpose_last_dims")

    def permute(self, permutations: Sequence[int]) -> "TensorLayout":
        return self._call("vx_layout_permute", _u32(permutations))

    def permute_ggml(self, permutations: Sequence[int]) -> "TensorLayout":
        return self._call("vx_layout_permute_ggml", _u32(permutations))

    def is_contiguous(self) -> bool:
        return bool(_lib.load().vx_layout_is_contiguous(C.byref(self._c)))

    def broadcast(self, other: "TensorLayout") -> Optional[Tuple["TensorLayout", "TensorLayout"]]:
        a, b = VxLayout(), VxLayout()
        st = _lib.load().vx_layout_broadcast(C.byref(self._c), C.byref(other._c), C.byref(a), C.byref(b))
        if st == _lib.VX_ERR_SHAPE:
            return None
        _lib.check(st)
        return TensorLayout._from_c(a), TensorLayout._from_c(b)

    def broadcast_assign(self, source: "TensorLayout"):
        a, b = VxLayout(), VxLayout()
        st = _lib.load().vx_layout_broadcast_assign(C.byref(self._c), C.byref(source._c),
                                                     C.byref(a), C.byref(b))
        if st == _lib.VX_ERR_SHAPE:
            return None
        _lib.check(st)
        return TensorLayout._from_c(a), TensorLayout._from_c(b)

    def view(self, offset: int, shape: Sequence[int], stride: Sequence[Optional[int]] = ()) -> "TensorLayout":
        """src/shapes.rs:407-441; `stride` entries may be None (derive)."""
        vals = [0 if s is None else s for s in stride]
        flags = (C.c_uint8 * max(1, len(stride)))(*[0 if s is None else 1 for s in stride])
        return self._call("vx_layout_view", offset, _u32(shape), len(shape), _u32(vals), flags, len(stride))

    def reshape(self, shape: Sequence[int]) -> "TensorLayout":
        return self._call("vx_layout_reshape", _u32(shape), len(shape))

    def narrow(self, axis: int, first_elt: int, new_nelts: int) -> "TensorLayout":
        return self._call("vx_layout_narrow", axis, first_elt, new_nelts)

    def matrix(self, matrix_id: int) -> "TensorLayout":
        return self._call("vx_layout_matrix", matrix_id)

    def columns(self, first_col: int, new_ncols: int) -> "TensorLayout":
        return self._call("vx_layout_columns", first_col, new_ncols)

    def column(self, col: int) -> "TensorLayout":
        return self.columns(col, 1)

    def rows(self, first_row: int, new_nrows: int) -> "TensorLayout":
        return self._call("vx_layout_rows", first_row, new_nrows)

    def row(self, row: int) -> "TensorLayout":
        return self.rows(row, 1)

    def f32_to_vec4(self) -> "TensorLayout":
        return self._call("vx_layout_f32_to_vec4")

    def len(self) -> int:
        return int(_lib.load().vx_layout_len(C.byref(self._c)))

    def __len__(self):
        return self.len()

    def is_empty(self) -> bool:
        return self.len() == 0

    def span(self) -> int:
        return int(_lib.load().vx_layout_span(C.byref(self._c)))


class TensorLayoutBuffers:
    """src/shapes.rs:541-640.  The reference caches one 32-byte uniform buffer per layout;
    here shapes travel by value as kernel parameters, so this keeps only the call shape."""

    def __init__(self, backend=None):
        self._seen = set()

    def insert(self, backend, shape: TensorLayout) -> None:
        self._seen.add(shape)

    def put_tmp(self, backend, shape: TensorLayout) -> None:
        self._seen.add(shape)

    def clear_tmp(self) -> None:
        pass

    def contains(self, shape: TensorLayout) -> bool:
        return shape in self._seen

    def get(self, shape: TensorLayout):
        return shape.into_gpu() if shape in self._seen else None
