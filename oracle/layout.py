"""Pure-Python restatement of vortx's TensorLayout (src/shapes.rs) — TEST INFRASTRUCTURE ONLY.

An independent second statement of the view algebra, used to cross-check the C host layer on
random inputs.  Pinned by the reference's own broadcast tests (src/shapes.rs:646-782), which
tests/test_layout.py replays against both statements.  A reference panic is LayoutPanic here.
u32 arithmetic wraps, as in the reference's release builds.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import List, Optional, Sequence, Tuple

M32 = 0xFFFFFFFF


class LayoutPanic(Exception):
    pass


@dataclass(frozen=True)
class Layout:
    size: Tuple[int, int, int, int]
    stride: Tuple[int, int, int, int]
    rank: int
    offset: int = 0

    # src/shapes.rs:85-99
    @staticmethod
    def contiguous(size: Sequence[int]) -> "Layout":
        if len(size) > 4:
            raise LayoutPanic("tensors of ranks > 4 not supported")
        rank = len(size)
        sz = list(size) + [1] * (4 - rank)
        st = [1, 1, 1, 1]
        cur = 1
        for k in reversed(range(rank)):
            st[k] = cur
            cur = (cur * sz[k]) & M32
        return Layout(tuple(sz), tuple(st), rank, 0)

    # src/shapes.rs:20-47
    def to_shape(self) -> Tuple[int, ...]:
        sz, st = list(self.size), list(self.stride)
        for k in range(self.rank, 4):
            sz[k] = 1
            st[k] = st[self.rank - 1] if self.rank > 0 else 1
        return tuple(sz + st)

    # src/shapes.rs:145-155
    def canonicalize(self) -> "Layout":
        if self.rank == 4:
            return self
        d = 4 - self.rank
        sz = [1] * d + list(self.size[: self.rank])
        res = Layout.contiguous(sz)
        st = list(res.stride)
        st[d:] = self.stride[: self.rank]
        return Layout(res.size, tuple(st), 4, 0)

    # src/shapes.rs:115-141
    def unsqueeze_to_rank(self, rank: int) -> Optional["Layout"]:
        if self.rank > 4 or rank < self.rank or rank > 4:
            return None
        if self.rank == rank:
            return self
        if self.rank == 0:
            return Layout((1,) * 4, (1,) * 4, rank, self.offset)
        sz, st = list(self.size), list(self.stride)
        default = (st[self.rank - 1] * sz[self.rank - 1]) & M32
        for k in range(self.rank, 4):
            sz[k], st[k] = 1, default
        return Layout(tuple(sz), tuple(st), rank, self.offset)

    # src/shapes.rs:161-175
    def unsqueeze(self, axis: int) -> Optional["Layout"]:
        if self.rank >= 4 or axis > self.rank:
            return None
        sz, st = list(self.size), list(self.stride)
        for i in reversed(range(axis, 3)):
            sz[i + 1], st[i + 1] = sz[i], st[i]
        sz[axis] = 1
        if axis + 1 > 3:
            raise LayoutPanic("stride[axis + 1] is out of bounds (the reference panics here)")
        st[axis] = st[axis + 1]
        return Layout(tuple(sz), tuple(st), self.rank + 1, self.offset)

    # src/shapes.rs:177-200
    def squeeze_axis(self, axis: int) -> "Layout":
        if axis >= self.rank:
            raise LayoutPanic("axis out of bounds")
        if self.size[axis] != 1:
            raise LayoutPanic("can only squeeze an axis with length 1")
        sz, st = list(self.size), list(self.stride)
        for k in range(axis, self.rank - 1):
            sz[k], st[k] = sz[k + 1], st[k + 1]
        rank = self.rank - 1
        sz[rank] = 1
        if rank > 0:
            p = 1
            for v in sz[: rank - 1]:
                p = (p * v) & M32
            st[rank] = p
        return Layout(tuple(sz), tuple(st), rank, self.offset)

    # src/shapes.rs:202-230
    def squeeze(self) -> "Layout":
        sz, st = list(self.size), list(self.stride)
        new_rank = 0
        for k in range(self.rank):
            if sz[k] != 1:
                sz[new_rank], st[new_rank] = sz[k], st[k]
                new_rank += 1
        if new_rank == 0:
            return Layout((1,) * 4, (1,) * 4, 0, self.offset)
        for k in range(new_rank, 4):
            sz[k] = 1
            st[k] = (st[new_rank - 1] * sz[new_rank - 1]) & M32
        return Layout(tuple(sz), tuple(st), new_rank, self.offset)

    # src/shapes.rs:232-234
    def index(self, i: int) -> "Layout":
        return self.narrow(0, i, 1).squeeze_axis(0)

    # src/shapes.rs:238-254
    def transpose(self, a: int, b: int) -> "Layout":
        if a >= self.rank or b >= self.rank:
            raise LayoutPanic("transpose axis index out of bounds")
        sz, st = list(self.size), list(self.stride)
        sz[a], sz[b] = sz[b], sz[a]
        st[a], st[b] = st[b], st[a]
        return Layout(tuple(sz), tuple(st), self.rank, self.offset)

    def transpose_last_dims(self) -> "Layout":
        if self.rank < 2:
            raise LayoutPanic("rank < 2")
        return self.transpose(self.rank - 2, self.rank - 1)

    # src/shapes.rs:268-329
    def permute(self, perm: Sequence[int]) -> "Layout":
        if len(set(perm)) != 4 or any(p > 3 for p in perm):
            raise LayoutPanic("Permutation indices must not overlap.")
        for k in range(self.rank):
            if perm[k] >= self.rank:
                raise LayoutPanic("permutation index exceeds this matrix rank")
        for k in range(self.rank, 4):
            if perm[k] != k:
                raise LayoutPanic("Indices exceeding the tensor rank must be identity")
        sz, st = [0] * 4, [0] * 4
        for k in range(4):
            sz[perm[k]], st[perm[k]] = self.size[k], self.stride[k]
        return Layout(tuple(sz), tuple(st), self.rank, self.offset)

    # src/shapes.rs:262-265
    def permute_ggml(self, perm: Sequence[int]) -> "Layout":
        p = list(perm)
        p[0], p[1] = p[1], p[0]
        ggml = (1, 0, 2, 3)
        if any(v > 3 for v in p):
            raise LayoutPanic("index out of range")
        return self.permute([ggml[v] for v in p])

    # src/shapes.rs:332-343
    def is_contiguous(self) -> bool:
        stride = 1
        for i in reversed(range(self.rank)):
            if self.stride[i] != 0 and self.stride[i] != stride:
                return False
            stride = (stride * self.size[i]) & M32
        return True

    # src/shapes.rs:346-389
    def broadcast(self, other: "Layout") -> Optional[Tuple["Layout", "Layout"]]:
        a, b = self, other
        flip = a.rank > b.rank
        if flip:
            a, b = b, a
        asz, ast = list(a.size), list(a.stride)
        bsz, bst = list(b.size), list(b.stride)
        d = b.rank - a.rank
        for k in reversed(range(a.rank)):
            asz[k + d], ast[k + d] = asz[k], ast[k]
        for k in range(d):
            asz[k] = 1
        rank = b.rank
        for k in range(rank):
            if asz[k] == 1:
                ast[k] = 0
            if bsz[k] == 1:
                bst[k] = 0
        for k in range(rank):
            if asz[k] != 1 and bsz[k] != 1 and asz[k] != bsz[k]:
                return None
        la = Layout(tuple(asz), tuple(ast), rank, a.offset)
        lb = Layout(tuple(bsz), tuple(bst), b.rank, b.offset)
        return (lb, la) if flip else (la, lb)

    # src/shapes.rs:393-404
    def broadcast_assign(self, source: "Layout"):
        r = self.broadcast(source)
        if r is None:
            return None
        t, s = r
        for k in range(t.rank):
            if t.size[k] < s.size[k]:
                return None
        return t, s

    # src/shapes.rs:407-441
    def view(self, offset: int, shape: Sequence[int], stride: Sequence[Optional[int]] = ()) -> "Layout":
        if len(shape) > 4 or len(stride) > len(shape):
            raise LayoutPanic("bad view arguments")
        if not self.is_contiguous():
            raise LayoutPanic("Cannot take a view of a non-contiguous tensor")
        avail = 1
        for v in self.size:
            avail = (avail * v) & M32
        need = 1
        for v in shape:
            need = (need * v) & M32
        need = (need + offset) & M32
        if need > avail:
            raise LayoutPanic("Source tensor is too small for reshaping")
        rank = len(shape)
        sz = list(shape) + [1] * (4 - rank)
        st = [0] * 4
        cur = 1
        for k in reversed(range(rank)):
            given = stride[k] if k < len(stride) else None
            st[k] = given if given is not None else cur
            cur = (st[k] * sz[k]) & M32
        return Layout(tuple(sz), tuple(st), rank, (self.offset + offset) & M32)

    def reshape(self, shape: Sequence[int]) -> "Layout":
        return self.view(0, shape, ())

    # src/shapes.rs:443-464
    def narrow(self, axis: int, first: int, count: int) -> "Layout":
        if axis >= self.rank:
            raise LayoutPanic("Axis index out of bounds.")
        if first + count > self.size[axis]:
            raise LayoutPanic("narrow out of range")
        sz = list(self.size)
        sz[axis] = count
        return Layout(tuple(sz), self.stride, self.rank, (self.offset + self.stride[axis] * first) & M32)

    # src/shapes.rs:467-489
    def matrix(self, i): return self.narrow(2, i, 1)
    def columns(self, first, n): return self.narrow(1, first, n)
    def column(self, c): return self.columns(c, 1)
    def rows(self, first, n): return self.narrow(0, first, n)
    def row(self, r): return self.rows(r, 1)

    # src/shapes.rs:492-519
    def f32_to_vec4(self) -> "Layout":
        dim = max(self.rank, 1) - 1
        if self.stride[dim] != 1 or self.size[dim] % 4 != 0:
            raise LayoutPanic("not convertible to vec4")
        st = []
        for s in self.stride:
            if not (s == 1 or s % 4 == 0):
                raise LayoutPanic("stride not a multiple of 4")
            st.append((s + 3) // 4)
        sz = list(self.size)
        sz[dim] //= 4
        return Layout(tuple(sz), tuple(st), self.rank, self.offset)

    # src/shapes.rs:527-533
    def len(self) -> int:
        n = 1
        for v in self.size[: self.rank]:
            n *= v
        return max(n, 1)
