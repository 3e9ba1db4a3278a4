"""Layout algebra (vx_layout_*, the C host layer) against the reference's own known answers and
against the independent Python restatement in oracle/layout.py.

The ten broadcast cases are the reference's unit tests, src/shapes.rs:646-782, read as text.
"""
import itertools
import random

import pytest

import vortx_b200 as vb
from oracle.layout import Layout, LayoutPanic

TL = vb.TensorLayout


def both(size):
    return TL.contiguous(size), Layout.contiguous(size)


def same(c: vb.TensorLayout, p: Layout):
    assert c.size == p.size and c.stride == p.stride and c.rank == p.rank and c.offset == p.offset, (c, p)


# ---- the reference's broadcast tests, on both statements --------------------------------------

@pytest.mark.parametrize("mk", [TL.contiguous, Layout.contiguous])
class TestReferenceBroadcast:
    def test_same_shape(self, mk):
        a, b = mk([3, 4]), mk([3, 4])
        ab, bb = a.broadcast(b)
        assert ab == a and bb == b

    def test_scalar_to_matrix(self, mk):
        s, m = mk([1]).broadcast(mk([3, 4]))
        assert tuple(s.size) == (1, 1, 1, 1) and tuple(m.size) == (3, 4, 1, 1)
        assert s.rank == 2 and m.rank == 2
        assert s.stride[0] == 0 and s.stride[1] == 0

    def test_vector_to_matrix(self, mk):
        v, m = mk([3, 1]).broadcast(mk([3, 4]))
        assert tuple(v.size) == (3, 1, 1, 1) and tuple(m.size) == (3, 4, 1, 1)
        assert v.stride[1] == 0

    def test_row_vector_to_matrix(self, mk):
        v, m = mk([1, 4]).broadcast(mk([3, 4]))
        assert tuple(v.size) == (1, 4, 1, 1) and tuple(m.size) == (3, 4, 1, 1)
        assert v.stride[0] == 0

    def test_different_ranks(self, mk):
        v, t = mk([2]).broadcast(mk([3, 4, 2]))
        assert v.rank == 3 and t.rank == 3
        assert (v.size[0], v.size[1], v.size[2]) == (1, 1, 2)
        assert v.stride[0] == 0 and v.stride[1] == 0

    def test_incompatible_shapes(self, mk):
        assert mk([3, 4]).broadcast(mk([8])) is None
        assert mk([3, 4]).broadcast(mk([3])) is None

    def test_incompatible_inner_dim(self, mk):
        assert mk([3, 4]).broadcast(mk([3, 5])) is None

    def test_3d_tensors(self, mk):
        a, b = mk([2, 1, 4]).broadcast(mk([2, 3, 4]))
        assert a.stride[1] == 0

    def test_preserves_order(self, mk):
        a, b = mk([3, 4, 5]), mk([5])
        ab, bb = a.broadcast(b)
        assert ab == a
        assert bb.rank == a.rank
        assert (bb.size[0], bb.size[1], bb.size[2]) == (1, 1, 5)
        assert (bb.stride[0], bb.stride[1], bb.stride[2]) == (0, 0, 1)

    def test_4d_tensors(self, mk):
        a, b = mk([2, 3, 1, 5]), mk([2, 1, 4, 5])
        ab, bb = a.broadcast(b)
        assert tuple(ab.size) == tuple(a.size) and tuple(bb.size) == tuple(b.size)
        assert ab.rank == 4 and bb.rank == 4
        assert ab.stride[2] == 0 and bb.stride[1] == 0


# ---- known answers read off the reference source ------------------------------------------------

def test_contiguous_and_canonicalize_known_answers():
    l = TL.contiguous([3, 4])
    assert l.size == (3, 4, 1, 1) and l.stride == (4, 1, 1, 1) and l.rank == 2
    c = l.canonicalize()               # ones prepended on the left, strides of the real dims kept
    assert c.size == (1, 1, 3, 4) and c.stride == (12, 12, 4, 1) and c.rank == 4 and c.offset == 0
    assert c.into_gpu().astuple() == (1, 1, 3, 4, 12, 12, 4, 1)
    # dims beyond the rank take the last real stride (src/shapes.rs:27-34)
    assert l.into_gpu().astuple() == (3, 4, 1, 1, 4, 1, 1, 1)
    assert TL.contiguous([]).into_gpu().astuple() == (1, 1, 1, 1, 1, 1, 1, 1)
    # config 0 of the benchmark: [1024,1024] -> [1,1,1024,1024], strides [1048576,1048576,1024,1]
    g = TL.contiguous([1024, 1024]).canonicalize()
    assert g.size == (1, 1, 1024, 1024) and g.stride == (1048576, 1048576, 1024, 1)


def test_canonicalize_drops_offset_and_keeps_view_strides():
    v = TL.contiguous([6, 8]).narrow(0, 2, 3).transpose(0, 1)
    assert v.offset == 16 and v.size[:2] == (8, 3) and v.stride[:2] == (1, 8)
    c = v.canonicalize()
    assert c.offset == 0 and c.size == (1, 1, 8, 3) and c.stride[2:] == (1, 8)


def test_vector_unsqueeze_as_in_reference_gemm_test():
    # src/linalg/gemm.rs:379-387: a 256-vector unsqueezed at axis 1 becomes [256, 1]
    v = TL.contiguous([256]).unsqueeze(1)
    assert v.rank == 2 and v.size[:2] == (256, 1)
    assert v.canonicalize().size == (1, 1, 256, 1)


def test_rows_columns_matrix_axes():
    t = TL.contiguous([5, 6, 7])
    assert t.rows(1, 2).size[:3] == (2, 6, 7) and t.rows(1, 2).offset == 42
    assert t.columns(2, 3).size[:3] == (5, 3, 7) and t.columns(2, 3).offset == 14
    assert t.matrix(4).size[:3] == (5, 6, 1) and t.matrix(4).offset == 4
    assert t.index(3).size[:2] == (6, 7) and t.index(3).offset == 126 and t.index(3).rank == 2


def test_panics_become_errors():
    with pytest.raises(vb.LayoutError):
        TL.contiguous([1, 2, 3, 4, 5])
    with pytest.raises(vb.LayoutError):
        TL.contiguous([3, 4]).transpose(0, 2)
    with pytest.raises(vb.LayoutError):
        TL.contiguous([3, 4]).narrow(1, 2, 3)
    with pytest.raises(vb.LayoutError):
        TL.contiguous([3, 4]).squeeze_axis(0)
    with pytest.raises(vb.LayoutError):
        TL.contiguous([3, 4]).transpose(0, 1).view(0, [12])   # view of a non-contiguous tensor
    with pytest.raises(vb.LayoutError):
        TL.contiguous([3, 4]).view(1, [3, 4])                  # too small
    with pytest.raises(vb.LayoutError):
        TL.contiguous([3, 4]).permute([0, 0, 2, 3])
    assert TL.contiguous([1, 2, 3, 4]).unsqueeze(0) is None
    assert TL.contiguous([3]).unsqueeze(2) is None


# ---- random cross-check of the two statements ---------------------------------------------------

def _rand_dims(rng, rank):
    return [rng.choice([1, 1, 2, 3, 4, 5, 8]) for _ in range(rank)]


def _apply(rng, c, p):
    """Applies one random operation to both statements; returns the new pair (or the old on a panic)."""
    ops = ["transpose", "narrow", "unsqueeze", "squeeze", "squeeze_axis", "permute", "canonicalize",
           "index", "view", "reshape", "unsqueeze_to_rank", "rows", "columns", "matrix", "f32_to_vec4",
           "transpose_last_dims", "permute_ggml"]
    op = rng.choice(ops)
    r = max(p.rank, 1)
    if op == "transpose":
        args = (rng.randrange(0, 4), rng.randrange(0, 4))
    elif op == "narrow":
        ax = rng.randrange(0, 4)
        first = rng.randrange(0, 4)
        args = (ax, first, rng.randrange(0, 4))
    elif op in ("unsqueeze", "squeeze_axis", "index", "matrix", "unsqueeze_to_rank"):
        args = (rng.randrange(0, 5),)
    elif op in ("permute", "permute_ggml"):
        perm = list(range(r)) if rng.random() < 0.8 else [rng.randrange(0, 4) for _ in range(r)]
        rng.shuffle(perm)
        args = (perm + list(range(len(perm), 4)),)
    elif op == "view":
        shape = _rand_dims(rng, rng.randrange(0, 4))
        stride = [rng.choice([None, None, 1, 2, 7]) for _ in range(rng.randrange(0, len(shape) + 1))]
        args = (rng.randrange(0, 3), shape, stride)
    elif op == "reshape":
        args = (_rand_dims(rng, rng.randrange(0, 4)),)
    elif op in ("rows", "columns"):
        args = (rng.randrange(0, 3), rng.randrange(0, 3))
    else:
        args = ()
    try:
        pn = getattr(p, op)(*args)
    except LayoutPanic:
        pn = "panic"
    try:
        cn = getattr(c, op)(*args)
    except vb.LayoutError:
        cn = "panic"
    if pn == "panic" or cn == "panic":
        assert pn == cn, (op, args, c, p, cn, pn)
        return c, p
    if pn is None or cn is None:
        assert pn is None and cn is None, (op, args, c, p)
        return c, p
    same(cn, pn)
    return cn, pn


def test_random_operation_chains_agree():
    rng = random.Random(1234)
    for _ in range(600):
        dims = _rand_dims(rng, rng.randrange(0, 5))
        c, p = both(dims)
        same(c, p)
        for _ in range(6):
            c, p = _apply(rng, c, p)
            assert c.is_contiguous() == p.is_contiguous()
            assert c.len() == p.len()
            assert c.into_gpu().astuple() == p.to_shape()


def test_random_broadcast_pairs_agree():
    rng = random.Random(99)
    for _ in range(500):
        a = _rand_dims(rng, rng.randrange(0, 5))
        b = _rand_dims(rng, rng.randrange(0, 5))
        (ca, pa), (cb, pb) = both(a), both(b)
        for name in ("broadcast", "broadcast_assign"):
            rc, rp = getattr(ca, name)(cb), getattr(pa, name)(pb)
            assert (rc is None) == (rp is None), (name, a, b)
            if rc is not None:
                same(rc[0], rp[0])
                same(rc[1], rp[1])
