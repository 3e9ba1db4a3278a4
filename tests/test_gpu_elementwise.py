"""OpAssign, Contiguous and Repeat on the GPU against the CPU oracle's restatement of the shaders
(vortx-shaders/src/linalg/{op_assign,contiguous,repeat}.rs).  Bar: bit-identical."""
import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import OpAssignVariant as OV, synth

pytestmark = pytest.mark.gpu


def _oshape(o, layout):
    c = layout.canonicalize()
    return o.Shape.of(c.size, c.stride)


def _t(backend, arr):
    return vb.Tensor(list(arr.shape) + [1] * (4 - arr.ndim), arr.ndim, backend.init_buffer(arr.ravel()))


@pytest.mark.parametrize("op", [OV.Add, OV.Sub, OV.Mul, OV.Div, OV.Copy])
@pytest.mark.parametrize("ashape,bshape", [((7,), (7,)), ((5, 9), (5, 9)), ((5, 9), (9,)), ((5, 9), (5, 1)),
                                           ((3, 4, 6), (1, 4, 1)), ((2, 3, 4, 5), (5,)), ((64, 1030), (1030,)),
                                           ((33, 17), (1,))])
def test_op_assign_broadcast_bit_exact(backend, oracle, op, ashape, bshape):
    A = synth.uniform_matrix(1, int(np.prod(ashape)), seed=1).reshape(ashape)
    B = (synth.uniform_matrix(1, int(np.prod(bshape)), seed=2).reshape(bshape) + np.float32(1.5)).astype(np.float32)
    a, b = _t(backend, A), _t(backend, B)
    vb.OpAssign().launch(backend, None, None, op, a, b)
    got = a.read(backend)
    la, lb = a.layout().broadcast_assign(b.layout())
    want = A.ravel().copy()
    oracle.op_assign(op, want, _oshape(oracle, la), B.ravel().copy(), _oshape(oracle, lb))
    assert np.array_equal(got.ravel().view(np.uint32), want.view(np.uint32))
    ref = {OV.Add: A + B, OV.Sub: A - B, OV.Mul: A * B, OV.Div: A / B, OV.Copy: np.broadcast_to(B, A.shape)}[op]
    assert np.array_equal(got.reshape(ashape), ref.astype(np.float32))


def test_op_assign_on_views_and_refusal(backend, oracle):
    A = synth.uniform_matrix(12, 20, seed=3)
    B = synth.uniform_matrix(20, 6, seed=4)
    a, b = _t(backend, A), _t(backend, B)
    # a[2:8, 5:11] += b[10:16, :]^T-free slice: rows 10..16 of b, all 6 columns
    av = a.as_view_mut().narrow(0, 2, 6).narrow(1, 5, 6)
    bv = b.narrow(0, 10, 6)
    vb.OpAssign().launch(backend, None, None, OV.Add, av, bv)
    want = A.copy()
    want[2:8, 5:11] += B[10:16, :]
    assert np.array_equal(a.read(backend), want)
    with pytest.raises(AssertionError):        # the reference panics: shapes cannot be broadcast
        vb.OpAssign().launch(backend, None, None, OV.Add, a, _t(backend, np.zeros((12, 19), np.float32)))
    with pytest.raises(AssertionError):        # assignment would grow the target
        vb.OpAssign().launch(backend, None, None, OV.Add, _t(backend, np.zeros((1, 20), np.float32)), a)


@pytest.mark.parametrize("dtype", [np.float32, np.uint32, np.int32])
def test_contiguous_gathers_views(backend, oracle, dtype):
    src = (np.arange(6 * 7 * 8) * 3 + 1).astype(dtype).reshape(6, 7, 8)
    t = _t(backend, src)
    for view, ref in ((t.transpose(0, 2), src.transpose(2, 1, 0)),
                      (t.narrow(1, 2, 3), src[:, 2:5, :]),
                      (t.transpose(1, 2).narrow(0, 1, 4), src.transpose(0, 2, 1)[1:5]),
                      (t.as_view(), src)):
        dims = list(view.layout().dims())
        out = vb.Tensor(dims + [1] * (4 - len(dims)), len(dims), backend.uninit_buffer(int(np.prod(dims)), dtype=dtype))
        vb.Contiguous().launch(backend, None, None, out, view)
        got = out.read(backend)
        assert np.array_equal(got, np.ascontiguousarray(ref))
        want = oracle.contiguous(src.ravel(), _oshape(oracle, view.layout()), view.layout().offset)
        assert np.array_equal(got.ravel(), want)
    bad = vb.Tensor([6, 7, 9, 1], 3, backend.uninit_buffer(6 * 7 * 9, dtype=dtype))
    with pytest.raises(AssertionError):
        vb.Contiguous().launch(backend, None, None, bad, t)


def test_repeat_tiles_the_source(backend, oracle):
    for dshape, sshape in (((6, 8), (1, 8)), ((6, 8), (6, 1)), ((4, 5, 6), (1, 5, 1)), ((3, 7), (1,)), ((5, 4), (5, 4))):
        S = synth.uniform_matrix(1, int(np.prod(sshape)), seed=7).reshape(sshape)
        d = _t(backend, np.full(dshape, np.nan, np.float32))
        s = _t(backend, S)
        vb.Repeat().launch(backend, None, None, d, s)
        got = d.read(backend)
        assert np.array_equal(got, np.broadcast_to(S, dshape))
        ld, ls = d.layout().broadcast_assign(s.layout())
        want = np.zeros(int(np.prod(dshape)), np.float32)
        oracle.repeat(want, _oshape(oracle, ld), S.ravel().copy(), _oshape(oracle, ls))
        assert np.array_equal(got.ravel().view(np.uint32), want.view(np.uint32))


def test_kernel_level_repeat_wraps_indices(backend, oracle):
    """The kernel itself (shape.rs:72-74) wraps: a 3-vector tiled into 10 slots."""
    import ctypes as C
    from vortx_b200 import _lib
    src = np.array([1.0, 2.0, 3.0], np.float32)
    d, s = backend.init_buffer(np.zeros(10, np.float32)), backend.init_buffer(src)
    sr = _lib.VxShape(1, 1, 1, 10, 10, 10, 10, 1)
    ss = _lib.VxShape(1, 1, 1, 3, 3, 3, 3, 1)
    _lib.check(_lib.load().vx_repeat(backend._ctx, d.ptr, C.byref(sr), 10, s.ptr, C.byref(ss), 3))
    got = np.zeros(10, np.float32)
    backend.slow_read_buffer(d, got)
    assert np.array_equal(got, np.tile(src, 4)[:10])
    want = np.zeros(10, np.float32)
    oracle.repeat(want, oracle.Shape(1, 1, 1, 10, 10, 10, 10, 1), src, oracle.Shape(1, 1, 1, 3, 3, 3, 3, 1))
    assert np.array_equal(got, want)


def test_tensor_append_and_shift_remove(backend):
    """src/tensor/tensor_impl.rs:673-815 over stream-ordered copies."""
    t = vb.Tensor.with_capacity(backend, 4)
    assert t.len() == 0 and t.capacity() == 4
    t.append(backend, np.array([1, 2, 3], np.float32))
    assert t.capacity() == 4 and np.array_equal(t.read(backend), [1, 2, 3])
    t.append(backend, np.array([4, 5, 6], np.float32))        # 6 >= 4: grows to the next power of two
    assert t.capacity() == 8 and np.array_equal(t.read(backend), [1, 2, 3, 4, 5, 6])
    assert t.shift_remove(backend, 1, 3) == 2
    assert np.array_equal(t.read(backend), [1, 4, 5, 6]) and t.capacity() == 8
    assert t.shift_remove(backend, 3) == 1 and np.array_equal(t.read(backend), [1, 4, 5])
    assert t.shift_remove(backend, 2, 2) == 0
    with pytest.raises(IndexError):
        t.shift_remove(backend, 1, 9)


# ---- the row, vector and tile forms of the kernels (layouts wide enough to take them) against the oracle and against
# ---- the general kernels ("elementwise.fast" = 0), bit for bit

def _shape(lib_mod, sizes, strides):
    s = lib_mod.VxShape()
    s.n, s.c, s.h, s.w = sizes
    s.n_stride, s.c_stride, s.h_stride, s.w_stride = strides
    return s


def _dense(sizes):
    n, c, h, w = sizes
    return (c * h * w, h * w, w, 1)


_FAST_CASES = [
    # name, sizes of a, strides of a, strides of b, offset a, offset b
    ("dense, float4 rows", (1, 1, 200, 520), None, None, 0, 0),
    ("dense 4-D, float4 rows", (3, 2, 70, 132), None, None, 0, 0),
    ("dense, width not a multiple of 4", (1, 1, 130, 1030), None, None, 0, 0),
    ("dense, rows off 16-byte alignment", (1, 1, 64, 256), (0, 0, 260, 1), (0, 0, 260, 1), 3, 5),
    ("b one row for every row", (1, 2, 90, 512), None, (0, 0, 0, 1), 0, 0),
    ("b one value per row", (1, 2, 90, 512), None, (0, 90, 1, 0), 0, 8),
    ("b one value per row, a off alignment", (1, 1, 90, 512), (0, 0, 513, 1), (0, 0, 1, 0), 1, 0),
    ("b transposed", (1, 1, 100, 70), None, (0, 0, 1, 100), 0, 0),
    ("b transposed, 4-D, ragged tiles", (2, 3, 65, 129), None, (3 * 65 * 129, 65 * 129, 1, 65), 0, 7),
    ("a strided along w", (1, 1, 40, 300), (0, 0, 600, 2), None, 0, 0),
    ("padded rows, float4 rows", (1, 2, 64, 256), (0, 64 * 260, 260, 1), (0, 64 * 264, 264, 1), 4, 8),
    ("padded rows longer than one batch", (1, 1, 5, 4400), (0, 0, 4404, 1), (0, 0, 4408, 1), 0, 0),
    ("dense, rows longer than one batch of float4 per thread", (1, 1, 6, 5000), None, None, 0, 0),
    ("b one row, rows longer than one batch", (1, 1, 5, 4400), None, (0, 0, 0, 1), 0, 0),
    ("b transposed, several tiles each way", (1, 1, 200, 333), None, (0, 0, 1, 200), 0, 0),
]


@pytest.mark.parametrize("op", [OV.Add, OV.Div, OV.Copy])
@pytest.mark.parametrize("case", _FAST_CASES, ids=[c[0] for c in _FAST_CASES])
def test_fast_forms_of_op_assign(backend, oracle, op, case):
    import ctypes as C
    from vortx_b200 import _lib
    lib = _lib.load()
    _, sizes, stra, strb, off_a, off_b = case
    stra = _dense(sizes) if stra is None else stra
    strb = _dense(sizes) if strb is None else strb

    def span(strides):
        return 1 + sum((sz - 1) * st for sz, st in zip(sizes, strides))
    A = synth.uniform_matrix(1, span(stra) + off_a + 4, seed=7).ravel()
    B = (synth.uniform_matrix(1, span(strb) + off_b + 4, seed=8).ravel() + np.float32(1.25)).astype(np.float32)
    want = A.copy()
    oracle.op_assign(op, want, oracle.Shape.of(sizes, stra), B.copy(), oracle.Shape.of(sizes, strb), off_a, off_b)
    sa, sb = _shape(_lib, sizes, stra), _shape(_lib, sizes, strb)
    outs = []
    for fast in (1, 0):
        backend.set_option("elementwise.fast", fast)
        a, b = backend.init_buffer(A), backend.init_buffer(B)
        _lib.check(lib.vx_op_assign(backend._ctx, op, a.ptr, C.byref(sa), A.size, b.ptr, C.byref(sb), B.size, off_a, off_b))
        got = np.empty_like(A)
        backend.slow_read_buffer(a, got)
        outs.append(got)
    backend.set_option("elementwise.fast", 1)
    assert np.array_equal(outs[0].view(np.uint32), want.view(np.uint32))
    assert np.array_equal(outs[1].view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("dtype", [np.float32, np.uint32])
@pytest.mark.parametrize("sizes,strides,offset", [((1, 1, 100, 70), (0, 0, 1, 100), 0),          # a transposed matrix
                                                  ((2, 3, 65, 129), (3 * 65 * 129, 65 * 129, 1, 65), 9),
                                                  ((1, 4, 50, 256), (0, 256, 1024, 1), 0),        # rows of a permuted view
                                                  ((1, 1, 300, 130), (0, 0, 131, 1), 2)])         # a narrowed view
def test_fast_forms_of_contiguous(backend, oracle, dtype, sizes, strides, offset):
    import ctypes as C
    from vortx_b200 import _lib
    lib = _lib.load()
    span = 1 + sum((sz - 1) * st for sz, st in zip(sizes, strides)) + offset
    rng = np.random.Generator(np.random.Philox(11))
    src = rng.integers(0, 2 ** 32, size=span, dtype=np.uint64).astype(np.uint32)        # every bit pattern, NaNs included
    want = oracle.contiguous(src, oracle.Shape.of(sizes, strides), offset)
    s = _shape(_lib, sizes, strides)
    n = int(np.prod(sizes))
    for fast in (1, 0):
        backend.set_option("elementwise.fast", fast)
        sb = backend.init_buffer(src.view(dtype))
        db = backend.init_buffer(np.zeros(n, dtype))
        _lib.check(lib.vx_contiguous(backend._ctx, db.ptr, n, sb.ptr, C.byref(s), span, offset))
        got = np.empty(n, dtype)
        backend.slow_read_buffer(db, got)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    backend.set_option("elementwise.fast", 1)


@pytest.mark.parametrize("rsizes,ssizes", [((1, 1, 37, 300), (1, 1, 5, 7)), ((2, 3, 20, 256), (1, 2, 20, 64)),
                                           ((1, 1, 10, 1000), (1, 1, 1, 1)), ((1, 1, 9, 130), (1, 1, 4, 300)),
                                           ((1, 1, 6, 2048), (1, 1, 3, 12)),      # float4 moves, the source wraps often
                                           ((1, 1, 7, 1000), (1, 1, 2, 8)),       # float4 moves, 256 threads a multiple of the source
                                           ((1, 1, 9, 132), (1, 1, 4, 300))])     # float4 moves, the source is wider
def test_fast_form_of_repeat(backend, oracle, rsizes, ssizes):
    import ctypes as C
    from vortx_b200 import _lib
    lib = _lib.load()
    S = synth.uniform_matrix(1, int(np.prod(ssizes)), seed=12).ravel()
    want = np.zeros(int(np.prod(rsizes)), np.float32)
    oracle.repeat(want, oracle.Shape.of(rsizes, _dense(rsizes)), S.copy(), oracle.Shape.of(ssizes, _dense(ssizes)))
    sr, ss = _shape(_lib, rsizes, _dense(rsizes)), _shape(_lib, ssizes, _dense(ssizes))
    for fast in (1, 0):
        backend.set_option("elementwise.fast", fast)
        rb = backend.init_buffer(np.zeros(want.size, np.float32))
        sb = backend.init_buffer(S)
        _lib.check(lib.vx_repeat(backend._ctx, rb.ptr, C.byref(sr), want.size, sb.ptr, C.byref(ss), S.size))
        got = np.empty_like(want)
        backend.slow_read_buffer(rb, got)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    backend.set_option("elementwise.fast", 1)
