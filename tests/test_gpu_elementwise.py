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
