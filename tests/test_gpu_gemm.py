"""GPU parity of the f32 GEMM against the CPU oracle, through the C ABI.

Bar: the SIMT kernels are bit-identical to the oracle's restatement of gemm_naive /
gemm_tiled (vortx-shaders/src/linalg/gemm.rs) on the same seeded inputs.
"""
import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import synth

pytestmark = pytest.mark.gpu


def _oracle_gemm(o, A, B, out_shape_sizes=None):
    m, k = A.shape
    _, n = B.shape
    so, sl, sr = o.shape_contiguous(1, 1, m, n), o.shape_contiguous(1, 1, m, k), o.shape_contiguous(1, 1, k, n)
    out = np.zeros(m * n, np.float32)
    o.gemm_dispatch(out, np.ascontiguousarray(A).ravel(), np.ascontiguousarray(B).ravel(), so, sl, sr,
                    o.hardware_threads())
    return out.reshape(m, n)


def _gpu_gemm(backend, A, B, how="dispatch"):
    gemm = vb.Gemm.from_backend(backend)
    shapes = vb.TensorLayoutBuffers(backend)
    m, k = A.shape
    _, n = B.shape
    a = vb.Tensor.matrix(backend, m, k, A)
    b = vb.Tensor.matrix(backend, k, n, B)
    c = vb.Tensor.matrix(backend, m, n, np.full((m, n), np.nan, np.float32))
    enc = backend.begin_encoding()
    p = enc.begin_pass("gemm", None)
    getattr(gemm, how)(backend, shapes, p, c, a, b)
    backend.submit(enc)
    backend.synchronize()
    return c.read(backend), vb.Gemm.last_kernel(backend)


@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (5, 7, 3), (31, 31, 31), (32, 16, 8), (33, 65, 31),
                                   (64, 64, 64), (65, 17, 129), (128, 128, 128), (200, 100, 52),
                                   (256, 256, 1), (257, 33, 260)])
@pytest.mark.parametrize("how", ["dispatch", "dispatch_naive", "dispatch_tiled"])
def test_gemm_bit_exact_small(backend, oracle, m, k, n, how):
    A = synth.uniform_matrix(m, k, seed=m * 1000 + k)
    B = synth.uniform_matrix(k, n, seed=n * 77 + 1)
    want = _oracle_gemm(oracle, A, B)
    got, kern = _gpu_gemm(backend, A, B, how)
    assert got.shape == want.shape
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (kern, np.abs(got - want).max())


def test_gemm_1024_config0_bit_exact(backend, oracle):
    """BASELINE config 0: M=N=K=1024, uniform[-1,1) from seed 0, row-major contiguous."""
    A = synth.uniform_matrix(1024, 1024, seed=0)
    B = synth.uniform_matrix(1024, 1024, seed=1)
    want = _oracle_gemm(oracle, A, B)
    for how in ("dispatch", "dispatch_naive"):
        got, kern = _gpu_gemm(backend, A, B, how)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), kern
    assert vb.Gemm.last_kernel(backend) == "naive"


def test_reference_test_replay_256_matvec(backend):
    """src/linalg/gemm.rs:365-444: 256x256 matrix times a 256-vector reshaped [256,1], compared
    with a host product within epsilon 1e-3 (inputs uniform in [0,1) as nalgebra's new_random)."""
    rng = np.random.Generator(np.random.Philox(5))
    m_cpu = rng.random((256, 256), dtype=np.float32)
    v_cpu = rng.random(256, dtype=np.float32)
    gemm = vb.Gemm.from_backend(backend)
    shapes = vb.TensorLayoutBuffers(backend)
    m = vb.Tensor.matrix_from_na(backend, m_cpu)
    v = vb.Tensor.vector(backend, v_cpu)
    v.unsqueeze(1)
    result = vb.Tensor.vector(backend, np.zeros(256, np.float32), vb.BufferUsages.STORAGE | vb.BufferUsages.COPY_SRC)
    result.unsqueeze(1)
    enc = backend.begin_encoding()
    p = enc.begin_pass("gemm", None)
    gemm.dispatch(backend, shapes, p, result, m, v)
    backend.submit(enc)
    backend.synchronize()
    gpu = np.empty(256, np.float32)
    backend.slow_read_buffer(result.buffer(), gpu)
    cpu = m_cpu.astype(np.float64) @ v_cpu.astype(np.float64)
    assert np.allclose(gpu, cpu, rtol=1e-3, atol=1e-3)


def test_gemm_strided_views_and_batches(backend, oracle):
    """Transposed lhs, column-narrowed rhs, a 2x3 batch: generic-stride kernel, bit-exact."""
    o = oracle
    n_b, c_b, m, k, n = 2, 3, 37, 29, 41
    A = synth.uniform_matrix(n_b * c_b * k, m, seed=3).reshape(n_b, c_b, k, m)   # stored transposed
    B = synth.uniform_matrix(n_b * c_b * k, n + 7, seed=4).reshape(n_b, c_b, k, n + 7)
    at = vb.Tensor(list(A.shape), 4, backend.init_buffer(A.ravel()))
    bt = vb.Tensor(list(B.shape), 4, backend.init_buffer(B.ravel()))
    ct = vb.Tensor([n_b, c_b, m, n], 4, backend.init_buffer(np.zeros(n_b * c_b * m * n, np.float32)))
    lhs = at.transpose(2, 3)
    rhs = bt.narrow(3, 5, n)
    gemm = vb.Gemm.from_backend(backend)
    gemm.dispatch(backend, vb.TensorLayoutBuffers(backend), None, ct, lhs, rhs)
    got = ct.read(backend)
    assert vb.Gemm.last_kernel(backend) == "simt_tiled_generic"
    # oracle on the same buffers and shapes
    ll, lr, lo = lhs.layout().canonicalize(), rhs.layout().canonicalize(), ct.layout().canonicalize()
    sl = o.Shape.of(ll.size, ll.stride)
    sr = o.Shape.of(lr.size, lr.stride)
    so = o.Shape.of(lo.size, lo.stride)
    want = np.zeros(n_b * c_b * m * n, np.float32)
    o.gemm_dispatch(want, A.ravel(), B.ravel()[rhs.layout().offset:].copy(), so, sl, sr, 4)
    assert np.array_equal(got.ravel().view(np.uint32), want.view(np.uint32))
    ref = np.einsum("bckm,bckn->bcmn", A.astype(np.float64), B[..., 5:5 + n].astype(np.float64))
    assert np.allclose(got, ref, atol=1e-4)


def test_gemm_shape_mismatch_is_refused(backend):
    a = vb.Tensor.matrix(backend, 4, 5, np.zeros((4, 5), np.float32))
    b = vb.Tensor.matrix(backend, 6, 3, np.zeros((6, 3), np.float32))
    c = vb.Tensor.matrix(backend, 4, 3, np.zeros((4, 3), np.float32))
    with pytest.raises(AssertionError):
        vb.Gemm().dispatch(backend, None, None, c, a, b)
