"""The tcgen05 TF32 GEMM against the exact SIMT kernel and the f64 oracle, through the C ABI.

Bar (stated by the benchmark definition): relative Frobenius error of the TF32 result against
the SIMT f32 result <= 5e-3.  TF32 keeps 10 explicit mantissa bits per operand, so the observed
error is near 1e-3 * sqrt(2) / sqrt(3) ~ 5e-4.
"""
import ctypes as C

import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import _lib, synth

pytestmark = pytest.mark.gpu

TOL = 5e-3


def _gemm(backend, how, A, B, out_rows=None):
    m, k = A.shape
    _, n = B.shape
    a = vb.Tensor.matrix(backend, m, k, A)
    b = vb.Tensor.matrix(backend, k, n, B)
    c = vb.Tensor.matrix(backend, m, n, np.full((m, n), np.nan, np.float32))
    getattr(vb.Gemm(), how)(backend, None, None, c, a, b)
    backend.synchronize()
    return c.read(backend), vb.Gemm.last_kernel(backend)


def _rel_fro(x, ref):
    return float(np.linalg.norm(x.astype(np.float64) - ref.astype(np.float64)) / np.linalg.norm(ref.astype(np.float64)))


@pytest.mark.parametrize("tile_m", [128, 256])
@pytest.mark.parametrize("m,k,n", [(128, 32, 256), (128, 64, 256), (256, 128, 512), (128, 8, 32), (1, 4, 4),
                                   (200, 100, 264), (129, 36, 260), (1000, 520, 72), (384, 1024, 768),
                                   (257, 40, 300), (512, 2048, 512)])
def test_tf32_matches_simt(backend, oracle, m, k, n, tile_m):
    backend.set_option("gemm.tf32.tile_m", tile_m)     # both tile shapes on every case
    A = synth.uniform_matrix(m, k, seed=m + k)
    B = synth.uniform_matrix(k, n, seed=n + 3)
    got, kern = _gemm(backend, "dispatch_tf32", A, B)
    backend.set_option("gemm.tf32.tile_m", 0)
    assert kern == "tcgen05_tf32", kern
    ref, _ = _gemm(backend, "dispatch_tiled", A, B)
    assert not np.isnan(got).any()
    assert _rel_fro(got, ref) <= TOL
    # and against the f64 product, so that an error common to both kernels cannot hide
    assert _rel_fro(got, oracle.gemm_f64(A, B)) <= TOL


def test_tf32_exact_on_tf32_representable_inputs(backend):
    """Inputs with at most 10 mantissa bits and small integer products: TF32 loses nothing, f32
    accumulation of exactly representable partial sums is exact, so the result must be exact."""
    rng = np.random.Generator(np.random.Philox(3))
    m, k, n = 256, 96, 512
    A = rng.integers(-8, 9, size=(m, k)).astype(np.float32)
    B = rng.integers(-8, 9, size=(k, n)).astype(np.float32)
    got, kern = _gemm(backend, "dispatch_tf32", A, B)
    assert kern == "tcgen05_tf32"
    assert np.array_equal(got, (A.astype(np.int64) @ B.astype(np.int64)).astype(np.float32))


def test_tf32_falls_back_when_tma_cannot_address(backend):
    """A transposed lhs view has no unit stride along its rows: the call must still succeed, on the SIMT kernel."""
    m, k, n = 96, 64, 128
    At = synth.uniform_matrix(k, m, seed=1)
    B = synth.uniform_matrix(k, n, seed=2)
    at = vb.Tensor.matrix(backend, k, m, At)
    b = vb.Tensor.matrix(backend, k, n, B)
    c = vb.Tensor.matrix(backend, m, n, np.zeros((m, n), np.float32))
    vb.Gemm().dispatch_tf32(backend, None, None, c, at.transpose(0, 1), b)
    assert vb.Gemm.last_kernel(backend) == "simt_tiled_generic"
    ref = At.T.astype(np.float64) @ B.astype(np.float64)
    assert np.allclose(c.read(backend), ref, atol=1e-4)


def test_tf32_batched_and_strided_rows(backend, oracle):
    """A 2 x 2 batch, lhs rows padded (pitch 72 for K = 64): TMA takes pitches, not just dense matrices."""
    nb, cb, m, k, n, pitch = 2, 2, 160, 64, 288, 72
    Abuf = synth.uniform_matrix(nb * cb * m, pitch, seed=5).reshape(nb, cb, m, pitch)
    B = synth.uniform_matrix(nb * cb * k, n, seed=6).reshape(nb, cb, k, n)
    at = vb.Tensor(list(Abuf.shape), 4, backend.init_buffer(Abuf.ravel()))
    bt = vb.Tensor(list(B.shape), 4, backend.init_buffer(B.ravel()))
    ct = vb.Tensor([nb, cb, m, n], 4, backend.init_buffer(np.zeros(nb * cb * m * n, np.float32)))
    vb.Gemm().dispatch_tf32(backend, None, None, ct, at.narrow(3, 0, k), bt)
    assert vb.Gemm.last_kernel(backend) == "tcgen05_tf32"
    got = ct.read(backend)
    ref = np.einsum("bcmk,bckn->bcmn", Abuf[..., :k].astype(np.float64), B.astype(np.float64))
    assert _rel_fro(got, ref) <= TOL


@pytest.mark.parametrize("tile_m", [128, 256])
def test_tf32_4096_against_simt(backend, tile_m):
    """A larger square case (several waves of tiles, both accumulators, the whole ring)."""
    dim = 4096
    A = synth.uniform_matrix(dim, dim, seed=0)
    B = synth.uniform_matrix(dim, dim, seed=1)
    backend.set_option("gemm.tf32.tile_m", tile_m)
    got, kern = _gemm(backend, "dispatch_tf32", A, B)
    backend.set_option("gemm.tf32.tile_m", 0)
    assert kern == "tcgen05_tf32"
    ref, _ = _gemm(backend, "dispatch_tiled", A, B)
    assert _rel_fro(got, ref) <= TOL


def test_tf32_8192_against_simt(backend):
    """The size the GEMM figures are quoted on: 8192^3, A and B uniform [-1, 1) from seeds 0 and 1, tensor-core
    result against the exact SIMT result at 5e-3 relative Frobenius; and the column panels 2 / 4 / 8 GPUs would
    compute, run here one after the other into one C, give the same bits as the unsharded product."""
    import ctypes as C
    lib = _lib.load()
    dim = 8192
    A = synth.uniform_matrix(dim, dim, seed=0)
    B = synth.uniform_matrix(dim, dim, seed=1)
    ad, bd = backend.init_buffer(A.ravel()), backend.init_buffer(B.ravel())
    c_tf32, c_simt, c_panels = (backend.uninit_buffer(dim * dim) for _ in range(3))

    def shapes(ncols):
        sh = _lib.VxShapes3()
        for s, (h, w, hs) in ((sh.out, (dim, ncols, dim)), (sh.lhs, (dim, dim, dim)), (sh.rhs, (dim, ncols, dim))):
            s.n = s.c = 1
            s.h, s.w = h, w
            s.n_stride = s.c_stride = h * hs
            s.h_stride, s.w_stride = hs, 1
        return sh

    sh = shapes(dim)
    _lib.check(lib.vx_gemm_f32(backend._ctx, _lib.VX_GEMM_TF32, c_tf32.ptr, ad.ptr, bd.ptr, C.byref(sh), 0, 0, 0))
    assert vb.Gemm.last_kernel(backend) == "tcgen05_tf32"
    _lib.check(lib.vx_gemm_f32(backend._ctx, _lib.VX_GEMM_SIMT_EXACT, c_simt.ptr, ad.ptr, bd.ptr, C.byref(sh), 0, 0, 0))
    got, ref = np.empty(dim * dim, np.float32), np.empty(dim * dim, np.float32)
    backend.slow_read_buffer(c_tf32, got)
    backend.slow_read_buffer(c_simt, ref)
    rel = _rel_fro(got, ref)
    print("TF32 against SIMT at 8192^3: relative Frobenius error", rel)
    assert rel <= TOL
    # a row of the exact result against the f64 product, to tie the comparison to something outside the library
    row64 = A[77].astype(np.float64) @ B.astype(np.float64)
    assert np.abs(ref.reshape(dim, dim)[77] - row64).max() <= 1e-3
    panels = np.empty(dim * dim, np.float32)
    for world in (2, 4, 8):
        ncols = dim // world
        shp = shapes(ncols)
        _lib.check(lib.vx_memset(backend._ctx, c_panels.ptr, 0xFF, dim * dim * 4))
        for r in range(world):
            _lib.check(lib.vx_gemm_f32(backend._ctx, _lib.VX_GEMM_TF32, c_panels.ptr + r * ncols * 4, ad.ptr,
                                       bd.ptr + r * ncols * 4, C.byref(shp), 0, 0, 0))
        backend.slow_read_buffer(c_panels, panels)
        assert _rel_fro(panels, ref) <= TOL, world
        # the same tensor-core arithmetic per element (k order and tile height do not depend on the panel width)
        assert np.array_equal(panels.view(np.uint32), got.view(np.uint32)), world


@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 520, 200), (129, 72, 40), (1024, 2048, 512)])
def test_tf32_scatter_epilogue_writes_every_destination(backend, m, n, k):
    """vx_gemm_tf32_scatter with two further buffers of the SAME GPU standing in for peers: the epilogue's tiled TMA
    stores must put the bits of the plain tensor-core GEMM into all three, clipped at ragged edges, and nothing
    outside the panel (the panel sits inside a wider C)."""
    import ctypes as C
    from vortx_b200 import _lib
    lib = _lib.load()
    rng = np.random.Generator(np.random.Philox(m * 7 + n))
    a = rng.random((m, k), dtype=np.float32) * 2 - 1
    b = rng.random((k, n), dtype=np.float32) * 2 - 1
    ad, bd = backend.init_buffer(a.ravel()), backend.init_buffer(b.ravel())
    ldc, col0 = n + 24, 8                                    # panel inside a wider C: 16-byte aligned pitch and base
    canary = np.full(m * ldc, np.float32(-7.5))
    outs = [backend.init_buffer(canary) for _ in range(3)]
    ref = backend.init_buffer(canary)
    sh = _lib.VxShapes3()
    for s, (h, w, hs) in ((sh.out, (m, n, ldc)), (sh.lhs, (m, k, k)), (sh.rhs, (k, n, n))):
        s.n = s.c = 1
        s.h, s.w = h, w
        s.n_stride = s.c_stride = h * hs
        s.h_stride, s.w_stride = hs, 1
    _lib.check(lib.vx_gemm_f32(backend._ctx, _lib.VX_GEMM_TF32, ref.ptr + col0 * 4, ad.ptr, bd.ptr, C.byref(sh), 0, 0, 0))
    assert vb.Gemm.last_kernel(backend) == "tcgen05_tf32"
    peers = (C.c_void_p * 2)(outs[1].ptr + col0 * 4, outs[2].ptr + col0 * 4)
    _lib.check(lib.vx_gemm_tf32_scatter(backend._ctx, outs[0].ptr + col0 * 4, ad.ptr, bd.ptr, C.byref(sh), peers, 2))
    want = np.empty(m * ldc, np.float32)
    backend.slow_read_buffer(ref, want)
    w2 = want.reshape(m, ldc)
    assert (w2[:, :col0] == -7.5).all() and (w2[:, col0 + n:] == -7.5).all()
    for o in outs:
        got = np.empty(m * ldc, np.float32)
        backend.slow_read_buffer(o, got)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_tf32_round_to_nearest_on_load_is_no_worse_than_truncation(backend):
    """With "gemm.tf32.round_nearest" (default) the TMA copies round A and B to TF32 to nearest; without it the
    tensor core drops the low mantissa bits.  Both sit inside the 5e-3 bar; rounding must not be the worse one."""
    import ctypes as C
    lib = _lib.load()
    n = 1024
    rng = np.random.Generator(np.random.Philox(99))
    a = rng.random((n, n), dtype=np.float32) * 2 - 1
    b = rng.random((n, n), dtype=np.float32) * 2 - 1
    want = a.astype(np.float64) @ b.astype(np.float64)
    ad, bd, cd = backend.init_buffer(a.ravel()), backend.init_buffer(b.ravel()), backend.uninit_buffer(n * n)
    sh = _lib.VxShapes3()
    for s in (sh.out, sh.lhs, sh.rhs):
        s.n = s.c = 1
        s.h = s.w = n
        s.n_stride = s.c_stride = n * n
        s.h_stride, s.w_stride = n, 1
    err = {}
    for rn in (0, 1):
        backend.set_option("gemm.tf32.round_nearest", rn)
        _lib.check(lib.vx_gemm_f32(backend._ctx, _lib.VX_GEMM_TF32, cd.ptr, ad.ptr, bd.ptr, C.byref(sh), 0, 0, 0))
        got = np.empty(n * n, np.float32)
        backend.slow_read_buffer(cd, got)
        err[rn] = np.linalg.norm(got.reshape(n, n) - want) / np.linalg.norm(want)
    backend.set_option("gemm.tf32.round_nearest", 1)
    print("relative Frobenius error: truncation", err[0], "round to nearest", err[1])
    assert err[0] <= 5e-3 and err[1] <= 5e-3
    assert err[1] <= err[0] * 1.05
