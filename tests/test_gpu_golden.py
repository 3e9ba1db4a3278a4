"""The CUDA path against the committed golden fixtures (tests/golden/, written by make_golden.py)."""
from pathlib import Path

import numpy as np
import pytest

import vortx_b200 as vb

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def test_gemm_golden_bit_exact(backend):
    g = np.load(GOLDEN / "gemm_f32.npz")
    for name in ("m33k65n31", "m64k16n64", "m5k7n3", "m130k40n70"):
        A, B, want = g[f"{name}_A"], g[f"{name}_B"], g[f"{name}_C"]
        m, k = A.shape
        n = B.shape[1]
        a, b = vb.Tensor.matrix(backend, m, k, A), vb.Tensor.matrix(backend, k, n, B)
        for how in ("dispatch", "dispatch_naive", "dispatch_tiled"):
            c = vb.Tensor.matrix(backend, m, n, np.zeros((m, n), np.float32))
            getattr(vb.Gemm(), how)(backend, None, None, c, a, b)
            assert np.array_equal(c.read(backend).view(np.uint32), want.view(np.uint32)), (name, how)


@pytest.mark.parametrize("name,qt", [("gemv_q8_0", vb.Q8_0), ("gemv_q4_0", vb.Q4_0)])
def test_gemv_golden(backend, name, qt):
    g = np.load(GOLDEN / f"{name}.npz")
    for case in ("r17c96b1", "r64c256b4"):
        w, x, blocks = g[f"{case}_w"], g[f"{case}_x"], g[f"{case}_blocks"]
        rows, cols = w.shape
        batch = x.shape[0]
        assert np.array_equal(vb.quantize(qt, w), blocks)
        qm = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
        deq = backend.uninit_buffer(rows * cols)
        qm.dequantize(deq)
        got = np.empty(rows * cols, np.float32)
        backend.slow_read_buffer(deq, got)
        assert np.array_equal(got.view(np.uint32), g[f"{case}_dequant"].ravel().view(np.uint32))
        for variant in (0, 1, 2):
            backend.set_option("gemv.variant", variant)
            xd = backend.init_buffer(x.ravel())
            yd = backend.init_buffer(np.zeros(batch * rows, np.float32))
            vb.Gemv().dispatch(backend, None, yd, qm, xd, batch=batch)
            y = np.empty(batch * rows, np.float32)
            backend.slow_read_buffer(yd, y)
            y = y.reshape(batch, rows)
            y64, absdot = g[f"{case}_y_f64"], g[f"{case}_absdot"]
            assert np.abs(y - y64).max() / np.abs(y64).max() <= 1e-4
            assert (np.abs(y - y64) <= 2e-6 * absdot).all()
        backend.set_option("gemv.variant", 2)
