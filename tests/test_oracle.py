"""CPU tests of the oracle itself: hand-computed known answers, the property the reference's own
GEMM test checks, the committed golden fixtures, and agreement with the library's host-side code.

The reference holds no golden vectors for this path (its one GEMM test compares unseeded random
inputs with a host product to 1e-3, src/linalg/gemm.rs:365-444), so the pins are: answers worked
out by hand below, that replayed property, and the frozen fixtures in tests/golden/.
"""
from pathlib import Path

import numpy as np
import pytest

import oracle as o
import vortx_b200 as vb
from vortx_b200 import synth

GOLDEN = Path(__file__).resolve().parent / "golden"


def _gemm(fn, A, B, *extra):
    m, k = A.shape
    _, n = B.shape
    out = np.zeros(m * n, np.float32)
    fn(out, np.ascontiguousarray(A).ravel(), np.ascontiguousarray(B).ravel(), o.shape_contiguous(1, 1, m, n),
       o.shape_contiguous(1, 1, m, k), o.shape_contiguous(1, 1, k, n), *extra)
    return out.reshape(m, n)


# ---- GEMM ------------------------------------------------------------------------------

def test_gemm_hand_computed():
    A = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    B = np.array([[7, 8], [9, 10], [11, 12]], np.float32)
    want = np.array([[58, 64], [139, 154]], np.float32)
    assert np.array_equal(_gemm(o.gemm_naive, A, B), want)
    assert np.array_equal(_gemm(o.gemm_tiled, A, B, 1), want)


def test_gemm_rounding_order_is_multiply_then_add_ascending_k():
    """acc = fl(acc + fl(a*b)) for k ascending: an input on which a fused multiply-add, or a different
    order, gives a different float."""
    a = np.float32(1 + 2 ** -12)
    A = np.array([[a, a, 1.0]], np.float32)
    B = np.array([[a], [-a], [2 ** -24]], np.float32)
    # fl(a*a) = 1 + 2^-11 (the 2^-24 term is lost); fl(a*a) - fl(a*a) = 0; + 2^-24
    assert _gemm(o.gemm_naive, A, B)[0, 0] == np.float32(2 ** -24)
    B2 = np.array([[2 ** -24], [a], [-a]], np.float32).reshape(3, 1)
    A2 = np.array([[1.0, a, a]], np.float32)
    # 2^-24 first: fl(2^-24 + (1 + 2^-11)) = 1 + 2^-11 (absorbed), then minus the same = 0
    assert _gemm(o.gemm_naive, A2, B2)[0, 0] == np.float32(0.0)


@pytest.mark.parametrize("m,k,n", [(1, 1, 1), (31, 17, 33), (64, 16, 64), (65, 33, 130), (100, 257, 3)])
def test_gemm_naive_equals_tiled_bitwise(m, k, n):
    A, B = synth.uniform_matrix(m, k, 1), synth.uniform_matrix(k, n, 2)
    a, b = _gemm(o.gemm_naive, A, B), _gemm(o.gemm_tiled, A, B, 3)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    assert np.allclose(a, o.gemm_f64(A, B), atol=1e-4)


def test_reference_test_property_256_matvec():
    """src/linalg/gemm.rs:365-444 on the oracle: 256x256 times [256,1], inputs in [0,1), within 1e-3 of a host product."""
    rng = np.random.Generator(np.random.Philox(5))
    M, v = rng.random((256, 256), dtype=np.float32), rng.random((256, 1), dtype=np.float32)
    got = _gemm(o.gemm_dispatch, M, v, 2)
    assert np.allclose(got, M.astype(np.float64) @ v.astype(np.float64), rtol=1e-3, atol=1e-3)


def test_gemm_strided_shapes_and_batch():
    """Shape::it indexing (shape.rs:46-48): a transposed lhs and a 2x3 batch through explicit strides."""
    nb, cb, m, k, n = 2, 3, 5, 7, 4
    At = synth.uniform_matrix(nb * cb * k, m, 3).reshape(nb, cb, k, m)
    B = synth.uniform_matrix(nb * cb * k, n, 4).reshape(nb, cb, k, n)
    so = o.shape_contiguous(nb, cb, m, n)
    sl = o.Shape(nb, cb, m, k, cb * k * m, k * m, 1, m)  # h and w strides swapped: a transposed view
    sr = o.shape_contiguous(nb, cb, k, n)
    for fn, extra in ((o.gemm_naive, ()), (o.gemm_tiled, (2,))):
        out = np.zeros(nb * cb * m * n, np.float32)
        fn(out, At.ravel(), B.ravel(), so, sl, sr, *extra)
        ref = np.einsum("bckm,bckn->bcmn", At.astype(np.float64), B.astype(np.float64))
        assert np.allclose(out.reshape(nb, cb, m, n), ref, atol=1e-5)


def test_gemm_golden():
    g = np.load(GOLDEN / "gemm_f32.npz")
    for name in ("m33k65n31", "m64k16n64", "m5k7n3", "m130k40n70"):
        got = _gemm(o.gemm_dispatch, g[f"{name}_A"], g[f"{name}_B"], 2)
        assert np.array_equal(got.view(np.uint32), g[f"{name}_C"].view(np.uint32)), name


# ---- f16 ---------------------------------------------------------------------------------

def test_f16_conversions_against_table_and_numpy():
    table = np.load(GOLDEN / "f16_table.npz")["f32"]
    idx = np.r_[0:2048, 0x3BF0:0x3C10, 0x7BF0:0x7C01, 0x8000:0x8800, 0xFBF0:0xFC01]
    for h in idx:
        f = o.f16_to_f32(int(h))
        assert np.float32(f).view(np.uint32) == table[h].view(np.uint32)
        assert o.f32_to_f16(float(table[h])) == h
    rng = np.random.Generator(np.random.Philox(9))
    xs = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 3e4)])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    assert all(o.f32_to_f16(float(x)) == w for x, w in zip(xs, want))
    # ties go to even: 1 + 2^-11 is halfway between 1 and 1 + 2^-10
    assert o.f32_to_f16(1.0 + 2.0 ** -11) == 0x3C00
    assert o.f32_to_f16(1.0 + 3 * 2.0 ** -11) == 0x3C02


# ---- quantisation ----------------------------------------------------------------------------

def test_q8_0_hand_computed_block():
    w = np.zeros((1, 32), np.float32)
    w[0, :4] = [127.0, -63.5, 1.0, 0.49]
    blocks = o.quantize(o.Q8_0, w)
    assert blocks.size == 34
    assert int(blocks[0]) | (int(blocks[1]) << 8) == 0x3C00          # d = 127/127 = 1.0
    assert list(blocks[2:6].view(np.int8)) == [127, -64, 1, 0]   # half away from zero: -63.5 -> -64
    assert np.array_equal(o.dequantize(o.Q8_0, blocks, 1, 32)[0, :4], [127.0, -64.0, 1.0, 0.0])


def test_q4_0_hand_computed_block():
    w = np.zeros((1, 32), np.float32)
    w[0, 0], w[0, 1], w[0, 16], w[0, 17] = -7.0, 3.4, 7.0, -2.5
    # largest magnitude is 7 at index 0 (first of the tie) and negative: d = -7 / 7 = -1
    blocks = o.quantize(o.Q4_0, w)
    assert blocks.size == 18
    assert int(blocks[0]) | (int(blocks[1]) << 8) == 0xBC00          # -1.0 in f16
    # q = round(w / d) + 8: -7 -> 15, 3.4 -> -3 + 8 = 5, 7 -> 1, -2.5 -> 3 (2.5 rounds away) + 8 = 11
    assert blocks[2] == (15 | (1 << 4))                    # elements 0 and 16 share byte 0
    assert blocks[3] == (5 | (11 << 4))                    # elements 1 and 17 share byte 1
    assert blocks[4] == (8 | (8 << 4))                     # zeros quantise to 8
    deq = o.dequantize(o.Q4_0, blocks, 1, 32)
    assert np.array_equal(deq[0, [0, 1, 16, 17, 2]], [-7.0, 3.0, 7.0, -3.0, 0.0])


def test_zero_block_and_clamps():
    w = np.zeros((2, 64), np.float32)
    for qt, neutral in ((o.Q8_0, 0), (o.Q4_0, 8 | (8 << 4))):
        b = o.quantize(qt, w)
        bb = o.BLOCK_BYTES[qt]
        assert all(b[i * bb] == 0 and b[i * bb + 1] == 0 for i in range(4))
        assert all(v == neutral for i in range(4) for v in b[i * bb + 2:(i + 1) * bb])
        assert not o.dequantize(qt, b, 2, 64).any()


@pytest.mark.parametrize("qt", [o.Q8_0, o.Q4_0])
def test_library_host_quantiser_matches_oracle(qt):
    w = synth.normal_matrix(37, 320, seed=4)
    w[5, 32:64] = 0.0
    a, b = o.quantize(qt, w), vb.quantize(qt, w)
    assert np.array_equal(a, b)
    assert np.array_equal(o.dequantize(qt, a, 37, 320).view(np.uint32),
                          vb.dequantize_host(qt, b, 37, 320).view(np.uint32))
    # quantisation error bound: half a step of the block's scale (Q4_0 clamps one side to 7 steps)
    deq = o.dequantize(qt, a, 37, 320)
    step = np.abs(w).reshape(37, 10, 32).max(axis=2, keepdims=True) / (127 if qt == o.Q8_0 else 7)
    assert (np.abs(deq - w).reshape(37, 10, 32) <= step * 0.5 * 1.002 + 1e-9).all()


@pytest.mark.parametrize("name,qt", [("gemv_q8_0", o.Q8_0), ("gemv_q4_0", o.Q4_0)])
def test_gemv_golden(name, qt):
    g = np.load(GOLDEN / f"{name}.npz")
    for case in ("r17c96b1", "r64c256b4"):
        w, x, blocks = g[f"{case}_w"], g[f"{case}_x"], g[f"{case}_blocks"]
        rows, cols = w.shape
        assert np.array_equal(o.quantize(qt, w), blocks)
        assert np.array_equal(o.dequantize(qt, blocks, rows, cols).view(np.uint32), g[f"{case}_dequant"].view(np.uint32))
        y = o.gemv(qt, blocks, rows, cols, x, nthreads=2)
        assert np.array_equal(y.view(np.uint32), g[f"{case}_y_f32"].view(np.uint32))
        y64, absdot = o.gemv_f64(qt, blocks, rows, cols, x)
        assert np.allclose(y64, g[f"{case}_y_f64"], rtol=1e-13)
        # the f32 GEMV is the dequantised matrix times x, to f32 rounding
        ref = g[f"{case}_dequant"].astype(np.float64) @ x.astype(np.float64).T
        assert np.allclose(y64, ref.T, rtol=1e-12, atol=1e-12)
        assert (np.abs(y - y64) <= 2e-6 * absdot).all()


def test_gemv_hand_computed():
    # one row, one block: w = d * (q - 8) with d = 0.5; x = 1..32
    blocks = np.zeros(18, np.uint8)
    blocks[0], blocks[1] = 0x00, 0x38            # 0.5 in f16
    q = (np.arange(32) % 16).astype(np.uint8)
    blocks[2:] = q[:16] | (q[16:] << 4)
    x = np.arange(1, 33, dtype=np.float32)
    want = 0.5 * float(((q.astype(np.int32) - 8) * x).sum())
    assert o.gemv(o.Q4_0, blocks, 1, 32, x)[0] == np.float32(want)


# ---- reductions -----------------------------------------------------------------------------------

def test_reduce_known_answers():
    v = np.arange(1, 346, dtype=np.float32)           # the reference test's length, src/linalg/reduce.rs:264
    assert o.reduce(v, "sum") == np.float32(345 * 346 / 2)
    assert o.reduce(v, "min") == 1.0 and o.reduce(v, "max") == 345.0
    assert o.reduce(np.full(10, 2.0, np.float32), "prod") == 1024.0
    assert o.reduce(np.array([3.0, 4.0], np.float32), "sqnorm") == 25.0
    u = np.array([7, 3, 9], np.uint32)
    assert (o.reduce(u, "sum"), o.reduce(u, "prod"), o.reduce(u, "min"), o.reduce(u, "max")) == (19, 189, 3, 9)
    i = np.array([-7, 3, -9], np.int32)
    assert (o.reduce(i, "sum"), o.reduce(i, "prod"), o.reduce(i, "min"), o.reduce(i, "max")) == (-13, 189, -9, 3)
    # the f32 min / max kernels start from +-1e18 (reduce.rs:292-295), which shows on an empty vector
    assert o.reduce(np.zeros(1, np.float32), "min", length=0) == np.float32(1e18)
    # strided walk
    assert o.reduce(np.arange(10, dtype=np.float32), "sum", stride=2) == 20.0
