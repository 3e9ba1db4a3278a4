"""Reductions on the GPU against the CPU oracle's restatement of the reference kernels.

Bars: ORDERED mode bit-identical for every type and operation (it keeps the reference kernel's order);
WIDE mode bit-identical for integers and f32 min / max, and within 1e-5 relative of the f64 value for f32
sum / product / norm, or of 4*sqrt(n)*2^-24 if that is larger (the reference's own test allows 1e-3 at
n = 345, src/linalg/reduce.rs:286)."""
import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import ReduceVariant as RV

pytestmark = pytest.mark.gpu

OPS = {"sum": RV.Sum, "prod": RV.Prod, "min": RV.Min, "max": RV.Max, "sqnorm": RV.SqNorm}


def _data(dtype, n, op, seed):
    rng = np.random.Generator(np.random.Philox(seed))
    if dtype == np.float32:
        if op == "prod":
            return (1.0 + (rng.random(n, dtype=np.float32) - 0.5) * 0.01).astype(np.float32)
        return rng.standard_normal(n, dtype=np.float32)
    info = np.iinfo(dtype)
    return rng.integers(info.min // 2 if op != "prod" else 1, info.max // 2 if op != "prod" else 4, size=n).astype(dtype)


def _gpu(backend, v, op, mode, stride=1):
    t = vb.Tensor.vector(backend, v)
    out = vb.Tensor.scalar(backend, 0, dtype=v.dtype)
    view = t.as_view() if stride == 1 else t.view(0, [len(v) // stride], [stride])
    vb.Reduce(mode=mode).launch(backend, None, None, OPS[op], view, out)
    return out.read(backend)[0]


@pytest.mark.parametrize("n", [0, 1, 127, 128, 129, 345, 4096, 100003])
@pytest.mark.parametrize("dtype", [np.float32, np.uint32, np.int32])
@pytest.mark.parametrize("op", ["sum", "prod", "min", "max", "sqnorm"])
def test_ordered_is_bit_identical(backend, oracle, n, dtype, op):
    if op == "sqnorm" and dtype != np.float32:
        pytest.skip("f32 only")
    v = _data(dtype, max(n, 1), op, seed=n + 1)[:n] if n else np.zeros(1, dtype)[:0]
    with np.errstate(over="ignore"):
        want = oracle.reduce(v if n else np.zeros(1, dtype), op, length=n)
    got = _gpu(backend, v if n else np.zeros(1, dtype), op, vb.Reduce.ORDERED) if n else None
    if n == 0:
        t = vb.Tensor.vector(backend, np.zeros(1, dtype))
        out = vb.Tensor.scalar(backend, 0, dtype=dtype)
        vb.Reduce().launch(backend, None, None, OPS[op], t.as_view().narrow(0, 0, 0), out)
        got = out.read(backend)[0]
    assert np.array([got]).view(np.uint32)[0] == np.array([want], dtype).view(np.uint32)[0], (got, want)


@pytest.mark.parametrize("n", [1, 345, 5000, 1 << 20, 3_000_001])
@pytest.mark.parametrize("dtype", [np.float32, np.uint32, np.int32])
@pytest.mark.parametrize("op", ["sum", "prod", "min", "max", "sqnorm"])
def test_wide_matches(backend, oracle, n, dtype, op):
    if op == "sqnorm" and dtype != np.float32:
        pytest.skip("f32 only")
    v = _data(dtype, n, op, seed=n + 7)
    got = _gpu(backend, v, op, vb.Reduce.WIDE)
    with np.errstate(over="ignore"):
        want = oracle.reduce(v, op)
    if dtype != np.float32 or op in ("min", "max"):
        assert got == want
    else:
        exact = {"sum": lambda a: a.astype(np.float64).sum(), "prod": lambda a: a.astype(np.float64).prod(),
                 "sqnorm": lambda a: (a.astype(np.float64) ** 2).sum()}[op](v)
        scale = {"sum": np.abs(v).astype(np.float64).sum(), "prod": abs(exact), "sqnorm": exact}[op]
        # random-walk growth of f32 rounding over n operations (a product compounds every step)
        tol = max(1e-5, 4.0 * np.sqrt(n) * 2.0 ** -24)
        assert abs(float(got) - exact) <= tol * scale
        assert abs(float(want) - exact) <= tol * scale   # the oracle sits within the same bar


def test_reference_test_replay_len_345(backend):
    """src/linalg/reduce.rs:249-290: a 345-vector, every variant, compared with a host value to 1e-3."""
    rng = np.random.Generator(np.random.Philox(2))
    v = rng.random(345, dtype=np.float32)
    host = {"min": v.min(), "max": v.max(), "sum": v.sum(dtype=np.float64), "prod": v.astype(np.float64).prod(),
            "sqnorm": (v.astype(np.float64) ** 2).sum()}
    for op, want in host.items():
        for mode in (vb.Reduce.ORDERED, vb.Reduce.WIDE):
            got = _gpu(backend, v, op, mode)
            assert abs(float(got) - float(want)) <= 1e-3 * max(1.0, abs(float(want)))


def test_strided_view(backend, oracle):
    v = _data(np.float32, 4000, "sum", seed=5)
    for mode in (vb.Reduce.ORDERED, vb.Reduce.WIDE):
        got = _gpu(backend, v, "sum", mode, stride=4)
        assert abs(float(got) - float(v[::4].astype(np.float64).sum())) < 1e-3
    assert _gpu(backend, v, "sum", vb.Reduce.ORDERED, stride=4) == oracle.reduce(v, "sum", stride=4, length=1000)
