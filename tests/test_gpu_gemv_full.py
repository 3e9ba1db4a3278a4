"""The Q4_0 GEMV at the sizes the benchmark quotes, against the CPU oracle, and the corner cases of its
fixed-point x: the 28672 x 8192 up-projection as one launch, as the 32-entry list launch the benchmark times,
and as the row slabs 2 / 4 / 8 GPUs would hold (all on one GPU); an x built to hurt the per-chunk fixed point;
NaN, infinity and denormal-range x.

Bars (as in test_gpu_gemv.py): max_i |y_i - t_i| / max_i |t_i| <= 1e-4 against the f64 oracle t and every
element within 2e-6 of its conditioning sum |w||x|.  Reported besides, and asserted: the PER-ELEMENT relative
error |y_i - t_i| / |t_i| over the elements with |t_i| >= 0.1 max|t| stays below 1e-4 too, and within a small
factor of what the f32 oracle itself achieves.
"""
import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import _lib, synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-4
COND_TOL = 2e-6
FLOOR = 0.1     # per-element relative error is taken over |t_i| >= FLOOR * max|t|


def _errors(got, y64, absdot):
    """(norm-wise relative, conditioning-relative, per-element relative over the large elements)."""
    diff = np.abs(got.astype(np.float64) - y64)
    big = np.abs(y64) >= FLOOR * np.abs(y64).max()
    return diff.max() / np.abs(y64).max(), (diff / np.maximum(absdot, 1e-30)).max(), (diff[big] / np.abs(y64[big])).max()


def _check(got, y64, absdot, ref32=None):
    rel, cond, elem = _errors(got, y64, absdot)
    assert rel <= REL_TOL, rel
    assert cond <= COND_TOL, cond
    assert elem <= REL_TOL, elem
    if ref32 is not None:
        # not worse than a few times the f32-accumulated CPU product's own error
        rel32, _, elem32 = _errors(ref32, y64, absdot)
        assert rel <= 4 * rel32 + 1e-6, (rel, rel32)
        assert elem <= 4 * elem32 + 1e-6, (elem, elem32)
    return rel, cond, elem


@pytest.fixture(scope="module")
def up_projection(backend):
    """W 28672 x 8192 ~ N(0, 0.02) quantised to Q4_0 (seed 100, the benchmark's rank-0 matrix at one GPU),
    resident on the device; 32 activation vectors ~ N(0, 1)."""
    rows, cols = 28672, 8192
    blocks = vb.quantize(vb.Q4_0, synth.normal_matrix(rows, cols, seed=100))
    qm = vb.QuantizedMatrix(backend, vb.Q4_0, blocks, rows, cols)
    xs = synth.normal_vectors(32, cols, seed=1)
    yield rows, cols, blocks, qm, xs
    qm.free()


def test_q4_0_28672x8192_single_launch_against_the_oracle(backend, oracle, up_projection, capsys):
    rows, cols, blocks, qm, xs = up_projection
    xd = backend.init_buffer(xs[0])
    yd = backend.init_buffer(np.full(rows, np.nan, np.float32))
    vb.Gemv().dispatch(backend, None, yd, qm, xd)
    got = np.empty(rows, np.float32)
    backend.slow_read_buffer(yd, got)
    y64, absdot = oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, xs[:1])
    y32 = oracle.gemv(vb.Q4_0, blocks, rows, cols, xs[:1], nthreads=oracle.hardware_threads())
    rel, cond, elem = _check(got, y64[0], absdot[0], y32[0])
    with capsys.disabled():
        print(f"\n[q4_0 28672x8192] norm-wise rel {rel:.2e}, conditioning {cond:.2e}, per-element rel {elem:.2e} "
              f"(f32 oracle: {_errors(y32[0], y64[0], absdot[0])[2]:.2e})")


def test_q4_0_28672x8192_list_of_32_against_the_oracle(backend, oracle, up_projection):
    """The benchmark's step: 32 products in ONE persistent launch (here the same matrix with 32 different x, so
    that every entry has its own answer).  Every entry is bit-identical to the same product launched alone, and
    three of them are checked against the f64 oracle."""
    rows, cols, blocks, qm, xs = up_projection
    xd = backend.init_buffer(xs.ravel())
    yd = backend.init_buffer(np.full(32 * rows, np.nan, np.float32))
    batch = vb.GemvBatch(backend, [{"w": qm, "x": xd.ptr + l * cols * 4, "y": yd.ptr + l * rows * 4} for l in range(32)])
    for rep in range(2):
        batch.launch()
    got = np.empty(32 * rows, np.float32)
    backend.slow_read_buffer(yd, got)
    got = got.reshape(32, rows)
    batch.free()
    single = backend.init_buffer(np.full(rows, np.nan, np.float32))
    one = np.empty(rows, np.float32)
    for l in range(32):
        vb.Gemv().dispatch(backend, None, single, qm, xd.ptr + l * cols * 4)
        backend.slow_read_buffer(single, one)
        assert np.array_equal(one.view(np.uint32), got[l].view(np.uint32)), l
    for l in (0, 13, 31):
        y64, absdot = oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, xs[l:l + 1])
        _check(got[l], y64[0], absdot[0])


@pytest.mark.parametrize("world", [2, 4, 8])
def test_q4_0_28672x8192_row_slabs_of_n_gpus_on_one(backend, oracle, up_projection, world):
    """What each of 2 / 4 / 8 GPUs computes (rows / world contiguous rows of W, x replicated), run on one GPU into
    its slice of y: the assembled y is the oracle's, and bit-identical to the unsharded product."""
    from vortx_b200.multi_gpu import row_shard, shard_blocks
    rows, cols, blocks, qm, xs = up_projection
    x = xs[5]
    xd = backend.init_buffer(x)
    yd = backend.init_buffer(np.full(rows, np.nan, np.float32))
    whole = backend.init_buffer(np.full(rows, np.nan, np.float32))
    vb.Gemv().dispatch(backend, None, whole, qm, xd)
    for r in range(world):
        row0, n = row_shard(rows, world, r)
        # the slab as its own weights object, as a rank would hold it
        slab = vb.QuantizedMatrix(backend, vb.Q4_0, shard_blocks(blocks, rows, cols, 18, world, r), n, cols)
        vb.Gemv().dispatch(backend, None, yd.ptr + row0 * 4, slab, xd)
        backend.synchronize()
        slab.free()
    got, full = np.empty(rows, np.float32), np.empty(rows, np.float32)
    backend.slow_read_buffer(yd, got)
    backend.slow_read_buffer(whole, full)
    assert np.array_equal(got.view(np.uint32), full.view(np.uint32))
    y64, absdot = oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, x[None, :])
    _check(got, y64[0], absdot[0])


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
def test_gemv_outliers_in_every_chunk(backend, oracle, qt, capsys):
    """x built against the per-chunk fixed point: every 32 consecutive values hold one of magnitude 1e4 among
    values of magnitude 1e-3, so the small ones keep only about one significant bit next to their chunk's
    maximum.  The product must still be as good as an f32-accumulated one: both errors against the f64 oracle
    are reported, and ours may not exceed a small multiple of the f32 oracle's."""
    rows, cols = 2048, 8192
    rng = np.random.Generator(np.random.Philox(77))
    w = synth.normal_matrix(rows, cols, seed=78)
    x = (rng.standard_normal(cols) * 1e-3).astype(np.float32)
    pos = np.arange(0, cols, 32) + rng.integers(0, 32, size=cols // 32)
    x[pos] = (np.sign(rng.standard_normal(cols // 32)) * 1e4).astype(np.float32)
    blocks = vb.quantize(qt, w)
    qm = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
    xd = backend.init_buffer(x)
    yd = backend.init_buffer(np.full(rows, np.nan, np.float32))
    vb.Gemv().dispatch(backend, None, yd, qm, xd)
    got = np.empty(rows, np.float32)
    backend.slow_read_buffer(yd, got)
    qm.free()
    y64, absdot = oracle.gemv_f64(qt, blocks, rows, cols, x[None, :])
    y32 = oracle.gemv(qt, blocks, rows, cols, x[None, :])
    rel, cond, elem = _check(got, y64[0], absdot[0], y32[0])
    with capsys.disabled():
        r32 = _errors(y32[0], y64[0], absdot[0])
        print(f"\n[outliers, qtype {qt}] ours: norm-wise {rel:.2e}, per-element {elem:.2e}; f32 oracle: {r32[0]:.2e}, {r32[2]:.2e}")
    # and with the outliers removed the small values alone are resolved to full precision
    x_small = x.copy()
    x_small[pos] = 0.0
    qm = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
    xd = backend.init_buffer(x_small)
    vb.Gemv().dispatch(backend, None, yd, qm, xd)
    backend.slow_read_buffer(yd, got)
    qm.free()
    y64, absdot = oracle.gemv_f64(qt, blocks, rows, cols, x_small[None, :])
    _check(got, y64[0], absdot[0])


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("variant", [0, 2])
def test_gemv_nan_inf_and_tiny_x(backend, oracle, qt, variant):
    """A NaN in x makes every row NaN, as through f32 products; an infinity makes every row non-finite; an x
    whose values are all around 1e-31 .. 1e-33 is still multiplied correctly (the fixed point is relative to each
    chunk's own maximum; below about 5e-32 it keeps fewer than 24 bits).  The streaming kernel (variant 2), the register-staged one (0) and the oracle agree."""
    rows, cols = 96, 2048
    w = synth.normal_matrix(rows, cols, seed=5)
    blocks = vb.quantize(qt, w)
    qm = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
    backend.set_option("gemv.variant", variant)
    try:
        base = synth.normal_vectors(1, cols, seed=6)[0]
        yd = backend.init_buffer(np.zeros(rows, np.float32))
        got = np.empty(rows, np.float32)
        for bad, where in ((np.float32(np.nan), 700), (np.float32(np.inf), 1), (np.float32(-np.inf), cols - 1)):
            x = base.copy()
            x[where] = bad
            xd = backend.init_buffer(x)
            vb.Gemv().dispatch(backend, None, yd, qm, xd)
            backend.slow_read_buffer(yd, got)
            want = oracle.gemv(qt, blocks, rows, cols, x[None, :])[0]
            assert not np.isfinite(want).any()
            assert not np.isfinite(got).any()
            if np.isnan(bad):
                assert np.isnan(got).all() and np.isnan(want).all()
        # the context is as usable as before
        for scale in (np.float32(1e-31), np.float32(1e-33)):
            x = base * scale
            xd = backend.init_buffer(x)
            vb.Gemv().dispatch(backend, None, yd, qm, xd)
            backend.slow_read_buffer(yd, got)
            y64, absdot = oracle.gemv_f64(qt, blocks, rows, cols, x[None, :])
            assert np.abs(got - y64[0]).max() / np.abs(y64[0]).max() <= 1e-3      # f32 itself is near its denormal range here
            assert np.abs(got).max() > 0
    finally:
        backend.set_option("gemv.variant", 2)
        qm.free()


@pytest.mark.parametrize("batch", [2, 4, 8])
def test_q4_0_batches_at_full_size_on_the_tensor_cores(backend, oracle, up_projection, batch):
    """Batches of 2 / 4 / 8 vectors over the 28672 x 8192 matrix through the tensor-core batch kernel, every vector
    against the f64 oracle and not worse than a few times the f32 oracle's own error; linearity as a size-independent
    property: the product of x0 + x1 (formed in f32) equals the sum of the two products to within the bars."""
    rows, cols, blocks, qm, xs = up_projection
    x = xs[:batch].copy()
    x[batch - 1] = (xs[0] + xs[1]).astype(np.float32)
    xd = backend.init_buffer(x.ravel())
    yd = backend.init_buffer(np.full(batch * rows, np.nan, np.float32))
    before = backend.launch_count()
    vb.Gemv().dispatch(backend, None, yd, qm, xd, batch=batch)
    assert backend.launch_count() - before == 2                # pre-pass + one pass over the weights
    got = np.empty(batch * rows, np.float32)
    backend.slow_read_buffer(yd, got)
    got = got.reshape(batch, rows)
    y64, absdot = oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, x)
    y32 = oracle.gemv(vb.Q4_0, blocks, rows, cols, x, nthreads=oracle.hardware_threads())
    for v in range(batch):
        _check(got[v], y64[v], absdot[v], y32[v])
    if batch > 2:
        lin = got[0].astype(np.float64) + got[1].astype(np.float64)
        assert np.abs(got[batch - 1] - lin).max() / np.abs(lin).max() <= 2 * REL_TOL


def test_q4_0_8192x8192_batch_of_8_and_three_matrices_sharing_it(backend, oracle):
    """BASELINE.json's 8192 x 8192 shape with 8 vectors: one matrix, and three matrices sharing the vectors in one
    call (vx_gemv_q_multi); both against the f64 oracle, and bit-identical to each other."""
    rows = cols = 8192
    x = synth.normal_vectors(8, cols, seed=1)
    qms, refs = [], []
    for i in range(3):
        blocks = vb.quantize(vb.Q4_0, synth.normal_matrix(rows, cols, seed=i))
        qms.append(vb.QuantizedMatrix(backend, vb.Q4_0, blocks, rows, cols))
        refs.append(oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, x))
    xd = backend.init_buffer(x.ravel())
    yds = [backend.init_buffer(np.full(8 * rows, np.nan, np.float32)) for _ in qms]
    vb.Gemv().dispatch_multi(backend, None, yds, qms, xd, batch=8)
    one = backend.init_buffer(np.full(8 * rows, np.nan, np.float32))
    for qm, yd, (y64, absdot) in zip(qms, yds, refs):
        got = np.empty(8 * rows, np.float32)
        backend.slow_read_buffer(yd, got)
        for v in range(8):
            _check(got.reshape(8, rows)[v], y64[v], absdot[v])
        vb.Gemv().dispatch(backend, None, one, qm, xd, batch=8)
        alone = np.empty(8 * rows, np.float32)
        backend.slow_read_buffer(one, alone)
        assert np.array_equal(alone.view(np.uint32), got.view(np.uint32))
    for qm in qms:
        qm.free()
