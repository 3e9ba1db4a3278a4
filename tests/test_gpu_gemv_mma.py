"""The tensor-core batch GEMV (vx_gemv_mma.cu) against the CPU oracle, through vx_gemv_q_rows.

Two and more vectors take it by default; "gemv.batch_mma" = 1 sends single vectors through it too, which is
how its one-MMA-per-block form (1 or 2 vectors) is reached.  Bars as for the streaming kernel: max-norm
relative error <= 1e-4 against the f64 oracle and every element within 2e-6 of its conditioning sum |w||x|.
x is held as 22-bit (Q4_0) or 19-bit (Q8_0) fixed point per slice of 128 or 256 columns here, so the second bar
is the tighter one.  The column count must be a multiple of 256.
"""
import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import _lib, synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-4
COND_TOL = 2e-6


def _check(got, y64, absdot):
    rel = np.abs(got - y64).max() / np.abs(y64).max()
    cond = (np.abs(got - y64) / np.maximum(absdot, 1e-30)).max()
    assert rel <= REL_TOL, rel
    assert cond <= COND_TOL, cond


def _run(backend, qm, x, row0=0, nrows=None, x_stride=None, y_stride=None):
    batch = x.shape[0]
    nrows = qm.rows - row0 if nrows is None else nrows
    xs = x.shape[1] if x_stride is None else x_stride
    ys = nrows if y_stride is None else y_stride
    xbuf = np.zeros(batch * xs, np.float32)
    for v in range(batch):
        xbuf[v * xs:v * xs + x.shape[1]] = x[v]
    xd = backend.init_buffer(xbuf)
    yd = backend.init_buffer(np.full(batch * ys, np.nan, np.float32))
    before = backend.launch_count()
    vb.Gemv().dispatch(backend, None, yd, qm, xd, batch=batch, x_stride=xs, y_stride=ys, row0=row0, nrows=nrows)
    launches = backend.launch_count() - before
    y = np.empty(batch * ys, np.float32)
    backend.slow_read_buffer(yd, y)
    out = np.stack([y[v * ys:v * ys + nrows] for v in range(batch)])
    pad = np.concatenate([y[v * ys + nrows:(v + 1) * ys] for v in range(batch)]) if ys > nrows else np.zeros(0)
    assert np.isnan(pad).all()                     # nothing outside the rows is written
    return out, launches


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("rows,cols,batch", [(16, 256, 2), (1, 512, 8), (37, 512, 3), (300, 768, 2), (300, 1536, 5),
                                             (130, 2048, 8), (1000, 4096, 4), (257, 8192, 8), (64, 8192, 2),
                                             (90, 14336, 6), (33, 28672, 8), (48, 1024, 11), (5000, 1024, 7)])
def test_batch_gemv_on_tensor_cores(backend, oracle, qt, rows, cols, batch):
    w = synth.normal_matrix(rows, cols, seed=rows + cols)
    x = synth.normal_vectors(batch, cols, seed=batch)
    blocks = oracle.quantize(qt, w)
    qm = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
    y64, absdot = oracle.gemv_f64(qt, blocks, rows, cols, x)
    got, launches = _run(backend, qm, x)
    assert launches == 2 * -(-batch // 8)          # pre-pass + main kernel per group of eight vectors
    _check(got, y64, absdot)
    # twice in a row from other vectors: planes, partial sums and counters are reused
    x2 = synth.normal_vectors(batch, cols, seed=batch + 50)
    y64b, absdotb = oracle.gemv_f64(qt, blocks, rows, cols, x2)
    got2, _ = _run(backend, qm, x2)
    _check(got2, y64b, absdotb)
    qm.free()


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("rows,cols", [(100, 256), (513, 4096), (2000, 8192), (24, 16384)])
def test_one_and_two_vectors_on_tensor_cores(backend, oracle, qt, batch, rows, cols):
    """The single-MMA form: the eight columns of the MMA are (vector, plane) pairs."""
    w = synth.normal_matrix(rows, cols, seed=rows)
    x = synth.normal_vectors(batch, cols, seed=cols)
    blocks = oracle.quantize(qt, w)
    qm = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
    y64, absdot = oracle.gemv_f64(qt, blocks, rows, cols, x)
    backend.set_option("gemv.batch_mma", 1)
    try:
        got, launches = _run(backend, qm, x)
    finally:
        backend.set_option("gemv.batch_mma", -1)
    assert launches == 2
    _check(got, y64, absdot)
    qm.free()


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("batch", [2, 5])
def test_many_column_phases(backend, oracle, qt, batch):
    """65536 columns: 32 phases of 2048 columns, the planes of a phase loaded while the one before is worked on."""
    rows, cols = 40, 65536
    w = synth.normal_matrix(rows, cols, seed=8)
    x = synth.normal_vectors(batch, cols, seed=9)
    blocks = oracle.quantize(qt, w)
    qm = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
    y64, absdot = oracle.gemv_f64(qt, blocks, rows, cols, x)
    got, launches = _run(backend, qm, x)
    assert launches == 2
    _check(got, y64, absdot)
    qm.free()


@pytest.mark.parametrize("batch", [2, 8])
def test_more_row_tiles_than_one_launch_takes(backend, oracle, batch):
    """120000 rows: 51 row tiles per thread block, more than a launch gives a block (14): the matrix is walked
    by four launches after one pre-pass ("gemv.mma_nbw" = 1 makes two phases out of 512 columns)."""
    rows, cols = 120000, 512
    w = synth.normal_matrix(rows, cols, seed=10)
    x = synth.normal_vectors(batch, cols, seed=11)
    blocks = oracle.quantize(vb.Q4_0, w)
    qm = vb.QuantizedMatrix(backend, vb.Q4_0, blocks, rows, cols)
    y64, absdot = oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, x)
    backend.set_option("gemv.mma_nbw", 1)
    try:
        got, launches = _run(backend, qm, x)
    finally:
        backend.set_option("gemv.mma_nbw", -1)
    import torch
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert launches == 1 + -(-(-(-rows // 16)) // (14 * sms))       # pre-pass + one launch per 14 row tiles per SM
    _check(got, y64, absdot)
    qm.free()


def test_batch_gemv_slabs_strides_and_unaligned_x(backend, oracle):
    rows, cols, batch = 700, 2048, 5
    w = synth.normal_matrix(rows, cols, seed=1)
    x = synth.normal_vectors(batch, cols, seed=2)
    blocks = oracle.quantize(vb.Q4_0, w)
    qm = vb.QuantizedMatrix(backend, vb.Q4_0, blocks, rows, cols)
    y64, absdot = oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, x)
    whole, _ = _run(backend, qm, x)
    # a slab of rows, vectors 3 floats out of 16-byte alignment from each other, y with room between the vectors
    part, _ = _run(backend, qm, x, row0=123, nrows=401, x_stride=cols + 3, y_stride=450)
    assert np.array_equal(part.view(np.uint32), whole[:, 123:524].view(np.uint32))
    _check(whole, y64, absdot)
    qm.free()


@pytest.mark.parametrize("cols,batch", [(1056, 4), (1056, 2)])
def test_batch_gemv_falls_back_when_the_columns_do_not_fit(backend, oracle, cols, batch):
    """Column counts that are not a multiple of 256 go through the streaming kernel, vector by vector."""
    rows = 64
    w = synth.normal_matrix(rows, cols, seed=3)
    x = synth.normal_vectors(batch, cols, seed=4)
    blocks = oracle.quantize(vb.Q4_0, w)
    qm = vb.QuantizedMatrix(backend, vb.Q4_0, blocks, rows, cols)
    y64, absdot = oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, x)
    got, launches = _run(backend, qm, x)
    assert launches == 1                            # one list launch of the streaming kernel
    _check(got, y64, absdot)
    qm.free()


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
def test_batch_gemv_nan_inf_outliers(backend, oracle, qt):
    rows, cols, batch = 96, 4096, 8
    w = synth.normal_matrix(rows, cols, seed=5)
    blocks = oracle.quantize(qt, w)
    qm = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
    x = synth.normal_vectors(batch, cols, seed=6)
    x[1, 700] = np.nan
    x[3, 4095] = np.inf
    rng = np.random.Generator(np.random.Philox(7))
    x[5] = (rng.standard_normal(cols) * 1e-3).astype(np.float32)      # one 1e4 outlier in every 256-column slice
    x[5, np.arange(0, cols, 256) + rng.integers(0, 256, size=cols // 256)] = 1e4
    x[6] *= np.float32(1e-33)
    got, _ = _run(backend, qm, x)
    assert np.isnan(got[1]).all() and not np.isfinite(got[3]).any()
    good = [0, 2, 4, 7]
    y64, absdot = oracle.gemv_f64(qt, blocks, rows, cols, x[good])
    _check(got[good], y64, absdot)
    # the outlier vector: values 1e-7 of their slice's maximum fall below the fixed point's last bit (as they fall
    # below an f32 sum's last bit); the product stays within the max-norm bar
    y64o, _ = oracle.gemv_f64(qt, blocks, rows, cols, x[5:6])
    y32o = oracle.gemv(qt, blocks, rows, cols, x[5:6])
    rel = np.abs(got[5] - y64o[0]).max() / np.abs(y64o[0]).max()
    rel32 = np.abs(y32o[0] - y64o[0]).max() / np.abs(y64o[0]).max()
    print(f"outlier vector, qtype {qt}: max-norm relative error {rel:.2e} (f32 oracle {rel32:.2e})")
    assert rel <= REL_TOL
    y64t, _ = oracle.gemv_f64(qt, blocks, rows, cols, x[6:7])
    assert np.abs(got[6] - y64t[0]).max() / np.abs(y64t[0]).max() <= 1e-3
    qm.free()


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("batch", [1, 2, 8, 11])
def test_several_matrices_share_the_vectors(backend, oracle, qt, batch):
    """vx_gemv_q_multi: matrices of different row counts, one column count, times the same vectors: the planes
    of x are made once per group of eight vectors and one launch walks the matrices.  Bit-identical to the single
    calls through the same kernel."""
    cols = 2048
    rows_of = [300, 16, 1000, 77, 513, 64, 200, 31, 129, 48]          # ten: two launches per group of vectors
    x = synth.normal_vectors(batch, cols, seed=40)
    qms, refs = [], []
    for i, rows in enumerate(rows_of):
        blocks = oracle.quantize(qt, synth.normal_matrix(rows, cols, seed=50 + i))
        qms.append(vb.QuantizedMatrix(backend, qt, blocks, rows, cols))
        refs.append(oracle.gemv_f64(qt, blocks, rows, cols, x))
    ys_stride = max(rows_of) + 5
    xd = backend.init_buffer(x.ravel())
    yds = [backend.init_buffer(np.full(batch * ys_stride, np.nan, np.float32)) for _ in rows_of]
    before = backend.launch_count()
    vb.Gemv().dispatch_multi(backend, None, yds, qms, xd, batch=batch, y_stride=ys_stride)
    launches = backend.launch_count() - before
    assert launches == 3 * -(-batch // 8)              # pre-pass + two main launches (8 + 2 matrices) per 8 vectors
    backend.set_option("gemv.batch_mma", 1)            # the single calls through the same kernel, also for one vector
    try:
        for qm, yd, rows, (y64, absdot) in zip(qms, yds, rows_of, refs):
            got = np.empty(batch * ys_stride, np.float32)
            backend.slow_read_buffer(yd, got)
            got = got.reshape(batch, ys_stride)
            assert np.isnan(got[:, rows:]).all()           # nothing outside the rows is written
            _check(got[:, :rows], y64, absdot)
            single, _ = _run(backend, qm, x)
            assert np.array_equal(single.view(np.uint32), got[:, :rows].view(np.uint32))
    finally:
        backend.set_option("gemv.batch_mma", -1)
    for qm in qms:
        qm.free()


def test_several_matrices_fall_back_and_refuse(backend, oracle):
    cols = 1056                                            # not a multiple of 256: one streaming call per matrix
    x = synth.normal_vectors(3, cols, seed=41)
    qms, refs = [], []
    for i, rows in enumerate((40, 100)):
        blocks = oracle.quantize(vb.Q4_0, synth.normal_matrix(rows, cols, seed=60 + i))
        qms.append(vb.QuantizedMatrix(backend, vb.Q4_0, blocks, rows, cols))
        refs.append(oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, x))
    xd = backend.init_buffer(x.ravel())
    yds = [backend.init_buffer(np.zeros(3 * 100, np.float32)) for _ in qms]
    vb.Gemv().dispatch_multi(backend, None, yds, qms, xd, batch=3)
    for qm, yd, (y64, absdot) in zip(qms, yds, refs):
        got = np.empty(300, np.float32)
        backend.slow_read_buffer(yd, got)
        _check(got.reshape(3, 100)[:, :qm.rows], y64, absdot)
    other = vb.QuantizedMatrix(backend, vb.Q4_0, oracle.quantize(vb.Q4_0, synth.normal_matrix(8, 512, seed=1)), 8, 512)
    with pytest.raises(vb.VortxError):                     # column counts differ
        vb.Gemv().dispatch_multi(backend, None, [yds[0], yds[1]], [qms[0], other], xd, batch=1)
    for qm in qms + [other]:
        qm.free()
