"""vx_gemv_batch_run_host: lists of products with host buffers, the copies overlapped with the kernels.

Same results as the lists launched plainly and read back in one copy (bit for bit), within the GEMV's bars of the
CPU oracle; stages without a copy up or down; bad stages refused with nothing run."""
import ctypes as C

import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def _pinned(n_floats):
    lib = _lib.load()
    p = C.c_void_p()
    _lib.check(lib.vx_host_alloc(n_floats * 4, C.byref(p)))
    arr = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(n_floats,))
    return p, arr


@pytest.mark.parametrize("recorded", [False, True])
@pytest.mark.parametrize("qt", [vb.Q4_0, vb.Q8_0])
@pytest.mark.parametrize("n_stages", [1, 3, 6])
def test_staged_lists_match_the_plain_launch(backend, oracle, qt, n_stages, recorded):
    lib = _lib.load()
    rows, cols, products = 300, 512, 6
    w = synth.normal_matrix(rows, cols, seed=31)
    xs = synth.normal_vectors(products, cols, seed=32)
    blocks = oracle.quantize(qt, w)
    qm = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
    y64, absdot = oracle.gemv_f64(qt, blocks, rows, cols, xs)
    xp, x_host = _pinned(products * cols)
    yp, y_host = _pinned(products * rows)
    x_host[:] = xs.ravel()
    xd = backend.init_buffer(np.zeros(products * cols, np.float32))
    yd = backend.init_buffer(np.zeros(products * rows, np.float32))
    per = products // n_stages
    batches, stages = [], []
    for i in range(n_stages):
        lo = i * per
        batches.append(vb.GemvBatch(backend, [{"w": qm, "x": xd.ptr + l * cols * 4, "y": yd.ptr + l * rows * 4}
                                              for l in range(lo, lo + per)]))
        stages.append({"batch": batches[-1],
                       "up": (xd.ptr + lo * cols * 4, xp.value + lo * cols * 4, per * cols * 4),
                       "down": (yp.value + lo * rows * 4, rows * 4, yd.ptr + lo * rows * 4, rows * 4, rows * 4, per)})
    run = vb.HostStages(backend, stages, recorded=recorded)     # recorded: one CUDA graph replayed per step
    for rep in range(3):                          # streams and events are reused from the second call on
        y_host[:] = np.nan
        if rep == 2:                              # new inputs in the same host buffers: nothing is baked in but pointers
            x_host[:] = xs.ravel()[::-1].copy()
            run.run()
            flipped = y_host.reshape(products, rows).copy()
            x_host[:] = xs.ravel()
            y_host[:] = np.nan
        run.run()
        got = y_host.reshape(products, rows).copy()
        assert np.abs(got - y64).max() / np.abs(y64).max() <= 1e-4
        assert (np.abs(got - y64) <= 2e-6 * absdot).all()
    # the plain way: one copy up, the lists, one copy down
    plain = np.empty(products * rows, np.float32)
    backend.write_buffer(xd, 0, xs.ravel())
    for b in batches:
        b.launch()
    backend.slow_read_buffer(yd, plain)
    assert np.array_equal(plain.view(np.uint32), got.ravel().view(np.uint32))
    y64f, absdotf = oracle.gemv_f64(qt, blocks, rows, cols, xs.ravel()[::-1].copy().reshape(products, cols))
    assert (np.abs(flipped - y64f) <= 2e-6 * absdotf).all()
    run.free()
    for b in batches:
        b.free()
    qm.free()
    _lib.check(lib.vx_host_free(xp))
    _lib.check(lib.vx_host_free(yp))


def test_stages_without_copies_and_bad_stages(backend, oracle):
    lib = _lib.load()
    rows, cols = 64, 256
    blocks = oracle.quantize(vb.Q8_0, synth.normal_matrix(rows, cols, seed=1))
    qm = vb.QuantizedMatrix(backend, vb.Q8_0, blocks, rows, cols)
    x = synth.normal_vectors(1, cols, seed=2)
    xd = backend.init_buffer(x.ravel())
    yd = backend.init_buffer(np.zeros(rows, np.float32))
    batch = vb.GemvBatch(backend, [{"w": qm, "x": xd.ptr, "y": yd.ptr}])
    vb.HostStages(backend, [{"batch": batch}]).run()          # nothing up, nothing down: the list still runs
    y = np.empty(rows, np.float32)
    backend.slow_read_buffer(yd, y)
    y64, absdot = oracle.gemv_f64(vb.Q8_0, blocks, rows, cols, x)
    assert (np.abs(y - y64[0]) <= 2e-6 * absdot[0]).all()
    vb.HostStages(backend, []).run()                          # no stages: a no-op
    before = backend.launch_count()
    bad = (_lib.VxHostStage * 2)()
    bad[0].batch = batch._h
    bad[1].batch = None                                       # a stage without a list: nothing of the call runs
    assert lib.vx_gemv_batch_run_host(backend._ctx, bad, 2) == 1      # VX_ERR_INVALID_ARGUMENT
    bad[1].batch = batch._h
    bad[1].down_host, bad[1].down_device = 1, yd.ptr
    bad[1].down_host_pitch, bad[1].down_device_pitch, bad[1].down_width_bytes, bad[1].down_rows = 4, 256, 256, 1
    assert lib.vx_gemv_batch_run_host(backend._ctx, bad, 2) == 1      # host pitch shorter than a row
    assert backend.launch_count() == before
    # a recorded step refuses pageable host memory (its copies could not be recorded)
    pageable = np.zeros(cols, np.float32)
    stage = (_lib.VxHostStage * 1)()
    stage[0].batch = batch._h
    stage[0].up_device, stage[0].up_host, stage[0].up_bytes = xd.ptr, pageable.ctypes.data, cols * 4
    h = C.c_void_p()
    assert lib.vx_host_pipeline_create(backend._ctx, stage, 1, C.byref(h)) == 1 and not h.value
    assert b"page-locked" in lib.vx_last_error()
    assert lib.vx_host_pipeline_run(None) == 1 and lib.vx_host_pipeline_free(None) == 0
    batch.free()
    qm.free()
