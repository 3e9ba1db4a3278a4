"""Failure paths on one GPU, none of which faults, traps or hangs anything.

* A bounded device-side wait that runs out: the kernel gives up after its budget (shortened here through the
  "wait_cycles" option), writes a code into the context's host-visible status word and RETURNS; the next
  vx_synchronize reports VX_ERR_DEVICE_TIMEOUT, and the same context then computes a correct GEMV.  The waits
  are made to run out with data nobody is ever going to deliver: an exchange vector whose header announces a
  generation its pairs do not carry, and a two-rank barrier whose second "rank" is a plain local buffer.
* A device allocation that fails ("debug.fail_alloc_after"): VX_ERR_OUT_OF_MEMORY, nothing leaked, context usable.
"""
import ctypes as C

import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import _lib, synth

pytestmark = pytest.mark.gpu

SHORT_WAIT = 4_000_000      # SM clocks: about 2 ms instead of 0.2 s


def _small_gemv_is_right(backend, oracle):
    rows, cols = 64, 512
    w = synth.normal_matrix(rows, cols, seed=2)
    x = synth.normal_vectors(1, cols, seed=3)
    blocks = vb.quantize(vb.Q4_0, w)
    qm = vb.QuantizedMatrix(backend, vb.Q4_0, blocks, rows, cols)
    xd = backend.init_buffer(x.ravel())
    yd = backend.init_buffer(np.full(rows, np.nan, np.float32))
    vb.Gemv().dispatch(backend, None, yd, qm, xd)
    y = np.empty(rows, np.float32)
    backend.slow_read_buffer(yd, y)
    qm.free()
    y64, _ = oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, x)
    assert np.abs(y - y64[0]).max() / np.abs(y64[0]).max() <= 1e-4


def test_unpack_of_a_vector_that_never_arrives_times_out(backend, oracle):
    lib = _lib.load()
    n = 512
    nbytes = lib.vx_xvec_bytes(n)
    raw = np.zeros(nbytes, np.uint8)
    raw[:4] = np.frombuffer(np.uint32(1).tobytes(), np.uint8)      # header: generation 1; every pair: generation 0
    vec = backend.init_buffer(raw)
    out = backend.init_buffer(np.zeros(n, np.float32))
    backend.synchronize()
    backend.set_option("wait_cycles", SHORT_WAIT)
    try:
        _lib.check(lib.vx_xvec_unpack(backend._ctx, vec.ptr, n, out.ptr))
        with pytest.raises(_lib.VortxError) as e:
            backend.synchronize()
        assert e.value.status == _lib.VX_ERR_DEVICE_TIMEOUT
        assert "stage code 32" in e.value.message
        backend.synchronize()                      # reported once; the status word is clear again
    finally:
        backend.set_option("wait_cycles", 0)
    _small_gemv_is_right(backend, oracle)


def test_flagged_gemv_whose_x_never_arrives_times_out(backend, oracle):
    """The GEMV kernel itself: x is an exchange vector one generation short.  Every block gives up, the launch
    ends by itself, synchronize reports the timeout (code 16: flagged x), the context stays usable."""
    lib = _lib.load()
    n = 1024
    qm = vb.QuantizedMatrix.from_f32(backend, vb.Q4_0, synth.normal_matrix(n, n, seed=4))
    nbytes = lib.vx_xvec_bytes(n)
    raw = np.zeros(nbytes, np.uint8)
    raw[:4] = np.frombuffer(np.uint32(3).tobytes(), np.uint8)
    xv = backend.init_buffer(raw)
    yv = backend.init_buffer(np.zeros(nbytes, np.uint8))
    backend.synchronize()
    backend.set_option("wait_cycles", SHORT_WAIT)
    try:
        _lib.check(lib.vx_gemv_q_rows_exchange(backend._ctx, qm._h, 0, n, xv.ptr, None, None, yv.ptr, None, 0, 0, 1))
        with pytest.raises(_lib.VortxError) as e:
            backend.synchronize()
        assert e.value.status == _lib.VX_ERR_DEVICE_TIMEOUT
        assert "stage code 16" in e.value.message
    finally:
        backend.set_option("wait_cycles", 0)
    qm.free()
    _small_gemv_is_right(backend, oracle)


def test_barrier_with_a_rank_that_never_arrives_times_out(backend, oracle):
    lib = _lib.load()
    mine = backend.init_buffer(np.zeros(64, np.uint32))
    absent = backend.init_buffer(np.zeros(64, np.uint32))          # stands for a peer that never runs its barrier
    flags = (C.c_void_p * 2)(mine.ptr, absent.ptr)
    backend.synchronize()
    backend.set_option("wait_cycles", SHORT_WAIT)
    try:
        _lib.check(lib.vx_peer_barrier(backend._ctx, flags, 2, 0))
        with pytest.raises(_lib.VortxError) as e:
            backend.synchronize()
        assert e.value.status == _lib.VX_ERR_DEVICE_TIMEOUT
        assert "stage code 31" in e.value.message
    finally:
        backend.set_option("wait_cycles", 0)
    # rank 0 did announce itself to the absent rank before it gave up
    seen = np.zeros(64, np.uint32)
    backend.slow_read_buffer(absent, seen)
    assert seen[40] == 1
    _small_gemv_is_right(backend, oracle)


def test_failed_device_allocation_is_reported_and_leaks_nothing(backend, oracle):
    import torch
    lib = _lib.load()
    backend.synchronize()
    free_before, _ = torch.cuda.mem_get_info(backend.device)
    # plain buffer
    backend.set_option("debug.fail_alloc_after", 1)
    p = C.c_void_p()
    st = lib.vx_alloc(backend._ctx, 1 << 20, C.byref(p))
    assert st == _lib.VX_ERR_OUT_OF_MEMORY and not p.value
    # quantised weights: the host staging buffer is released, no device memory is kept
    blocks = vb.quantize(vb.Q4_0, synth.normal_matrix(256, 1024, seed=8))
    backend.set_option("debug.fail_alloc_after", 1)
    with pytest.raises(_lib.VortxError) as e:
        vb.QuantizedMatrix(backend, vb.Q4_0, blocks, 256, 1024)
    assert e.value.status == _lib.VX_ERR_OUT_OF_MEMORY
    # a long GEMV list: its device copy cannot be allocated
    qm = vb.QuantizedMatrix(backend, vb.Q4_0, blocks, 256, 1024)
    x = backend.init_buffer(np.zeros(1024, np.float32))
    y = backend.init_buffer(np.zeros(256, np.float32))
    backend.set_option("debug.fail_alloc_after", 1)
    with pytest.raises(_lib.VortxError) as e:
        vb.GemvBatch(backend, [{"w": qm, "x": x.ptr, "y": y.ptr}] * 12)
    assert e.value.status == _lib.VX_ERR_OUT_OF_MEMORY
    backend.set_option("debug.fail_alloc_after", 0)
    qm.free()
    x.free()
    y.free()
    backend.synchronize()
    free_after, _ = torch.cuda.mem_get_info(backend.device)
    assert free_after >= free_before
    _small_gemv_is_right(backend, oracle)
