"""vx_reduce_static: the reduction entry point that allocates nothing.

Some hosts cannot allocate when they call into the library — they gave the device to their own arena at
start-up, or they sit in a loop where a cudaMalloc's device-wide stall is unacceptable — so this entry
point keeps its per-block partials in a fixed array inside the library instead of allocated scratch, and
takes a device ordinal and a stream instead of a context.  It must give what vx_reduce's WIDE mode gives.

The file name sorts last on purpose: a run that stops at the first failure has then already run every
other test.  The test also passes alone in a fresh process (it does its own set-up).
"""
import ctypes as C

import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import _lib

pytestmark = pytest.mark.gpu

OPS = {"sum": 0, "prod": 1, "min": 2, "max": 3, "sqnorm": 4}
DTYPES = {np.dtype(np.float32): 0, np.dtype(np.uint32): 1, np.dtype(np.int32): 2}


def _shape(n, stride=1):
    return _lib.VxShape(1, 1, 1, n, n * stride, n * stride, n * stride, stride)


def _both(backend, v, op):
    """The same input through the allocating entry point (WIDE) and the allocation-free one."""
    lib = _lib.load()
    d_in = backend.init_buffer(v)
    d_a = backend.init_buffer(np.zeros(1, v.dtype))
    d_b = backend.init_buffer(np.zeros(1, v.dtype))
    shape = _shape(len(v))
    code = DTYPES[v.dtype]
    _lib.check(lib.vx_reduce(backend._ctx, OPS[op], code, 1, d_in.ptr, C.byref(shape), len(v), d_a.ptr))
    _lib.check(lib.vx_reduce_static(backend.device, C.c_void_p(backend.stream), OPS[op], code, d_in.ptr,
                                    C.byref(shape), d_b.ptr))
    a, b = np.zeros(1, v.dtype), np.zeros(1, v.dtype)
    backend.slow_read_buffer(d_a, a)
    backend.slow_read_buffer(d_b, b)
    return a[0], b[0]


def test_static_reduction_matches_the_allocating_one_twice_in_a_row(backend):
    rng = np.random.Generator(np.random.Philox(11))
    # two calls in a row on different data and sizes: the second must not see the first one's partials
    first = rng.standard_normal(3_000_001, dtype=np.float32)
    second = rng.standard_normal(70_001, dtype=np.float32) + 5.0
    for v in (first, second):
        for op in ("sum", "sqnorm", "min", "max"):
            a, b = _both(backend, v, op)
            exact = {"sum": v.astype(np.float64).sum(), "sqnorm": (v.astype(np.float64) ** 2).sum(),
                     "min": v.min(), "max": v.max()}[op]
            scale = {"sum": np.abs(v).astype(np.float64).sum(), "sqnorm": exact, "min": 1.0, "max": 1.0}[op]
            tol = max(1e-5, 4.0 * np.sqrt(len(v)) * 2.0 ** -24)     # the bar of tests/test_gpu_reduce.py
            assert abs(float(b) - float(exact)) <= tol * max(scale, 1e-30)
            assert abs(float(a) - float(b)) <= 2 * tol * max(scale, 1e-30)   # against the existing entry point
            if op in ("min", "max"):
                assert a == b
    for dtype in (np.uint32, np.int32):
        for v in (rng.integers(0, 1000, size=1_000_003).astype(dtype), rng.integers(1, 3, size=257).astype(dtype)):
            for op in ("sum", "prod", "min", "max"):
                a, b = _both(backend, v, op)
                assert a == b


def test_static_reduction_limits_and_errors(backend):
    lib = _lib.load()
    d = backend.init_buffer(np.ones(8, np.float32))
    out = backend.init_buffer(np.zeros(1, np.float32))
    too_long = _shape(67_108_865)
    st = lib.vx_reduce_static(backend.device, C.c_void_p(backend.stream), 0, 0, d.ptr, C.byref(too_long), out.ptr)
    assert st == _lib.VX_ERR_UNSUPPORTED and b"at most 67108864" in lib.vx_last_error()
    ok = _shape(8)
    assert lib.vx_reduce_static(99, None, 0, 0, d.ptr, C.byref(ok), out.ptr) == _lib.VX_ERR_INVALID_ARGUMENT
    assert lib.vx_reduce_static(backend.device, C.c_void_p(backend.stream), 4, 1, d.ptr, C.byref(ok), out.ptr) \
        == _lib.VX_ERR_UNSUPPORTED                                   # squared norm of integers
    # an empty vector reduces to the operation's identity
    empty = _shape(0)
    _lib.check(lib.vx_reduce_static(backend.device, C.c_void_p(backend.stream), 0, 0, d.ptr, C.byref(empty), out.ptr))
    r = np.ones(1, np.float32)
    backend.slow_read_buffer(out, r)
    assert r[0] == 0.0


def test_static_reduction_leaves_device_memory_alone(backend):
    """What the entry point is for: after the first call on a device (which looks the array's address up and
    loads the code of every kernel it can launch), further calls, of any operation and type, change nothing in
    the device's free memory."""
    import torch
    lib = _lib.load()
    rng = np.random.Generator(np.random.Philox(12))
    inputs = {dt: backend.init_buffer(rng.integers(1, 3, size=200_001).astype(dt)) for dt in (np.float32, np.uint32, np.int32)}
    out = backend.init_buffer(np.zeros(1, np.float32))
    shape = _shape(200_001)
    stream = C.c_void_p(backend.stream)
    _lib.check(lib.vx_reduce_static(backend.device, stream, 0, 0, inputs[np.float32].ptr, C.byref(shape), out.ptr))
    backend.synchronize()
    free_before, _ = torch.cuda.mem_get_info(backend.device)
    for rep in range(3):
        for dt, code in ((np.float32, 0), (np.uint32, 1), (np.int32, 2)):
            for op in range(5 if code == 0 else 4):
                _lib.check(lib.vx_reduce_static(backend.device, stream, op, code, inputs[dt].ptr, C.byref(shape), out.ptr))
    backend.synchronize()
    free_after, _ = torch.cuda.mem_get_info(backend.device)
    assert free_after == free_before
