"""GPU parity of the Q8_0 / Q4_0 GEMV and dequantisation against the CPU oracle, through the C ABI.

Bars: dequantised weights bit-exact; GEMV outputs within max relative error 1e-4, where the
relative error of an output vector is max_i |y_i - t_i| / max_i |t_i| against the f64
oracle t, and additionally every element within 2e-6 of its own conditioning sum |w||x|.
"""
import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import synth

pytestmark = pytest.mark.gpu

REL_TOL = 1e-4
COND_TOL = 2e-6


def _check(got, y64, absdot):
    rel = np.abs(got - y64).max() / np.abs(y64).max()
    cond = (np.abs(got - y64) / np.maximum(absdot, 1e-30)).max()
    assert rel <= REL_TOL, rel
    assert cond <= COND_TOL, cond
    return rel


def _run(backend, qt, blocks, rows, cols, x, **kw):
    w = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
    batch = x.shape[0]
    xd = backend.init_buffer(x.ravel())
    yd = backend.init_buffer(np.full(batch * rows, np.nan, np.float32))
    vb.Gemv().dispatch(backend, None, yd, w, xd, batch=batch, **kw)
    y = np.empty(batch * rows, np.float32)
    backend.slow_read_buffer(yd, y)
    w.free()
    return y.reshape(batch, rows)


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 64), (17, 96), (64, 256), (100, 1056), (513, 4096)])
def test_dequant_bit_exact(backend, oracle, qt, rows, cols):
    w = synth.normal_matrix(rows, cols, seed=rows + cols)
    blocks = oracle.quantize(qt, w)
    assert np.array_equal(blocks, vb.quantize(qt, w))  # product quantiser == oracle quantiser
    want = oracle.dequantize(qt, blocks, rows, cols)
    qm = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
    out = backend.uninit_buffer(rows * cols)
    qm.dequantize(out)
    got = np.empty(rows * cols, np.float32)
    backend.slow_read_buffer(out, got)
    assert np.array_equal(got.view(np.uint32), want.ravel().view(np.uint32))


@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("rows,cols,batch", [(1, 32, 1), (7, 96, 1), (33, 1056, 2), (257, 2048, 1),
                                             (64, 256, 4), (130, 512, 8), (96, 4096, 3), (40, 512, 11)])
def test_gemv_small(backend, oracle, qt, rows, cols, batch, variant):
    backend.set_option("gemv.variant", variant)
    w = synth.normal_matrix(rows, cols, seed=11 * rows + cols)
    x = synth.normal_vectors(batch, cols, seed=rows)
    blocks = oracle.quantize(qt, w)
    y64, absdot = oracle.gemv_f64(qt, blocks, rows, cols, x)
    for rpw in (1, 2, 4):
        backend.set_option("gemv.rows_per_warp", rpw)
        got = _run(backend, qt, blocks, rows, cols, x)
        _check(got, y64, absdot)
    backend.set_option("gemv.rows_per_warp", 2)
    backend.set_option("gemv.variant", 2)
    # the f32 oracle itself sits within the same bar
    _check(oracle.gemv(qt, blocks, rows, cols, x), y64, absdot)


def test_gemv_q8_0_config1(backend, oracle):
    """BASELINE config 1: Q8_0, W 4096x4096 ~ N(0, 0.02), x ~ N(0,1), seeds 0 and 1."""
    rows = cols = 4096
    w = synth.normal_matrix(rows, cols, seed=0)
    x = synth.normal_vectors(1, cols, seed=1)
    blocks = vb.quantize(vb.Q8_0, w)
    y64, absdot = oracle.gemv_f64(vb.Q8_0, blocks, rows, cols, x)
    _check(_run(backend, vb.Q8_0, blocks, rows, cols, x), y64, absdot)


@pytest.mark.parametrize("batch", [1, 4, 8])
def test_gemv_q4_0_config2(backend, oracle, batch):
    """BASELINE config 2: Q4_0, W 8192x8192, batch 1/4/8."""
    rows = cols = 8192
    w = synth.normal_matrix(rows, cols, seed=0)
    x = synth.normal_vectors(batch, cols, seed=1)
    blocks = vb.quantize(vb.Q4_0, w)
    y64, absdot = oracle.gemv_f64(vb.Q4_0, blocks, rows, cols, x)
    _check(_run(backend, vb.Q4_0, blocks, rows, cols, x), y64, absdot)


def test_gemv_row_slab_matches_full(backend, oracle):
    """Row-sharded call (rows [r0, r0+n)) equals the matching slice of the full product."""
    rows, cols = 448, 1024
    w = synth.normal_matrix(rows, cols, seed=9)
    x = synth.normal_vectors(1, cols, seed=10)
    blocks = vb.quantize(vb.Q4_0, w)
    full = _run(backend, vb.Q4_0, blocks, rows, cols, x)
    part = _run(backend, vb.Q4_0, blocks, rows, cols, x, row0=112, nrows=224)
    assert np.array_equal(part[0, :224].view(np.uint32), full[0, 112:336].view(np.uint32))
    assert np.isnan(part[0, 224:]).all()  # nothing beyond the slab is written


def test_gemv_linearity_full_size(backend):
    """Size-independent property at the 28672x8192 shape: W(a x1 + b x2) = a W x1 + b W x2 (to rounding)."""
    rows, cols = 28672, 8192
    rng = np.random.Generator(np.random.Philox(42))
    # random block stream directly (any bytes are valid Q4_0 once the scale is a sane f16)
    nblocks = rows * cols // 32
    blocks = rng.integers(0, 256, size=(nblocks, 18), dtype=np.uint8)
    scales = (rng.random(nblocks, dtype=np.float32) * 0.01 + 0.001).astype(np.float16).view(np.uint16)
    blocks[:, 0] = scales & 0xFF
    blocks[:, 1] = scales >> 8
    x1, x2 = synth.normal_vectors(2, cols, seed=7)
    xs = np.stack([x1, x2, 2.0 * x1 - 0.5 * x2]).astype(np.float32)
    y = _run(backend, vb.Q4_0, blocks.ravel(), rows, cols, xs)
    lin = 2.0 * y[0].astype(np.float64) - 0.5 * y[1].astype(np.float64)
    assert np.abs(y[2] - lin).max() / np.abs(lin).max() < 1e-5


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("n", [256, 1024, 4096, 16384])
def test_exchange_chain_on_one_gpu_matches_plain_chain(backend, qt, n):
    """The flagged form of the GEMV (x read from {value, generation} pairs, rows written as pairs) with no
    peers: a chain of square products ends on the same bits as the same chain through plain vectors."""
    from vortx_b200 import _lib
    lib = _lib.load()
    links = 5
    w = synth.normal_matrix(n, n, seed=n + 5) * np.float32(50.0 / np.sqrt(n))
    blocks = vb.quantize(qt, w)
    x0 = synth.normal_vectors(1, n, seed=3)[0]
    xd = backend.init_buffer(x0)
    full = vb.QuantizedMatrix(backend, qt, blocks, n, n)
    # plain chain
    ya = backend.uninit_buffer(n)
    yb = backend.uninit_buffer(n)
    src = xd
    for l in range(links):
        dst = ya if l % 2 == 0 else yb
        vb.Gemv().dispatch(backend, None, dst, full, src)
        src = dst
    want = np.empty(n, np.float32)
    backend.slow_read_buffer(src, want)
    # flagged chain
    nbytes = lib.vx_xvec_bytes(n)
    assert nbytes == 256 + 8 * n
    vecs = [backend.uninit_buffer(nbytes, dtype=np.uint8) for _ in range(2)]
    for v in vecs:
        _lib.check(lib.vx_memset(backend._ctx, v.ptr, 0, nbytes))
    out = backend.uninit_buffer(n)
    plain = backend.uninit_buffer(n)
    got = np.empty(n, np.float32)
    for rep in range(2):                      # twice: generations keep advancing
        for l in range(links):
            _lib.check(lib.vx_gemv_q_rows_exchange(
                backend._ctx, full._h, 0, n, vecs[(l - 1) % 2].ptr if l else None, xd.ptr if l == 0 else None,
                plain.ptr, vecs[l % 2].ptr, None, 0, 0, 1))
        _lib.check(lib.vx_xvec_unpack(backend._ctx, vecs[(links - 1) % 2].ptr, n, out.ptr))
        backend.slow_read_buffer(out, got)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        backend.slow_read_buffer(plain, got)   # the plain copy of the last link's rows
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("rows,cols,count", [(8, 64, 3), (100, 1056, 5), (1300, 2048, 7), (7000, 4096, 4),
                                             (3000, 8192, 6), (64, 16384, 3)])
def test_batch_of_independent_gemvs_matches_single_launches(backend, qt, rows, cols, count):
    """One persistent launch over a list of products (different weights, row counts and x) gives the bits the
    products give when launched one by one."""
    ws, entries, singles = [], [], []
    xs = synth.normal_vectors(2, cols, seed=cols)
    xd = backend.init_buffer(xs.ravel())
    for i in range(count):
        r = max(1, rows - 37 * i)             # ragged row counts: the tile rotation differs per entry
        w = vb.QuantizedMatrix.from_f32(backend, qt, synth.normal_matrix(r, cols, seed=100 * i + rows))
        ws.append(w)
        xp = xd.ptr + ((i // 2) % 2) * cols * 4   # two x in turn: every other entry shares it with its predecessor
        ya = backend.init_buffer(np.full(r, np.nan, np.float32))
        yb = backend.init_buffer(np.full(r, np.nan, np.float32))
        entries.append({"w": w, "x": xp, "y": ya.ptr})
        singles.append((w, xp, ya, yb, r))
    batch = vb.GemvBatch(backend, entries)
    for rep in range(2):
        batch.launch()
    for w, xp, ya, yb, r in singles:
        vb.Gemv().dispatch(backend, None, yb, w, xp)
        a, b = np.empty(r, np.float32), np.empty(r, np.float32)
        backend.slow_read_buffer(ya, a)
        backend.slow_read_buffer(yb, b)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    batch.free()


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("n", [256, 2048, 8192])
def test_batch_chain_through_exchange_vectors_on_one_gpu(backend, qt, n):
    """A chain of dependent products in ONE launch: each entry reads the exchange vector its predecessor
    writes, pair by pair as other thread blocks of the same grid deliver them.  Same bits as the plain chain."""
    from vortx_b200 import _lib
    lib = _lib.load()
    links = 6
    w = synth.normal_matrix(n, n, seed=n + 9) * np.float32(50.0 / np.sqrt(n))
    full = vb.QuantizedMatrix.from_f32(backend, qt, w)
    x0 = synth.normal_vectors(1, n, seed=4)[0]
    xd = backend.init_buffer(x0)
    ya, yb = backend.uninit_buffer(n), backend.uninit_buffer(n)
    src = xd
    for l in range(links):
        dst = ya if l % 2 == 0 else yb
        vb.Gemv().dispatch(backend, None, dst, full, src)
        src = dst
    want = np.empty(n, np.float32)
    backend.slow_read_buffer(src, want)
    nbytes = lib.vx_xvec_bytes(n)
    vecs = [backend.uninit_buffer(nbytes, dtype=np.uint8) for _ in range(2)]
    for v in vecs:
        _lib.check(lib.vx_memset(backend._ctx, v.ptr, 0, nbytes))
    entries = [{"w": full, "x": xd.ptr, "y_xvec": vecs[0].ptr}]
    for l in range(1, links):
        entries.append({"w": full, "x_xvec": vecs[(l - 1) % 2].ptr, "y_xvec": vecs[l % 2].ptr})
    batch = vb.GemvBatch(backend, entries)
    out = backend.uninit_buffer(n)
    got = np.empty(n, np.float32)
    for rep in range(3):                       # generations advance by three per vector and launch
        batch.launch()
        _lib.check(lib.vx_xvec_unpack(backend._ctx, vecs[(links - 1) % 2].ptr, n, out.ptr))
        backend.slow_read_buffer(out, got)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    batch.free()


@pytest.mark.parametrize("qt,rows,cols", [(vb.Q4_0, 40, 28672), (vb.Q4_0, 19, 32768), (vb.Q8_0, 33, 14336),
                                          (vb.Q8_0, 12, 16384)])
def test_gemv_long_rows(backend, oracle, qt, rows, cols):
    """Rows too long for two 8-row stages stream in tiles of 4 rows (the down-projection shape, 28672 columns)."""
    w = synth.normal_matrix(rows, cols, seed=rows + cols)
    x = synth.normal_vectors(2, cols, seed=rows)
    blocks = oracle.quantize(qt, w)
    y64, absdot = oracle.gemv_f64(qt, blocks, rows, cols, x)
    _check(_run(backend, qt, blocks, rows, cols, x), y64, absdot)


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("rows,cols,pad", [(1, 32, 0), (37, 96, 0), (300, 1056, 32), (64, 4096, 0), (129, 2048, 5)])
def test_device_quantiser_matches_host_quantiser(backend, oracle, qt, rows, cols, pad):
    """vx_qweights_from_device gives the very weights vx_quantize + upload give: dequantised planes and GEMV
    outputs are bit-identical.  Ties, zero blocks, extreme magnitudes and unaligned row strides included."""
    w = synth.normal_matrix(rows, cols, seed=3 * rows + cols).copy()
    w[0, :32] = 0.0                                   # a zero block: neutral quants
    if cols >= 64:
        w[0, 32:64] = np.float32(0.5)                 # all equal: the first element fixes the scale
        w[0, 40] = np.float32(-0.5)                   # same magnitude later on: must not take over
    w[rows - 1, :8] = np.float32([1e-30, -1e-30, 65000.0, -3e4, 7.0, -7.0, 3.5, -3.5])
    stride = cols + pad
    padded = np.zeros((rows, stride), np.float32)
    padded[:, :cols] = w
    wd = backend.init_buffer(padded.ravel())
    on_dev = vb.QuantizedMatrix.from_device_f32(backend, qt, wd.ptr, rows, cols, stride)
    on_host = vb.QuantizedMatrix(backend, qt, oracle.quantize(qt, w), rows, cols)
    outs = []
    for qm in (on_dev, on_host):
        buf = backend.uninit_buffer(rows * cols)
        qm.dequantize(buf)
        got = np.empty(rows * cols, np.float32)
        backend.slow_read_buffer(buf, got)
        outs.append(got)
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
    x = synth.normal_vectors(1, cols, seed=9)
    xd = backend.init_buffer(x.ravel())
    ys = []
    for qm in (on_dev, on_host):
        yd = backend.init_buffer(np.full(rows, np.nan, np.float32))
        vb.Gemv().dispatch(backend, None, yd, qm, xd)
        y = np.empty(rows, np.float32)
        backend.slow_read_buffer(yd, y)
        ys.append(y)
    assert np.array_equal(ys[0].view(np.uint32), ys[1].view(np.uint32))


def test_batch_rejects_what_it_cannot_run(backend):
    """A list refuses mixed formats or column counts, entries without x or y, rows outside the matrix and an
    entry that reads the vector it writes — with a status, before anything is launched."""
    from vortx_b200 import _lib
    w4 = vb.QuantizedMatrix.from_f32(backend, vb.Q4_0, synth.normal_matrix(16, 64, seed=1))
    w8 = vb.QuantizedMatrix.from_f32(backend, vb.Q8_0, synth.normal_matrix(16, 64, seed=2))
    wide = vb.QuantizedMatrix.from_f32(backend, vb.Q4_0, synth.normal_matrix(16, 128, seed=3))
    x = backend.init_buffer(np.zeros(128, np.float32))
    y = backend.uninit_buffer(64)
    vec = backend.init_buffer(np.zeros(256 + 8 * 64, np.uint8))
    before = backend.launch_count()
    good = {"w": w4, "x": x.ptr, "y": y.ptr}
    for bad, status in (([good, {"w": w8, "x": x.ptr, "y": y.ptr}], _lib.VX_ERR_UNSUPPORTED),
                        ([good, {"w": wide, "x": x.ptr, "y": y.ptr}], _lib.VX_ERR_UNSUPPORTED),
                        ([{"w": w4, "y": y.ptr}], _lib.VX_ERR_INVALID_ARGUMENT),
                        ([{"w": w4, "x": x.ptr}], _lib.VX_ERR_INVALID_ARGUMENT),
                        ([{"w": w4, "x": x.ptr, "y": y.ptr, "row0": 10, "nrows": 7}], _lib.VX_ERR_OUT_OF_BOUNDS),
                        ([{"w": w4, "x_xvec": vec.ptr, "y_xvec": vec.ptr}], _lib.VX_ERR_INVALID_ARGUMENT)):
        with pytest.raises(_lib.VortxError) as e:
            vb.GemvBatch(backend, bad)
        assert e.value.status == status, e.value
    assert backend.launch_count() == before


@pytest.mark.parametrize("qt", [vb.Q8_0, vb.Q4_0])
@pytest.mark.parametrize("at_end", [False, True])
@pytest.mark.parametrize("rows,cols,segs", [(1024, 512, 2), (4096, 2048, 4), (3584, 1024, 8)])
def test_batch_chain_with_windowed_x(backend, qt, rows, cols, segs, at_end):
    """rows > cols: the next product's x is a window of the previous y — the first cols / segs elements of each of
    `segs` equal slabs, or the last ones (what a row-sharded chain reads: a piece of every rank's slab).  One list launch against
    the same chain done with plain products and device copies."""
    from vortx_b200 import _lib
    lib = _lib.load()
    links = 4
    w = synth.normal_matrix(rows, cols, seed=rows + 3) * np.float32(50.0 / np.sqrt(cols))
    qm = vb.QuantizedMatrix.from_f32(backend, qt, w)
    x0 = synth.normal_vectors(1, cols, seed=6)[0]
    xd = backend.init_buffer(x0)
    seg_len, seg_stride = cols // segs, rows // segs
    first = seg_stride - seg_len if at_end else 0
    # plain chain
    y = backend.uninit_buffer(rows)
    xn = backend.uninit_buffer(cols)
    src = xd
    for l in range(links):
        vb.Gemv().dispatch(backend, None, y, qm, src)
        for s in range(segs):
            _lib.check(lib.vx_copy(backend._ctx, xn.ptr + s * seg_len * 4, y.ptr + (s * seg_stride + first) * 4, seg_len * 4))
        src = xn
    want = np.empty(rows, np.float32)
    backend.slow_read_buffer(y, want)
    # the same as one list
    nbytes = lib.vx_xvec_bytes(rows)
    vecs = [backend.uninit_buffer(nbytes, dtype=np.uint8) for _ in range(2)]
    for v in vecs:
        _lib.check(lib.vx_memset(backend._ctx, v.ptr, 0, nbytes))
    entries = [{"w": qm, "x": xd.ptr, "y_xvec": vecs[0].ptr}]
    for l in range(1, links):
        entries.append({"w": qm, "x_xvec": vecs[(l - 1) % 2].ptr, "y_xvec": vecs[l % 2].ptr,
                        "x_seg_len": seg_len, "x_seg_stride": seg_stride, "x_seg_first": first})
    batch = vb.GemvBatch(backend, entries)
    out = backend.uninit_buffer(rows)
    got = np.empty(rows, np.float32)
    for rep in range(2):
        batch.launch()
        _lib.check(lib.vx_xvec_unpack(backend._ctx, vecs[(links - 1) % 2].ptr, rows, out.ptr))
        backend.slow_read_buffer(out, got)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    batch.free()
