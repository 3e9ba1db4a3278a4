"""2, 4 and 8 GPUs, one process each: the row-sharded GEMV whose epilogue stores y into the peers' memory, followed
by the cross-GPU barrier kernel, against the CPU oracle; the NCCL all-gather form of the same product; chains of
dependent products with the exchange fused into the kernel; the column-sharded TF32 GEMM.

Every test runs at each world size the box has GPUs for and is skipped otherwise.  Ranks are child processes;
each leaves only after a final host barrier, with no kernel in flight."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import vortx_b200 as vb
    from vortx_b200 import synth
    from vortx_b200.multi_gpu import PeerScatterGemv, ShardedGemv, shard_blocks
    be = vb.Backend(rank)
    rows, cols, slots = 1024, 2048, 3
    results = {}
    for qt, name in ((vb.Q4_0, "q4"), (vb.Q8_0, "q8")):
        w = synth.normal_matrix(rows, cols, seed=21)
        blocks = vb.quantize(qt, w)
        mine = shard_blocks(blocks, rows, cols, 18 if qt == vb.Q4_0 else 34, world, rank)
        g = PeerScatterGemv(be, rows, cols, slots)
        qm = vb.QuantizedMatrix(be, qt, mine, g.nrows, cols)
        xs = synth.normal_vectors(slots, cols, seed=22)
        xd = be.init_buffer(xs.ravel())
        for rep in range(2):                     # twice: the device-side barrier count must keep advancing
            for s in range(slots):
                g.dispatch(qm, xd.ptr + s * cols * 4, s)
        be.synchronize()
        y = np.empty(slots * rows, np.float32)
        be.slow_read_buffer(g.y.local, y.view(np.uint8))
        results[f"{name}_peer"] = y.reshape(slots, rows)
        dist.barrier()
        # the same products as one list launch with plain peer rows and a single barrier
        lib = vb.load()
        vb._lib.check(lib.vx_memset(be._ctx, g.y.local.ptr, 0xFF, slots * rows * 4))
        be.synchronize()
        dist.barrier()
        batch = g.scatter_batch([qm] * slots, [xd.ptr + s * cols * 4 for s in range(slots)])
        batch.launch()
        g.finish()
        be.synchronize()
        y2 = np.empty(slots * rows, np.float32)
        be.slow_read_buffer(g.y.local, y2.view(np.uint8))
        results[f"{name}_peer_list"] = y2.reshape(slots, rows)
        batch.free()
        dist.barrier()
        # the same products with HOST buffers, one stage per product: x up from pinned memory, list launch,
        # barrier, the whole gathered y down to pinned memory, the copies beside the neighbouring stages' kernels
        vb._lib.check(lib.vx_memset(be._ctx, g.y.local.ptr, 0xFF, slots * rows * 4))
        be.synchronize()
        dist.barrier()
        xs_pin = torch.from_numpy(xs.copy()).pin_memory()
        ys_pin = torch.full((slots, rows), float("nan")).pin_memory()
        x_up = be.init_buffer(np.zeros(slots * cols, np.float32))
        singles = [g.scatter_batch([qm], [x_up.ptr + s * cols * 4], first_slot=s) for s in range(slots)]
        stages = [{"batch": singles[s],
                   "up": (x_up.ptr + s * cols * 4, xs_pin.data_ptr() + s * cols * 4, cols * 4),
                   "down": (ys_pin.data_ptr() + s * rows * 4, rows * 4, g.y.local.ptr + s * rows * 4, rows * 4, rows * 4, 1),
                   "barrier": (list(g.flags.ptrs), rank)} for s in range(slots)]
        run = vb.HostStages(be, stages)
        run.run()
        run.run()
        results[f"{name}_peer_host"] = ys_pin.numpy().copy()
        ys_pin.fill_(float("nan"))
        dist.barrier()
        rec = vb.HostStages(be, stages, recorded=True)        # the step as one CUDA graph, barriers included
        rec.run()
        rec.run()
        results[f"{name}_peer_host_recorded"] = ys_pin.numpy().copy()
        rec.free()
        for b in singles:
            b.free()
        dist.barrier()
        g.close()
        # NCCL form through torch tensors on the same stream
        sg = ShardedGemv.for_backend(be, qt, mine, rows, cols)
        stream = torch.cuda.ExternalStream(be.stream)
        with torch.cuda.stream(stream):
            xt = torch.from_numpy(xs[:1]).cuda()
            yt = torch.zeros(1, rows, device="cuda")
            sg.dispatch(xt, yt)
            stream.synchronize()
        results[f"{name}_nccl"] = yt.cpu().numpy()
    # the same sharded product through the C ABI's own group (vx_group_*: NCCL communicator + IPC peer buffers made
    # by the library itself; torch only carries the 128-byte id), and the list form on group-allocated buffers
    from vortx_b200.multi_gpu import Group
    grp = Group.from_torch(be)
    w = synth.normal_matrix(rows, cols, seed=21)
    blocks = vb.quantize(vb.Q4_0, w)
    mine = shard_blocks(blocks, rows, cols, 18, world, rank)
    g2 = PeerScatterGemv(be, rows, cols, slots, vectors=0, vx_group=grp)
    qm = vb.QuantizedMatrix(be, vb.Q4_0, mine, g2.nrows, cols)
    xs = synth.normal_vectors(slots, cols, seed=22)
    xd = be.init_buffer(xs.ravel())
    for rep in range(2):
        for s in range(slots):
            grp.gemv_q(qm, g2.row0, xd.ptr + s * cols * 4, g2.y.ptrs, s * rows * 4)
    be.synchronize()
    y = np.empty(slots * rows, np.float32)
    be.slow_read_buffer(g2.y.local, y.view(np.uint8))
    results["q4_group"] = y.reshape(slots, rows)
    gathered = be.init_buffer(np.zeros(world * 16, np.float32))
    be.write_buffer(gathered, rank * 16, np.full(16, float(rank + 1), np.float32))
    grp.all_gather(gathered.ptr, 64)
    ag = np.empty(world * 16, np.float32)
    be.slow_read_buffer(gathered, ag)
    results["group_all_gather"] = ag
    grp.barrier()
    be.synchronize()
    dist.barrier()
    g2.close()
    grp.close()
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **results)
    dist.barrier()
    be.close()
    os._exit(0)   # every rank is past the final barrier with nothing in flight; no communicator teardown


def _chain_worker(rank, world, port, out_dir):
    """A chain of GEMVs whose exchange is fused into the kernel: link l reads the exchange vector link l - 1
    wrote on every GPU, pair by pair as the rows arrive.  Run twice from different x0 so that a link that read
    too early would pick up the first run's values; with contiguous slabs and with rows dealt out in turn."""
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import vortx_b200 as vb
    from vortx_b200 import synth
    from vortx_b200.multi_gpu import PeerScatterGemv, shard_blocks
    be = vb.Backend(rank)
    n, links = 2048, 6
    w = synth.normal_matrix(n, n, seed=31) * np.float32(50.0 / 45.0)
    blocks = vb.quantize(vb.Q4_0, w)
    results = {}
    x0 = synth.normal_vectors(2, n, seed=32)
    xd = be.init_buffer(x0.ravel())
    for cyclic in (False, True):
        g = PeerScatterGemv(be, n, n, links, cyclic=cyclic)
        if cyclic:
            per_row = n // 32 * 18
            mine = np.ascontiguousarray(blocks.reshape(n, per_row)[rank::world]).ravel()
        else:
            mine = shard_blocks(blocks, n, n, 18, world, rank)
        qm = vb.QuantizedMatrix(be, vb.Q4_0, mine, g.nrows, n)
        for run in range(2):
            # link l reads vector (l - 1) % 2 and writes vector l % 2; every link is also unpacked into
            # y[l] so that each can be checked on its own
            for l in range(links):
                if l == 0:
                    g.dispatch_chained(qm, 0, x_ptr=xd.ptr + run * n * 4)
                else:
                    g.dispatch_chained(qm, l % 2, x_vec=(l - 1) % 2)
                g.unpack(l % 2, g.y_ptr(l))
            be.synchronize()
            y = np.empty(links * n, np.float32)
            be.slow_read_buffer(g.y.local, y.view(np.uint8))
            results[f"run{run}_{int(cyclic)}"] = y.reshape(links, n).copy()
            # the same chain with nothing between the links: only the in-kernel waits order them
            for rep in range(3):
                g.dispatch_chained(qm, 0, x_ptr=xd.ptr + run * n * 4)
                for l in range(1, links):
                    g.dispatch_chained(qm, l % 2, x_vec=(l - 1) % 2)
                g.unpack((links - 1) % 2, g.y_ptr(0))
            be.synchronize()
            be.slow_read_buffer(g.y.local, y.view(np.uint8))
            results[f"pure{run}_{int(cyclic)}"] = y[:n].copy()
            # and as one persistent launch per GPU
            batch = g.chain_batch([qm] * links, xd.ptr + run * n * 4)
            for rep in range(3):
                batch.launch()
                g.unpack((links - 1) % 2, g.y_ptr(1))
            be.synchronize()
            be.slow_read_buffer(g.y.local, y.view(np.uint8))
            results[f"batch{run}_{int(cyclic)}"] = y[n:2 * n].copy()
            batch.free()
            dist.barrier()
        g.close()
    # rows > cols with contiguous slabs: x of the next link is the tail of every rank's slab (a windowed read);
    # against the same chain computed on this GPU alone from the whole matrix, with plain products and copies
    from vortx_b200 import _lib
    lib = _lib.load()
    rows, cols, wl = 4096, 2048, 5
    w2 = synth.normal_matrix(rows, cols, seed=41) * np.float32(50.0 / 45.0)
    blocks2 = vb.quantize(vb.Q4_0, w2)
    g = PeerScatterGemv(be, rows, cols, 1)
    mine = vb.QuantizedMatrix(be, vb.Q4_0, shard_blocks(blocks2, rows, cols, 18, world, rank), g.nrows, cols)
    whole = vb.QuantizedMatrix(be, vb.Q4_0, blocks2, rows, cols)
    seg_len, seg_stride = cols // world, rows // world
    yp, xn = be.uninit_buffer(rows), be.uninit_buffer(cols)
    src = xd.ptr
    for l in range(wl):
        vb.Gemv().dispatch(be, None, yp, whole, src)
        for s_ in range(world):
            _lib.check(lib.vx_copy(be._ctx, xn.ptr + s_ * seg_len * 4,
                                   yp.ptr + (s_ * seg_stride + seg_stride - seg_len) * 4, seg_len * 4))   # the slab's tail
        src = xn.ptr
    want = np.empty(rows, np.float32)
    be.slow_read_buffer(yp, want)
    batch = g.chain_batch([mine] * wl, xd.ptr, window=True)
    for rep in range(3):
        batch.launch()
        g.unpack((wl - 1) % 2, g.y_ptr(0))
    be.synchronize()
    got = np.empty(rows, np.float32)
    be.slow_read_buffer(g.y.local, got.view(np.uint8))
    results["window_want"], results["window_got"] = want, got
    batch.free()
    dist.barrier()
    # the same chain WITHOUT a window reads the vector's first `cols` elements: rows of the first ranks only.  A rank
    # none of whose rows is among them would never be waited for; the library must refuse its list, launching nothing.
    before = be.launch_count()
    try:
        bad = g.chain_batch([mine] * wl, xd.ptr, window=False)
        bad.free()
        results["unwindowed_refused"] = np.array([0])
    except _lib.VortxError as e:
        assert e.status == _lib.VX_ERR_UNSUPPORTED, e
        results["unwindowed_refused"] = np.array([1])
    assert be.launch_count() == before
    results["row0"] = np.array([g.row0])
    dist.barrier()
    g.close()
    np.savez(os.path.join(out_dir, f"chain{rank}.npz"), **results)
    dist.barrier()
    be.close()
    os._exit(0)


def _run_ranks(target, world, out_dir):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, out_dir)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.kill()          # the exact child started above
            pytest.fail("a rank did not finish in time")
        assert p.exitcode == 0


WORLDS = [2, 4, 8]


def _need(world):
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")


@pytest.mark.parametrize("world", WORLDS)
def test_chained_gemv_with_fused_exchange(tmp_path, oracle, world):
    import vortx_b200 as vb
    from vortx_b200 import synth
    _need(world)
    _run_ranks(_chain_worker, world, str(tmp_path))
    n, links = 2048, 6
    w = synth.normal_matrix(n, n, seed=31) * np.float32(50.0 / 45.0)
    blocks = vb.quantize(vb.Q4_0, w)
    x0 = synth.normal_vectors(2, n, seed=32)
    got = [np.load(tmp_path / f"chain{r}.npz") for r in range(world)]
    for cyclic in (0, 1):
        for run in range(2):
            key = f"run{run}_{cyclic}"
            ys = got[0][key]
            for r in range(1, world):
                assert np.array_equal(ys.view(np.uint32), got[r][key].view(np.uint32))   # one y everywhere
            prev = x0[run]
            for l in range(links):
                y64, absdot = oracle.gemv_f64(vb.Q4_0, blocks, n, n, prev[None, :])
                assert (np.abs(ys[l] - y64[0]) <= 2e-6 * absdot[0]).all(), f"{key} link {l}"
                prev = ys[l]
            for r in range(world):   # the kernel is deterministic: the unattended chain ends on the same bits
                assert np.array_equal(got[r][f"pure{run}_{cyclic}"].view(np.uint32), ys[links - 1].view(np.uint32))
                assert np.array_equal(got[r][f"batch{run}_{cyclic}"].view(np.uint32), ys[links - 1].view(np.uint32))
        assert not np.array_equal(got[0][f"run0_{cyclic}"], got[0][f"run1_{cyclic}"])
    for r in range(world):
        assert np.array_equal(got[r]["window_got"].view(np.uint32), got[r]["window_want"].view(np.uint32))
        assert np.isfinite(got[r]["window_got"]).all() and np.abs(got[r]["window_got"]).max() > 0
        # 4096 rows, 2048 columns: only ranks whose slab starts below row 2048 are among the awaited elements
        assert int(got[r]["unwindowed_refused"][0]) == (1 if int(got[r]["row0"][0]) >= 2048 else 0), r


@pytest.mark.parametrize("world", WORLDS)
def test_peer_scatter_and_nccl_gemv(tmp_path, oracle, world):
    import vortx_b200 as vb
    from vortx_b200 import synth
    _need(world)
    _run_ranks(_worker, world, str(tmp_path))
    rows, cols, slots = 1024, 2048, 3
    w = synth.normal_matrix(rows, cols, seed=21)
    xs = synth.normal_vectors(slots, cols, seed=22)
    for qt, name in ((vb.Q4_0, "q4"), (vb.Q8_0, "q8")):
        y64, absdot = oracle.gemv_f64(qt, vb.quantize(qt, w), rows, cols, xs)
        for r in range(world):
            got = np.load(tmp_path / f"rank{r}.npz")
            peer, nccl = got[f"{name}_peer"], got[f"{name}_nccl"]
            assert np.abs(peer - y64).max() / np.abs(y64).max() <= 1e-4
            assert (np.abs(peer - y64) <= 2e-6 * absdot).all()
            assert np.array_equal(nccl[0].view(np.uint32), peer[0].view(np.uint32))   # same kernel, same rows
            assert np.array_equal(got[f"{name}_peer_list"].view(np.uint32), peer.view(np.uint32))
            assert np.array_equal(got[f"{name}_peer_host"].view(np.uint32), peer.view(np.uint32))   # vx_gemv_batch_run_host
            assert np.array_equal(got[f"{name}_peer_host_recorded"].view(np.uint32), peer.view(np.uint32))   # vx_host_pipeline
            if name == "q4":
                assert np.array_equal(got["q4_group"].view(np.uint32), peer.view(np.uint32))       # vx_group_gemv_q
                assert np.array_equal(got["group_all_gather"], np.repeat(np.arange(1, world + 1, dtype=np.float32), 16))


def _gemm_worker(rank, world, port, out_dir):
    """Column-sharded TF32 GEMM: peer-store epilogue + barrier kernel, and the NCCL all-gather + re-layout form."""
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import vortx_b200 as vb
    from vortx_b200.multi_gpu import ShardedGemm
    be = vb.Backend(rank)
    stream = torch.cuda.ExternalStream(be.stream)
    results = {}
    for m, n, k in GEMM_CASES:
        rng = np.random.Generator(np.random.Philox(m + n + k))
        a = rng.random((m, k), dtype=np.float32) * 2 - 1
        b = rng.random((k, n), dtype=np.float32) * 2 - 1
        ad, bd = be.init_buffer(a.ravel()), be.init_buffer(b.ravel())   # B whole on every rank; each uses its columns
        g = ShardedGemm(be, m, n, k)
        even = n % world == 0 and (n // world) % 32 == 0
        for form in ("peer", "nccl") if even else ("peer",):
            for rep in range(2):
                with torch.cuda.stream(stream):
                    if form == "peer":
                        g.dispatch_peer(ad.ptr, bd.ptr + g.col0 * 4, n)
                    else:
                        g.dispatch_nccl(ad.ptr, bd.ptr + g.col0 * 4, n)
            be.synchronize()
            c = np.empty(m * n, np.float32)
            be.slow_read_buffer(g.c.local, c.view(np.uint8))
            results[f"{form}_{m}_{n}_{k}"] = c.reshape(m, n)
            dist.barrier()
        g.close()
    np.savez(os.path.join(out_dir, f"gemm{rank}.npz"), **results)
    dist.barrier()
    be.close()
    os._exit(0)


GEMM_CASES = [(512, 512, 256), (300, 1024, 200), (1024, 2048, 1024), (200, 1000, 96), (129, 72, 40)]


@pytest.mark.parametrize("world", WORLDS)
def test_column_sharded_tf32_gemm(tmp_path, world):
    _need(world)
    _run_ranks(_gemm_worker, world, str(tmp_path))
    got = [np.load(tmp_path / f"gemm{r}.npz") for r in range(world)]
    for m, n, k in GEMM_CASES:
        rng = np.random.Generator(np.random.Philox(m + n + k))
        a = rng.random((m, k), dtype=np.float32) * 2 - 1
        b = rng.random((k, n), dtype=np.float32) * 2 - 1
        want = a.astype(np.float64) @ b.astype(np.float64)
        key = f"{m}_{n}_{k}"
        for r in range(world):
            peer = got[r][f"peer_{key}"]
            rel = np.linalg.norm(peer - want) / np.linalg.norm(want)
            assert rel <= 5e-3, (key, r, rel)                       # TF32 inputs, f32 accumulate
            if f"nccl_{key}" in got[r]:                             # equal panels only
                assert np.array_equal(peer.view(np.uint32), got[r][f"nccl_{key}"].view(np.uint32))   # same kernel, same tiles
            assert np.array_equal(peer.view(np.uint32), got[0][f"peer_{key}"].view(np.uint32))   # one C everywhere


# ------------------------------------------------- the benchmark's own shape, 28672 x 8192 Q4_0 ----

BIG_ROWS, BIG_COLS, BIG_LINKS = 28672, 8192, 3


def _big_slab(world, rank):
    """Rank `rank`'s rows of the 28672 x 8192 matrix, each slab from its own seed (as the benchmark does)."""
    from vortx_b200 import synth
    return synth.normal_matrix(BIG_ROWS // world, BIG_COLS, seed=100 + rank) * np.float32(25.0 / 45.0)


def _big_worker(rank, world, port, out_dir):
    """Row slabs of the up-projection on `world` GPUs: (a) independent products whose rows the epilogue stores on
    every GPU, completed by one barrier (what the benchmark times); (b) a chain of dependent products in one list
    launch per GPU, x of link l the tail of every rank's slab of link l - 1 (the benchmark's chained form)."""
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import vortx_b200 as vb
    from vortx_b200 import synth
    from vortx_b200.multi_gpu import PeerScatterGemv
    be = vb.Backend(rank)
    qm = vb.QuantizedMatrix.from_f32(be, vb.Q4_0, _big_slab(world, rank))
    xs = synth.normal_vectors(BIG_LINKS, BIG_COLS, seed=1)
    xd = be.init_buffer(xs.ravel())
    results = {}
    g = PeerScatterGemv(be, BIG_ROWS, BIG_COLS, BIG_LINKS)
    # (a) independent products, rows stored on every GPU by the epilogue, one barrier
    batch = g.scatter_batch([qm] * BIG_LINKS, [xd.ptr + l * BIG_COLS * 4 for l in range(BIG_LINKS)])
    for rep in range(2):
        batch.launch()
        g.finish()
    be.synchronize()
    y = np.empty(BIG_LINKS * BIG_ROWS, np.float32)
    be.slow_read_buffer(g.y.local, y.view(np.uint8))
    results["scatter"] = y.reshape(BIG_LINKS, BIG_ROWS).copy()
    batch.free()
    dist.barrier()
    # (b) the chain; every link also leaves its own rows as plain f32 so that each link can be checked alone
    plain = be.init_buffer(np.zeros(BIG_LINKS * g.nrows, np.float32))
    entries = []
    seg_len, seg_stride = BIG_COLS // world, BIG_ROWS // world
    for l in range(BIG_LINKS):
        e = {"w": qm, "nrows": g.nrows, "y": plain.ptr + l * g.nrows * 4, "y_xvec": g.vectors[l % 2].local.ptr,
             "peers": [g.vectors[l % 2].ptrs[r] for r in g._others], "y_row0": g.row0, "y_stride": 1}
        if l == 0:
            e["x"] = xd.ptr
        else:
            e["x_xvec"] = g.vectors[(l - 1) % 2].local.ptr
            e["x_seg_len"], e["x_seg_stride"], e["x_seg_first"] = seg_len, seg_stride, seg_stride - seg_len
        entries.append(e)
    chain = vb.GemvBatch(be, entries)
    for rep in range(3):
        chain.launch()
        g.unpack((BIG_LINKS - 1) % 2, g.y_ptr(0))
    be.synchronize()
    be.slow_read_buffer(g.y.local, y.view(np.uint8))
    results["chain_last"] = y[:BIG_ROWS].copy()                       # the whole last vector, as this GPU received it
    mine = np.empty(BIG_LINKS * g.nrows, np.float32)
    be.slow_read_buffer(plain, mine)
    results["chain_rows"] = mine.reshape(BIG_LINKS, g.nrows)
    chain.free()
    dist.barrier()
    g.close()
    np.savez(os.path.join(out_dir, f"big{rank}.npz"), **results)
    dist.barrier()
    be.close()
    os._exit(0)


@pytest.mark.parametrize("world", WORLDS)
def test_q4_0_28672x8192_sharded_over_the_gpus(tmp_path, oracle, world):
    import vortx_b200 as vb
    from vortx_b200 import synth
    _need(world)
    _run_ranks(_big_worker, world, str(tmp_path))
    got = [np.load(tmp_path / f"big{r}.npz") for r in range(world)]
    shard = BIG_ROWS // world
    blocks = [vb.quantize(vb.Q4_0, _big_slab(world, r)) for r in range(world)]
    xs = synth.normal_vectors(BIG_LINKS, BIG_COLS, seed=1)

    def product(x):
        parts = [oracle.gemv_f64(vb.Q4_0, blocks[r], shard, BIG_COLS, x[None, :]) for r in range(world)]
        return np.concatenate([p[0][0] for p in parts]), np.concatenate([p[1][0] for p in parts])

    # (a) every GPU holds every product, all of it
    for l in range(BIG_LINKS):
        y64, absdot = product(xs[l])
        for r in range(world):
            y = got[r]["scatter"][l]
            assert np.abs(y - y64).max() / np.abs(y64).max() <= 1e-4, (l, r)
            assert (np.abs(y - y64) <= 2e-6 * absdot).all(), (l, r)
            assert np.array_equal(y.view(np.uint32), got[0]["scatter"][l].view(np.uint32))
    # (b) link by link: each link against the oracle applied to the x the GPUs actually used
    seg_len = BIG_COLS // world
    x = xs[0]
    for l in range(BIG_LINKS):
        y64, absdot = product(x)
        y = np.concatenate([got[r]["chain_rows"][l] for r in range(world)])
        assert np.abs(y - y64).max() / np.abs(y64).max() <= 1e-4, l
        assert (np.abs(y - y64) <= 2e-6 * absdot).all(), l
        x = np.concatenate([y[(r + 1) * shard - seg_len:(r + 1) * shard] for r in range(world)])   # the slabs' tails
    for r in range(world):
        assert np.array_equal(got[r]["chain_last"].view(np.uint32), y.view(np.uint32)), r          # one vector everywhere
