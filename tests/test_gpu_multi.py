"""Two GPUs, one process each: the row-sharded GEMV whose epilogue stores y into the peer's memory, followed
by the cross-GPU barrier kernel, against the CPU oracle; and the NCCL all-gather form of the same product.

Skipped on a box with one GPU.  Ranks are child processes; each leaves only after a final host barrier, with
no kernel in flight."""
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
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **results)
    dist.barrier()
    be.close()
    os._exit(0)   # skip NCCL teardown, which has hung on these boxes after all work was done


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


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_chained_gemv_with_fused_exchange_on_two_gpus(tmp_path, oracle):
    import vortx_b200 as vb
    from vortx_b200 import synth
    world = 2
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


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_peer_scatter_and_nccl_gemv_on_two_gpus(tmp_path, oracle):
    import torch.multiprocessing as mp
    import vortx_b200 as vb
    from vortx_b200 import synth
    world = 2
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.kill()          # the exact child started above
            pytest.fail("a rank did not finish in time")
        assert p.exitcode == 0
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


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_column_sharded_tf32_gemm_on_two_gpus(tmp_path):
    world = 2
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
