"""Host logic of the row-sharded GEMV on CPU: world size 2 (and 3, uneven) over gloo.

The shard arithmetic and the gather are the library's (vortx_b200/multi_gpu.py); the per-rank product is
the CPU oracle here, because the CUDA kernel needs a GPU.  The gathered y must equal the unsharded product."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as o
from vortx_b200 import synth
from vortx_b200.multi_gpu import ShardedGemv, row_shard, shard_blocks


def test_row_shard_partitions_exactly():
    for rows in (1, 7, 8, 28672, 1001):
        for world in (1, 2, 3, 4, 8):
            spans = [row_shard(rows, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(n for _, n in spans) == rows
            for (a0, an), (b0, _) in zip(spans, spans[1:]):
                assert a0 + an == b0
            assert max(n for _, n in spans) - min(n for _, n in spans) <= 1
    assert row_shard(28672, 8, 3) == (3 * 3584, 3584)
    with pytest.raises(ValueError):
        row_shard(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, rows, cols, batch, qt, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = synth.normal_matrix(rows, cols, seed=3)
        x = torch.from_numpy(synth.normal_vectors(batch, cols, seed=4))
        blocks = o.quantize(qt, w)
        mine = shard_blocks(blocks, rows, cols, o.BLOCK_BYTES[qt], world, rank)

        def compute(xv, y_slice):
            y = o.gemv(qt, mine, y_slice.shape[1], cols, xv.numpy())
            y_slice.copy_(torch.from_numpy(np.atleast_2d(y)))

        g = ShardedGemv(rows, cols, compute)
        assert (g.row0, g.nrows) == row_shard(rows, world, rank)
        y = torch.full((batch, rows), float("nan"))
        g.dispatch(x, y)
        np.save(os.path.join(out_dir, f"y{rank}.npy"), y.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,rows,batch", [(2, 64, 1), (2, 64, 3), (3, 50, 1), (2, 33, 2)])
def test_sharded_gemv_gathers_the_full_product(tmp_path, world, rows, batch):
    cols, qt = 256, o.Q4_0
    mp.spawn(_worker, args=(world, _free_port(), rows, cols, batch, qt, str(tmp_path)), nprocs=world, join=True)
    w = synth.normal_matrix(rows, cols, seed=3)
    x = synth.normal_vectors(batch, cols, seed=4)
    want = np.atleast_2d(o.gemv(qt, o.quantize(qt, w), rows, cols, x))
    for r in range(world):
        got = np.load(tmp_path / f"y{r}.npy")
        # each row's sum is computed by exactly one rank with the oracle's own order: bit-identical
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), r


# ------------------------------------------------------------------ column-sharded GEMM ----

from vortx_b200.multi_gpu import col_shard, panel_relayout_shape  # noqa: E402


def test_col_shard_partitions_in_whole_blocks():
    for cols in (32, 64, 1024, 8192, 1000, 96 + 5):
        for world in (1, 2, 3, 4, 8):
            spans = [col_shard(cols, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(n for _, n in spans) == cols
            for (a0, an), (b0, _) in zip(spans, spans[1:]):
                assert a0 + an == b0
            assert all(c0 % 32 == 0 for c0, _ in spans)
            assert all(n % 32 == 0 for _, n in spans[:-1])
    assert col_shard(8192, 8, 5) == (5 * 1024, 1024)


def _gemm_worker(rank, world, port, m, n, k, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.Generator(np.random.Philox(7))
        a = rng.random((m, k), dtype=np.float32) * 2 - 1
        b = rng.random((k, n), dtype=np.float32) * 2 - 1
        col0, ncols = col_shard(n, world, rank)
        # the per-rank panel through the oracle's restatement of the reference GEMM
        panel = np.zeros((m, ncols), np.float32)
        o.gemm_dispatch(panel, a, np.ascontiguousarray(b[:, col0:col0 + ncols]),
                        o.shape_contiguous(1, 1, m, ncols), o.shape_contiguous(1, 1, m, k),
                        o.shape_contiguous(1, 1, k, ncols))
        stack = torch.empty(world * m * ncols)      # rank-major: [world][m][ncols]
        dist.all_gather_into_tensor(stack, torch.from_numpy(panel).reshape(-1))
        sizes, strides = panel_relayout_shape(m, world, ncols)
        c = o.contiguous(stack.numpy().ravel(), o.Shape(*sizes, *strides))
        np.save(os.path.join(out_dir, f"c{rank}.npy"), c.reshape(m, n))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,m,n,k", [(2, 48, 128, 40), (4, 33, 256, 64)])
def test_column_sharded_gemm_relayout_gives_the_unsharded_product(tmp_path, world, m, n, k):
    """All-gather of rank-major panels + the strided gather (panel_relayout_shape) equals the unsharded GEMM,
    bit for bit: every element is computed by exactly one rank in the reference's own order."""
    mp.spawn(_gemm_worker, args=(world, _free_port(), m, n, k, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.Generator(np.random.Philox(7))
    a = rng.random((m, k), dtype=np.float32) * 2 - 1
    b = rng.random((k, n), dtype=np.float32) * 2 - 1
    want = np.zeros((m, n), np.float32)
    o.gemm_dispatch(want, a, b, o.shape_contiguous(1, 1, m, n), o.shape_contiguous(1, 1, m, k),
                    o.shape_contiguous(1, 1, k, n))
    for r in range(world):
        got = np.load(tmp_path / f"c{r}.npy")
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), r


# ------------------------------------------------------------------ a rank that leaves ----

from vortx_b200.multi_gpu import PeerLost, RankWatch  # noqa: E402


def _leaving_worker(rank, world, port, out_dir):
    """Three steps of a sharded product; rank `world - 1` leaves, between steps, after the first.  The others
    must learn of it on the host before they launch step 2 (PeerLost), not by hanging in a collective."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    watch = RankWatch.for_default_group()
    steps_done, error = 0, ""
    try:
        for step in range(1, 4):
            if rank == world - 1 and step == 2:
                watch.leave()                      # between steps, nothing in flight
                break
            watch.announce(step)
            watch.await_all(step, timeout_s=5.0)
            t = torch.full((4,), float(rank + step))
            parts = [torch.empty(4) for _ in range(world)]
            dist.all_gather(parts, t)              # the step's exchange
            assert [float(p[0]) for p in parts] == [float(r + step) for r in range(world)]
            steps_done = step
    except PeerLost as e:
        error = str(e)
    with open(os.path.join(out_dir, f"leave{rank}.txt"), "w") as f:
        f.write(f"{steps_done}|{error}")
    # rank 0 hosts the store: it stays until the others have written their result
    if rank == 0:
        import time
        deadline = time.monotonic() + 15
        while time.monotonic() < deadline and not all(
                os.path.exists(os.path.join(out_dir, f"leave{r}.txt")) for r in range(world)):
            time.sleep(0.01)
    os._exit(0)      # no collective teardown with a rank missing


@pytest.mark.parametrize("world", [2, 3])
def test_a_rank_that_leaves_between_steps_is_noticed_on_the_host(tmp_path, world):
    import time
    t0 = time.monotonic()
    mp.spawn(_leaving_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert time.monotonic() - t0 < 60
    for r in range(world):
        done, error = (tmp_path / f"leave{r}.txt").read_text().split("|", 1)
        if r == world - 1:
            assert (done, error) == ("1", "")
        else:
            assert done == "1" and f"rank {world - 1} has left the group before step 2" in error


def test_a_rank_that_falls_silent_costs_one_timeout():
    """No process group: the watch over a plain in-memory store.  A rank that never announces the step makes
    await_all raise after its timeout, naming the rank."""
    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode()

        def get(self, k):
            return self[k]

    st = Store()
    a, b = RankWatch(st, 0, 2), RankWatch(st, 1, 2)
    a.announce(1)
    b.announce(1)
    a.await_all(1, timeout_s=0.2)
    a.announce(2)
    with pytest.raises(PeerLost, match="rank 1 has not reached step 2"):
        a.await_all(2, timeout_s=0.05)
