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
