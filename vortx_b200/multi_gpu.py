"""Row-sharded quantised GEMV over several GPUs of one node: one process per GPU,
torch.distributed for the plumbing (NCCL over NVLink on GPUs, gloo in the CPU tests).

Rank r holds rows [row0, row0 + nrows) of W — a contiguous slab of the block stream — computes its
part of y straight into its slice of the full-length y and the slices are all-gathered in place.
x is replicated; no collective ever touches the weights.  vortx has no multi-device notion beyond a
device ordinal (src/linalg/gemm.rs:353); this layer has no reference counterpart.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import numpy as np


def row_shard(rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous balanced slabs: the first rows % world ranks take one extra row."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside a world of {world}")
    base, extra = divmod(rows, world)
    row0 = rank * base + min(rank, extra)
    return row0, base + (1 if rank < extra else 0)


def shard_blocks(blocks: np.ndarray, rows: int, cols: int, block_bytes: int, world: int, rank: int) -> np.ndarray:
    """The slab of a host block stream that belongs to `rank` (a view, no copy)."""
    per_row = cols // 32 * block_bytes
    if blocks.size != rows * per_row:
        raise ValueError(f"block stream has {blocks.size} bytes, expected {rows * per_row}")
    row0, n = row_shard(rows, world, rank)
    return blocks[row0 * per_row:(row0 + n) * per_row]


class ShardedGemv:
    """y = W x with W split by rows across the ranks of `group`.

    `compute(x, y_slice)` runs this rank's GEMV: x a torch tensor [batch, cols] (replicated), y_slice the
    rank's view [batch, nrows] of the full y.  On GPUs it is the CUDA kernel (see `for_backend`)."""

    def __init__(self, rows: int, cols: int, compute: Callable, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.rows, self.cols = rows, cols
        self.row0, self.nrows = row_shard(rows, self.world, self.rank)
        self.compute = compute
        self.even = rows % self.world == 0

    @classmethod
    def for_backend(cls, backend, qtype: int, shard_stream: np.ndarray, rows: int, cols: int, group=None):
        """Uploads this rank's slab and binds the CUDA GEMV to it.  `shard_stream` is the rank's part of the
        block stream (see shard_blocks)."""
        from . import _lib
        from .linalg import QuantizedMatrix
        self = cls(rows, cols, None, group)
        self.weights = QuantizedMatrix(backend, qtype, shard_stream, self.nrows, cols)
        lib = _lib.load()

        def compute(x, y_slice):
            batch = x.shape[0]
            if x.stride(1) != 1 or y_slice.stride(1) != 1:
                raise ValueError("x and y must be contiguous along their vectors")
            _lib.check(lib.vx_gemv_q_rows(backend._ctx, self.weights._h, 0, self.nrows, x.data_ptr(), x.stride(0),
                                          y_slice.data_ptr(), y_slice.stride(0), batch))
        self.compute = compute
        return self

    def dispatch(self, x, y_full) -> None:
        """x: [batch, cols]; y_full: [batch, rows] on every rank; on return every rank holds all of y."""
        if x.shape[-1] != self.cols or y_full.shape[-1] != self.rows or x.shape[0] != y_full.shape[0]:
            raise ValueError(f"shapes {tuple(x.shape)} -> {tuple(y_full.shape)} do not fit a {self.rows} x {self.cols} matrix")
        mine = y_full[:, self.row0:self.row0 + self.nrows]
        self.compute(x, mine)
        if self.world == 1:
            return
        batch = x.shape[0]
        if self.even and batch == 1:
            # in place: rank r's slab already sits at its final position
            self.dist.all_gather_into_tensor(y_full.view(-1), mine.reshape(-1), group=self.group)
            return
        # Uneven slabs or several vectors: gather equal-sized (padded) parts, then place them.
        widest = -(-self.rows // self.world)
        send = y_full.new_zeros((batch, widest))
        send[:, :self.nrows] = mine
        parts: List = [y_full.new_empty((batch, widest)) for _ in range(self.world)]
        self.dist.all_gather(parts, send, group=self.group)
        for r, part in enumerate(parts):
            r0, n = row_shard(self.rows, self.world, r)
            y_full[:, r0:r0 + n] = part[:, :n]
