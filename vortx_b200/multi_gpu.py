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

from .backend import GpuBuffer


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


def col_shard(cols: int, world: int, rank: int, multiple: int = 32) -> Tuple[int, int]:
    """Contiguous panels of whole `multiple`-column blocks, balanced like row_shard; the last panel also takes
    the columns beyond the last whole block."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside a world of {world}")
    blocks = cols // multiple
    b0, nb = row_shard(blocks, world, rank)
    col0, ncols = b0 * multiple, nb * multiple
    if rank == world - 1:
        ncols = cols - col0
    return col0, ncols


def panel_relayout_shape(m: int, world: int, ncols: int):
    """(sizes, strides) in elements of the 4-D view that reads a rank-major stack of C panels
    [world][m][ncols] in the order of the row-major C [m][world * ncols]: element (i, r, j) of the result is
    element (r, i, j) of the stack."""
    return (1, m, world, ncols), (world * m * ncols, ncols, m * ncols, 1)


class PeerLost(RuntimeError):
    """A rank of the group has left, or has not reached the step the others are about to launch."""


class RankWatch:
    """Host-side liveness of the ranks, checked BEFORE a step's kernels are launched.

    The fused kernels wait for their peers on the device with a bounded budget, and a collective on a
    communicator that has lost a rank ends in a process-group timeout at best; both are late and costly ways
    to learn that a peer is gone.  Each rank therefore publishes, in the key-value store the process group was
    built on, the number of the step it is about to launch (`announce`), and `await_all` waits, with a short
    timeout, until every rank has announced that step.  A rank that leaves on purpose says so (`leave`): the
    others then raise PeerLost at their next `await_all` without waiting; a rank that died silently costs them
    one timeout.  A rank leaves only between steps, with none of its kernels or collectives in flight."""

    def __init__(self, store, rank: int, world: int, name: str = "vx_watch"):
        self.store, self.rank, self.world, self.name = store, rank, world, name
        self.store.set(self._key(rank), "0")

    @classmethod
    def for_default_group(cls, name: str = "vx_watch") -> "RankWatch":
        import torch.distributed as dist
        from torch.distributed.distributed_c10d import _get_default_store
        return cls(_get_default_store(), dist.get_rank(), dist.get_world_size(), name)

    def _key(self, r: int) -> str:
        return f"{self.name}/{r}"

    def announce(self, step: int) -> None:
        self.store.set(self._key(self.rank), str(int(step)))

    def leave(self) -> None:
        self.store.set(self._key(self.rank), "gone")

    def await_all(self, step: int, timeout_s: float = 5.0) -> None:
        """Returns once every rank has announced `step` (or a later one); raises PeerLost otherwise."""
        import time
        deadline = time.monotonic() + timeout_s
        for r in range(self.world):
            if r == self.rank:
                continue
            while True:
                try:
                    v = self.store.get(self._key(r)).decode()
                except Exception as e:      # the store itself is gone: its host rank has exited
                    raise PeerLost(f"rank {self.rank}: the store is unreachable ({e})") from e
                if v == "gone":
                    raise PeerLost(f"rank {r} has left the group before step {step}")
                if int(v) >= step:
                    break
                if time.monotonic() > deadline:
                    raise PeerLost(f"rank {r} has not reached step {step} within {timeout_s} s (last seen at {v})")
                time.sleep(0.002)


class PeerBuffers:
    """One device buffer per rank, each mapped into every other rank's process with CUDA IPC.

    `local` is this rank's buffer (a GpuBuffer from vx_alloc), `ptrs[r]` the device pointer through which
    this process reaches rank r's buffer (its own pointer for r == rank).  Handles travel through the
    process group (all_gather_object); the mapping is peer-store only by convention of its users."""

    def __init__(self, backend, nbytes: int, group=None, vx_group: Optional["Group"] = None):
        import ctypes as C
        from . import _lib
        self.backend, self.group, self.vx_group = backend, group, vx_group
        if vx_group is not None:
            # the C ABI's own group: allocation, handle exchange (over NCCL) and mapping in one call, no torch
            self.world, self.rank = vx_group.world, vx_group.rank
            self.ptrs = vx_group.peer_alloc(nbytes)
            self.local = GpuBuffer(backend, self.ptrs[self.rank], nbytes, np.uint8, owned=False)
            self._mapped = []
            return
        import torch.distributed as dist
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        lib = _lib.load()
        self.local = backend.uninit_buffer(nbytes, dtype=np.uint8)
        _lib.check(lib.vx_memset(backend._ctx, self.local.ptr, 0, nbytes))
        backend.synchronize()
        handle = (C.c_ubyte * 64)()
        _lib.check(lib.vx_ipc_export(backend._ctx, self.local.ptr, handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ptrs = []
        self._mapped = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local.ptr)
                continue
            p = C.c_void_p()
            buf = (C.c_ubyte * 64).from_buffer_copy(h)
            _lib.check(lib.vx_ipc_import(backend._ctx, buf, C.byref(p)))
            self.ptrs.append(p.value)
            self._mapped.append(p.value)

    def close(self) -> None:
        from . import _lib
        if self.vx_group is not None:
            if self.ptrs:
                self.vx_group.peer_free(self.ptrs)
            self.ptrs = []
            return
        lib = _lib.load()
        for p in self._mapped:
            lib.vx_ipc_release(self.backend._ctx, p)
        self._mapped = []


class PeerScatterGemv:
    """Row-sharded GEMV whose kernel stores each finished row into every peer's memory directly (NVLink
    stores from the epilogue) — no collective.  Two forms:

    * `dispatch(weights, x_ptr, slot)`: plain f32 rows into y[slot] everywhere, then a one-warp arrival
      barrier kernel across the GPUs; after it, on this rank's stream, y[slot] is complete on this GPU.
    * `dispatch_chained(...)`: for chains of dependent GEMVs.  Rows travel as {value, generation} pairs into
      an exchange vector on every GPU, and the next link reads its x from such a vector, re-reading pairs
      that have not arrived yet while its weight stream is already running.  Nothing runs between the links:
      no barrier, no flag, no fence.  `unpack(vec, out_ptr)` ends a chain with plain f32 on this GPU.

    `cyclic=True` deals the rows out in turn (rank r owns rows r, r + world, ...; its slab is still one
    contiguous block stream) instead of contiguous slabs; only the chained form supports it."""

    def __init__(self, backend, rows: int, cols: int, slots: int, group=None, vectors: int = 2, cyclic: bool = False,
                 vx_group: Optional["Group"] = None):
        import ctypes as C
        from . import _lib
        self.backend, self.rows, self.cols, self.slots = backend, rows, cols, slots
        if vx_group is not None:
            self.world, self.rank = vx_group.world, vx_group.rank
        else:
            import torch.distributed as dist
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 GPUs of one node")
        self.cyclic = cyclic
        if cyclic:
            self.row0, self.nrows = self.rank, len(range(self.rank, rows, self.world))
        else:
            self.row0, self.nrows = row_shard(rows, self.world, self.rank)
        self.y = PeerBuffers(backend, max(1, slots) * rows * 4, group, vx_group)
        self.flags = PeerBuffers(backend, 64 * 4, group, vx_group)
        self.vectors = [PeerBuffers(backend, _lib.load().vx_xvec_bytes(rows), group, vx_group) for _ in range(vectors)]
        self._others = [r for r in range(self.world) if r != self.rank]
        self._flags_all = (C.c_void_p * self.world)(*self.flags.ptrs)
        self._vec_peers = [(C.c_void_p * max(1, len(self._others)))(*[v.ptrs[r] for r in self._others])
                           for v in self.vectors]
        if vx_group is None:
            dist.barrier(group=group)

    def y_ptr(self, slot: int) -> int:
        return self.y.local.ptr + slot * self.rows * 4

    def _peer_y(self, off: int):
        import ctypes as C
        return (C.c_void_p * max(1, len(self._others)))(*[self.y.ptrs[r] + off for r in self._others])

    def dispatch(self, weights, x_ptr: int, slot: int) -> None:
        """weights: this rank's QuantizedMatrix slab (nrows x cols)."""
        from . import _lib
        if self.cyclic:
            raise ValueError("the barrier form takes contiguous slabs")
        lib = _lib.load()
        off = (slot * self.rows + self.row0) * 4
        _lib.check(lib.vx_gemv_q_rows_scatter(self.backend._ctx, weights._h, 0, self.nrows, x_ptr,
                                              self.y.local.ptr + off, self._peer_y(off), len(self._others)))
        self.finish()

    def dispatch_chained(self, weights, y_vec: int, x_vec: Optional[int] = None, x_ptr: int = 0) -> None:
        """One link: this rank's rows of W x into exchange vector `y_vec` on every GPU.  x is exchange vector
        `x_vec` (its first `cols` elements, awaited pair by pair) or, for the first link, the plain `x_ptr`.
        A vector may be written again only after every rank has read it: alternate two.  That holds only if
        every thread block of every rank owns a row the next link waits for (nobody can then run ahead of a
        block that is still reading): the library shrinks the grid until it does, and refuses the launch
        (VX_ERR_UNSUPPORTED) when none of this rank's rows is among the first `cols` elements, as with
        contiguous slabs of a matrix with more rows than columns; deal such rows out in turn (cyclic=True)
        or use `chain_batch(window=True)`."""
        from . import _lib
        lib = _lib.load()
        xv = self.vectors[x_vec].local.ptr if x_vec is not None else None
        _lib.check(lib.vx_gemv_q_rows_exchange(self.backend._ctx, weights._h, 0, self.nrows, xv, x_ptr or None, None,
                                               self.vectors[y_vec].local.ptr, self._vec_peers[y_vec],
                                               len(self._others), self.row0, self.world if self.cyclic else 1))

    def scatter_batch(self, weights_list, x_ptrs, first_slot: int = 0):
        """Independent products as ONE persistent launch per GPU: product l reads the plain x_ptrs[l] and stores
        its rows into y[first_slot + l] here and on every peer.  After `launch()`, one `finish()` completes all
        of them."""
        from .linalg import GemvBatch
        if self.cyclic:
            raise ValueError("plain peer rows take contiguous slabs")
        entries = []
        for l, w in enumerate(weights_list):
            off = ((first_slot + l) * self.rows + self.row0) * 4
            entries.append({"w": w, "nrows": self.nrows, "x": x_ptrs[l], "y": self.y.local.ptr + off,
                            "peer_y": [self.y.ptrs[r] + off for r in self._others]})
        return GemvBatch(self.backend, entries)

    def chain_batch(self, weights_list, x_ptr: int, window: bool = False, window_at_end: bool = True):
        """The whole chain as ONE persistent launch per GPU (GemvBatch): link 0 reads the plain x, link l reads
        exchange vector (l - 1) % 2 and writes l % 2.  Returns the batch; after `launch()`, `unpack((len - 1) % 2, ...)`
        ends the chain.  x of a link is the vector's first `cols` elements, or with `window` (contiguous slabs,
        rows > cols) cols / world elements of every rank's slab — its last ones by default, the rows every rank
        computes last, so that the link waits for the end of the previous one as a product over all rows would —:
        rows of every rank, and each tile's rows still leave for a peer as one contiguous store."""
        from .linalg import GemvBatch
        if window and (self.cyclic or self.cols % self.world or self.rows % self.world or (self.cols // self.world) % 32):
            raise ValueError("the windowed chain takes equal contiguous slabs and cols / world a multiple of 32")
        entries = []
        for l, w in enumerate(weights_list):
            e = {"w": w, "nrows": self.nrows, "y_xvec": self.vectors[l % 2].local.ptr,
                 "peers": [self.vectors[l % 2].ptrs[r] for r in self._others],
                 "y_row0": self.row0, "y_stride": self.world if self.cyclic else 1}
            if l == 0:
                e["x"] = x_ptr
            else:
                e["x_xvec"] = self.vectors[(l - 1) % 2].local.ptr
                if window:
                    e["x_seg_len"], e["x_seg_stride"] = self.cols // self.world, self.rows // self.world
                    e["x_seg_first"] = e["x_seg_stride"] - e["x_seg_len"] if window_at_end else 0
            entries.append(e)
        return GemvBatch(self.backend, entries)

    def unpack(self, vec: int, out_ptr: int, n: Optional[int] = None) -> None:
        """Exchange vector -> plain f32 at out_ptr, waiting on the device for the pairs still under way."""
        from . import _lib
        _lib.check(_lib.load().vx_xvec_unpack(self.backend._ctx, self.vectors[vec].local.ptr,
                                              self.rows if n is None else n, out_ptr))

    def finish(self) -> None:
        """Arrival barrier across the GPUs, stream-ordered: after it every rank's earlier rows have landed."""
        from . import _lib
        _lib.check(_lib.load().vx_peer_barrier(self.backend._ctx, self._flags_all, self.world, self.rank))

    def close(self) -> None:
        self.backend.synchronize()
        self.y.close()
        self.flags.close()
        for v in self.vectors:
            v.close()


class ShardedGemm:
    """C[m, n] = A[m, k] B[k, n] (f32 in, TF32 tensor cores, f32 accumulate) with B and C split by columns
    across the ranks; A is replicated.  The full C ends up on every GPU, either way:

    * `dispatch_peer`: the kernel's epilogue stores every tile into each peer's C as well (NVLink stores,
      row stride n), then the arrival barrier kernel.
    * `dispatch_nccl`: the panel goes into a rank-major stack, NCCL all-gathers the stack, and a strided
      gather kernel (vortx's Contiguous) lays it out as row-major C."""

    def __init__(self, backend, m: int, n: int, k: int, group=None):
        import ctypes as C
        import torch.distributed as dist
        self.backend, self.m, self.n, self.k, self.group = backend, m, n, k, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("at most 8 GPUs of one node")
        self.col0, self.ncols = col_shard(n, self.world, self.rank)
        self.c = PeerBuffers(backend, m * n * 4, group)
        self.flags = PeerBuffers(backend, 64 * 4, group)
        self._others = [r for r in range(self.world) if r != self.rank]
        self._flags_all = (C.c_void_p * self.world)(*self.flags.ptrs)
        self._peer_c = (C.c_void_p * max(1, len(self._others)))(*[self.c.ptrs[r] + self.col0 * 4 for r in self._others])
        self._stack = None
        dist.barrier(group=group)

    def _shapes(self, out_stride: int, b_stride: int):
        from . import _lib
        sh = _lib.VxShapes3()
        for s, (h, w, hs) in ((sh.out, (self.m, self.ncols, out_stride)), (sh.lhs, (self.m, self.k, self.k)),
                              (sh.rhs, (self.k, self.ncols, b_stride))):
            s.n = s.c = 1
            s.h, s.w = h, w
            s.n_stride = s.c_stride = h * hs
            s.h_stride, s.w_stride = hs, 1
        return sh

    def dispatch_peer(self, a_ptr: int, b_panel_ptr: int, b_stride: int) -> None:
        """a_ptr: A, row-major contiguous.  b_panel_ptr: this rank's columns of B (first element), rows
        b_stride elements apart.  After the call, stream-ordered, self.c.local holds the whole C."""
        import ctypes as C
        from . import _lib
        sh = self._shapes(self.n, b_stride)
        if self.ncols:      # with fewer 32-column blocks than ranks, a rank may own no columns: it only takes part in the barrier
            _lib.check(_lib.load().vx_gemm_tf32_scatter(self.backend._ctx, self.c.local.ptr + self.col0 * 4, a_ptr,
                                                        b_panel_ptr, C.byref(sh), self._peer_c, len(self._others)))
        _lib.check(_lib.load().vx_peer_barrier(self.backend._ctx, self._flags_all, self.world, self.rank))

    def dispatch_nccl(self, a_ptr: int, b_panel_ptr: int, b_stride: int) -> None:
        """Same result through NCCL; needs equal panels.  The caller's current torch stream must be the
        backend's stream."""
        import ctypes as C
        import torch
        from . import _lib
        if self.n % self.world or (self.n // self.world) % 32:
            raise ValueError("the collective form takes equal panels of whole 32-column blocks")
        lib = _lib.load()
        if self._stack is None:
            self._stack = torch.empty(self.world, self.m, self.ncols, device="cuda", dtype=torch.float32)
        mine = self._stack[self.rank]
        sh = self._shapes(self.ncols, b_stride)
        _lib.check(lib.vx_gemm_f32(self.backend._ctx, _lib.VX_GEMM_TF32, mine.data_ptr(), a_ptr, b_panel_ptr,
                                   C.byref(sh), 0, 0, 0))
        self.dist_all_gather(mine)
        sizes, strides = panel_relayout_shape(self.m, self.world, self.ncols)
        shape = _lib.VxShape(*sizes, *strides)
        _lib.check(lib.vx_contiguous(self.backend._ctx, self.c.local.ptr, self.m * self.n, self._stack.data_ptr(),
                                     C.byref(shape), self._stack.numel(), 0))

    def dist_all_gather(self, mine) -> None:
        import torch.distributed as dist
        dist.all_gather_into_tensor(self._stack, mine, group=self.group)

    def close(self) -> None:
        self.backend.synchronize()
        self.c.close()
        self.flags.close()


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


class Group:
    """vx_group of the C ABI: an NCCL communicator plus IPC-mapped peer buffers, with no torch on the path.

    `Group.from_torch(backend)` only uses torch.distributed to carry rank 0's 128-byte unique id to the other
    ranks; a host without torch passes the bytes by any other means and calls `Group(backend, world, rank, id)`."""

    def __init__(self, backend, world: int, rank: int, unique_id: Optional[bytes]):
        import ctypes as C
        from . import _lib
        h = C.c_void_p()
        buf = (C.c_ubyte * 128).from_buffer_copy(unique_id) if unique_id else None
        _lib.check(_lib.load().vx_group_create(backend._ctx, world, rank, buf, C.byref(h)))
        self.backend, self.world, self.rank, self._h = backend, world, rank, h

    @staticmethod
    def unique_id() -> bytes:
        import ctypes as C
        from . import _lib
        buf = (C.c_ubyte * 128)()
        _lib.check(_lib.load().vx_group_unique_id(buf))
        return bytes(buf)

    @classmethod
    def from_torch(cls, backend) -> "Group":
        import torch.distributed as dist
        world, rank = dist.get_world_size(), dist.get_rank()
        box = [cls.unique_id() if rank == 0 and world > 1 else None]
        if world > 1:
            dist.broadcast_object_list(box, src=0)
        return cls(backend, world, rank, box[0])

    def peer_alloc(self, nbytes: int) -> List[int]:
        import ctypes as C
        from . import _lib
        ptrs = (C.c_void_p * self.world)()
        _lib.check(_lib.load().vx_group_peer_alloc(self._h, nbytes, ptrs))
        return [int(p or 0) for p in ptrs]

    def peer_free(self, ptrs: List[int]) -> None:
        import ctypes as C
        from . import _lib
        _lib.check(_lib.load().vx_group_peer_free(self._h, (C.c_void_p * self.world)(*ptrs)))

    def all_gather(self, recv_ptr: int, bytes_per_rank: int, send_ptr: int = 0) -> None:
        from . import _lib
        _lib.check(_lib.load().vx_group_all_gather(self._h, send_ptr or None, recv_ptr, bytes_per_rank))

    def broadcast(self, ptr: int, nbytes: int, root: int) -> None:
        from . import _lib
        _lib.check(_lib.load().vx_group_broadcast(self._h, ptr, nbytes, root))

    def barrier(self) -> None:
        from . import _lib
        _lib.check(_lib.load().vx_group_barrier(self._h))

    def gemv_q(self, slab, row0: int, x_ptr: int, y_all: List[int], y_offset: int = 0) -> None:
        """Row-sharded GEMV: `slab` is this rank's QuantizedMatrix; the whole y lands on every GPU."""
        import ctypes as C
        from . import _lib
        _lib.check(_lib.load().vx_group_gemv_q(self._h, slab._h, row0, x_ptr, (C.c_void_p * self.world)(*y_all), y_offset))

    def gemm_tf32(self, a_ptr: int, b_panel_ptr: int, m: int, n: int, k: int, col0: int, ncols: int, b_stride: int,
                  c_all: List[int]) -> None:
        import ctypes as C
        from . import _lib
        _lib.check(_lib.load().vx_group_gemm_tf32(self._h, a_ptr, b_panel_ptr, m, n, k, col0, ncols, b_stride,
                                                   (C.c_void_p * self.world)(*c_all)))

    def close(self) -> None:
        from . import _lib
        if self._h:
            self.backend.synchronize()
            _lib.load().vx_group_destroy(self._h)
        self._h = None
