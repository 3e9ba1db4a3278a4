#!/usr/bin/env python
"""Benchmark of the block-quantised GEMV hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("q4_0_gemv_28672x8192_x32"): the Q4_0 GEMV y = W x with W 28672 x 8192 (the FFN up-projection
shape of the multi-GPU configuration), x f32 of length 8192, W ~ N(0, 0.02) before quantisation,
x ~ N(0, 1), all seeded and synthetic.  One STEP is a pass over 32 such matrices held at 32 different
addresses (4.2 GB of weights at N = 1, far beyond the 126 MB L2), issued as ONE persistent list launch and
replayed from a CUDA graph.  With N > 1 the rows of every matrix are split into N contiguous slabs (strong
scaling: total work fixed); each rank computes its slab, and the kernel's epilogue stores every finished row
into the y of every GPU over NVLink (the all-gather of the output, fused into the GEMV); one barrier kernel per
step tells every rank that all rows of all 32 products have landed.  The same dependency structure at every N:
32 independent products.  The CHAINED form (product l + 1 takes its x from the rows every rank computed last
in product l, exchanged through flagged pairs inside the kernel) is reported at every N, 1 included, under
`extra.chained`, and NCCL's all-gather after every product under `extra.nccl_all_gather`.

The line printed by rank 0:
  value      algorithmic bytes per step / device time per step (weights resident in HBM, CUDA events, max over
             ranks; bytes per GEMV = 132 120 576 of blocks + 32 768 n of x + 114 688 of y).  The timed region is
             repeated in blocks of K steps for at least a second; the median block is reported, min / max beside it
  check      outside the timed region: products of the last step against the CPU oracle (f64), the gathered y
             identical on every rank, and the chained form bit for bit against the same chain run plainly on one GPU
  e2e        the same through the public API with host buffers: the step's x vectors are copied from pinned
             host memory, the products are read back to the host
  roofline   the list launch against the measured HBM copy bandwidth (and a read-only pass measured here)
  cpu_baseline  the CPU oracle's GEMV on the host cores, on a bounded sample (rank 0, N = 1)
`--impl reference` times that CPU implementation alone, on the same configuration.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS, COLS, LAYERS = 28672, 8192, 32
QBLOCK = 18  # bytes per Q4_0 block
METRIC = "q4_0_gemv_hbm_bandwidth"
UNIT = "GB/s"
WORKLOAD = "q4_0_gemv_28672x8192_x32"
CHECKED_PRODUCTS = (0, 13, 31)
# The end-to-end step runs as this many list launches, copies overlapped with their neighbours: 4 on one GPU; 2 on
# several, where every further stage costs a barrier kernel across the GPUs (measured at N = 2: 0.463 ms with 2
# stages, 0.482 with 4, 0.487 with 1).
E2E_STAGES_1GPU, E2E_STAGES_MULTI = 4, 2
# DRAM traffic of one 28672 x 8192 product inside a list launch: ncu dram__bytes_read + write of a list of 8
# (1060.5 MB, second captured launch) / 8, from profiles/gemv_stream_list_q4_0_28672x8192_x8.md
NCU_TRAFFIC_PER_PRODUCT = 132_560_000


def gemv_bytes(rows: int, cols: int, n_gpus: int = 1, batch: int = 1, qblock: int = QBLOCK) -> int:
    """Algorithmic bytes of one GEMV: weights once, x on each GPU, y once."""
    return rows * cols // 32 * qblock + batch * cols * 4 * n_gpus + batch * rows * 4


def measured_peak_hbm():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def slab_matrix(rows: int, seed: int) -> np.ndarray:
    """The f32 weights of one slab before quantisation: rows x COLS ~ N(0, 0.02)."""
    from vortx_b200 import synth
    return synth.normal_matrix(rows, COLS, seed)


# ------------------------------------------------------------------------ CPU arm ----

CPU_GEMVS_PER_STEP = 4  # of the step's 32: bounds the CPU arm to a fraction of a second per step


def cpu_gemv_rate(blocks: np.ndarray, rows: int, steps: int, warmup: int):
    """Times the CPU oracle's Q4_0 GEMV with all host threads: CPU_GEMVS_PER_STEP full-size GEMVs per step."""
    import oracle as o
    o.build()
    from vortx_b200 import synth
    threads = o.hardware_threads()
    x = synth.normal_vectors(1, COLS, seed=1)[0]
    for _ in range(max(warmup, 1)):
        o.gemv(o.Q4_0, blocks, rows, COLS, x, nthreads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        for _ in range(CPU_GEMVS_PER_STEP):
            o.gemv(o.Q4_0, blocks, rows, COLS, x, nthreads=threads)
    dt = (time.perf_counter() - t0) / steps
    gbs = CPU_GEMVS_PER_STEP * gemv_bytes(rows, COLS) / dt / 1e9
    return gbs, dt, threads


def run_reference(args):
    """`--impl reference`: the reference has no quantised GEMV and its CPU backend (khal) cannot be
    built here, so this arm times the CPU oracle's GEMV, the stand-in the parity tests use.  Nothing of the
    product library is loaded: the weights are quantised by the oracle's own quantiser."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle as o
    o.build()
    blocks = o.quantize(o.Q4_0, slab_matrix(ROWS, seed=100))
    gbs, dt, threads = cpu_gemv_rate(blocks, ROWS, args.steps, args.warmup)
    sample = (f"each step is {CPU_GEMVS_PER_STEP} of the workload's {LAYERS} GEMVs ({ROWS} x {COLS} Q4_0), "
              f"{threads} host threads; C++ restatement of the GEMV, not khal")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "q4_0 x f32 -> f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows": ROWS, "cols": COLS, "batch": 1, "sampled": sample},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------ GPU arm ----

def run_ours(args):
    # NCCL is only the rendezvous and the comparison form here.  NVLS off: a rank must never end while NCCL has
    # buffers bound to an NVLink multicast object.
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist
    import vortx_b200 as vb
    from vortx_b200 import _lib, synth
    from vortx_b200.multi_gpu import PeerBuffers

    t_start = time.perf_counter()

    def note(msg):
        if os.environ.get("VX_BENCH_VERBOSE"):
            print(f"[bench {time.perf_counter() - t_start:7.1f}s rank {os.environ.get('RANK', '0')}] {msg}",
                  file=sys.stderr, flush=True)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    note("process group ready")
    lib = _lib.load()
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    be = vb.Backend(local, stream=stream.cuda_stream)

    n = world
    assert ROWS % n == 0 and COLS % n == 0
    shard = ROWS // n
    row0 = rank * shard
    others = [r for r in range(n) if r != rank]

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        t = torch.tensor(list(values), device=dev, dtype=torch.float64)
        if n > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    # One quantised slab per rank (its own seed), uploaded LAYERS times to distinct addresses (identical bytes
    # are still distinct cache lines, and the step walks all of them before coming back).
    blocks = vb.quantize(vb.Q4_0, slab_matrix(shard, seed=100 + rank))
    layers = [vb.QuantizedMatrix(be, vb.Q4_0, blocks, shard, COLS) for _ in range(LAYERS)]
    xs_host = synth.normal_vectors(LAYERS, COLS, seed=1)        # e2e: one x per product; x 0 is the timed step's x
    x_dev = torch.from_numpy(xs_host[0]).to(dev)

    # Buffers every rank can store into: y of every product (full length), the barrier's flags, two exchange vectors.
    if n > 1:
        y_all = PeerBuffers(be, LAYERS * ROWS * 4)
        flags = PeerBuffers(be, 64 * 4)
        vecs = [PeerBuffers(be, lib.vx_xvec_bytes(ROWS)) for _ in range(2)]
        y_ptrs, flag_ptrs = y_all.ptrs, flags.ptrs
        vec_ptrs = [v.ptrs for v in vecs]
    else:
        y_buf = torch.zeros(LAYERS * ROWS, device=dev, dtype=torch.float32)
        vec_bufs = [torch.zeros(lib.vx_xvec_bytes(ROWS), device=dev, dtype=torch.uint8) for _ in range(2)]
        y_ptrs, flag_ptrs = [y_buf.data_ptr()], None
        vec_ptrs = [[v.data_ptr()] for v in vec_bufs]
    y_local = y_ptrs[rank]
    import ctypes as C
    flags_arr = (C.c_void_p * n)(*flag_ptrs) if n > 1 else None

    def finish():
        """One arrival barrier across the GPUs: after it, on this stream, every rank's rows have landed here."""
        if n > 1:
            _lib.check(lib.vx_peer_barrier(be._ctx, flags_arr, n, rank))

    def gather_list(x_ptrs, lo=0, hi=LAYERS):
        """Products lo .. hi - 1 of the step as ONE list launch: product l reads x_ptrs[l]; its rows go into y[l]
        here and on every peer."""
        entries = []
        for l in range(lo, hi):
            off = (l * ROWS + row0) * 4
            entries.append({"w": layers[l], "nrows": shard, "x": x_ptrs[l], "y": y_local + off,
                            "peer_y": [y_ptrs[r] + off for r in others]})
        return vb.GemvBatch(be, entries)

    def chain_list():
        """The chained step as one list launch: product 0 reads the plain x, product l the last COLS / n elements
        of every rank's slab of exchange vector (l - 1) % 2 — the rows every rank computes last — and writes
        vector l % 2 on every GPU."""
        seg_len, seg_stride = COLS // n, ROWS // n
        entries = []
        for l in range(LAYERS):
            e = {"w": layers[l], "nrows": shard, "y_xvec": vec_ptrs[l % 2][rank],
                 "peers": [vec_ptrs[l % 2][r] for r in others], "y_row0": row0, "y_stride": 1}
            if l == 0:
                e["x"] = x_dev.data_ptr()
            else:
                e["x_xvec"] = vec_ptrs[(l - 1) % 2][rank]
                e["x_seg_len"], e["x_seg_stride"], e["x_seg_first"] = seg_len, seg_stride, seg_stride - seg_len
            entries.append(e)
        return vb.GemvBatch(be, entries)

    value_batch = gather_list([x_dev.data_ptr()] * LAYERS)
    chain_batch = chain_list()
    chain_out = torch.zeros(ROWS, device=dev, dtype=torch.float32)

    def step_value():
        value_batch.launch()
        finish()

    def step_chain():
        chain_batch.launch()
        _lib.check(lib.vx_xvec_unpack(be._ctx, vec_ptrs[(LAYERS - 1) % 2][rank], ROWS, chain_out.data_ptr()))

    graphs = []     # every CUDA graph made here; all are destroyed before the process group goes away

    def capture(fn):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
        torch.cuda.synchronize()
        graphs.append(g)
        return g

    def time_blocks(g, steps, warmup, min_seconds=1.0, max_blocks=400):
        """Blocks of exactly `steps` replays, each bracketed by a barrier + synchronize and timed with CUDA events
        on the launching stream, repeated until `min_seconds` of device time have been covered.  Returns the
        per-step times (ms) of all blocks, each the max over ranks."""
        for _ in range(max(warmup, 3)):
            g.replay()
        barrier()
        blocks_ms, total = [], 0.0
        while True:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record(stream)
            for _ in range(steps):
                g.replay()
            e1.record(stream)
            barrier()
            blocks_ms.append(e0.elapsed_time(e1))
            total += blocks_ms[-1]
            # every rank must take the same number of blocks: decide on the max over ranks
            if max_over_ranks([total])[0] >= min_seconds * 1e3 or len(blocks_ms) >= max_blocks:
                break
        return [v / steps for v in max_over_ranks(blocks_ms)]

    note("weights uploaded")
    launches_before = be.launch_count()
    step_value()
    launches_per_step = be.launch_count() - launches_before
    graph = capture(step_value)
    note("step captured")

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    per_step = time_blocks(graph, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = statistics.median(per_step)
    bytes_per_step = LAYERS * gemv_bytes(ROWS, COLS, n)
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9
    note(f"timed region done: {len(per_step)} blocks of {args.steps} steps")

    # ---- check (outside the timed region): the last step's products against the oracle, on every rank's copy
    check = {"ok": True}
    import oracle as o
    o.build()
    y_host = np.empty(LAYERS * ROWS, np.float32)
    _lib.check(lib.vx_download(be._ctx, y_host.ctypes.data, y_local, y_host.nbytes))
    y_host = y_host.reshape(LAYERS, ROWS)
    want64, absdot = o.gemv_f64(o.Q4_0, blocks, shard, COLS, xs_host[:1])       # this rank's rows of every product
    if n > 1:
        parts = [torch.empty(2, shard, device=dev, dtype=torch.float64) for _ in range(n)]
        dist.all_gather(parts, torch.from_numpy(np.stack([want64[0], absdot[0]])).to(dev))
        full = torch.cat(parts, dim=1).cpu().numpy()
        want_full, absdot_full = full[0], full[1]
    else:
        want_full, absdot_full = want64[0], absdot[0]
    rels = []
    for l in CHECKED_PRODUCTS:
        diff = np.abs(y_host[l].astype(np.float64) - want_full)
        rels.append(float(diff.max() / np.abs(want_full).max()))
        check["ok"] = check["ok"] and rels[-1] <= 1e-4 and bool((diff <= 2e-6 * absdot_full).all())
    same = all(np.array_equal(y_host[l].view(np.uint32), y_host[0].view(np.uint32)) for l in range(LAYERS))
    check["ok"] = check["ok"] and same      # 32 copies of one matrix times one x: 32 identical products
    check["max_rel"] = max(rels)
    check["what"] = (f"products {list(CHECKED_PRODUCTS)} of the last timed step, all {ROWS} rows as gathered on this GPU, "
                     "against the f64 CPU oracle (max-norm relative <= 1e-4, every row within 2e-6 of sum|w||x|); "
                     "all 32 products bit-identical")
    if n > 1:
        # the gathered y is the same on every GPU
        digest = torch.from_numpy(y_host.view(np.int32).astype(np.int64).sum(axis=1)).to(dev)
        lo, hi = digest.clone(), digest.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        check["same_on_every_rank"] = bool(torch.equal(lo, hi))
        check["ok"] = check["ok"] and check["same_on_every_rank"]
    note("value form checked")

    # ---- the chained form, at every N
    chain_graph = capture(step_chain)
    chain_steps = time_blocks(chain_graph, args.steps, args.warmup, min_seconds=0.3)
    chain_ms = statistics.median(chain_steps)
    chain_got = chain_out.cpu().numpy()
    chained = {"ms_per_step": chain_ms, "GB/s": bytes_per_step / (chain_ms * 1e-3) / 1e9,
               "us_per_product": chain_ms * 1e3 / LAYERS,
               "what": "32 dependent products in one list launch per GPU; x of product l + 1 = the last 8192 / N rows "
                       "every rank computed in product l, exchanged as {value, generation} pairs inside the kernel"}
    # bit for bit against the same chain run plainly on ONE GPU (rank 0 gets every slab)
    if n > 1:
        mine = torch.from_numpy(blocks).to(dev)
        slabs = [torch.empty_like(mine) for _ in range(n)]
        dist.all_gather(slabs, mine)
        whole_blocks = torch.cat(slabs).cpu().numpy() if rank == 0 else None
    else:
        whole_blocks = blocks
    chain_ok = True
    if rank == 0:
        whole = vb.QuantizedMatrix(be, vb.Q4_0, whole_blocks, ROWS, COLS)
        yp = torch.empty(ROWS, device=dev, dtype=torch.float32)
        xn = torch.empty(COLS, device=dev, dtype=torch.float32)
        seg_len, seg_stride = COLS // n, ROWS // n
        src = x_dev.data_ptr()
        for l in range(LAYERS):
            _lib.check(lib.vx_gemv_q_rows(be._ctx, whole._h, 0, ROWS, src, COLS, yp.data_ptr(), ROWS, 1))
            for s_ in range(n):
                _lib.check(lib.vx_copy(be._ctx, xn.data_ptr() + s_ * seg_len * 4,
                                       yp.data_ptr() + ((s_ + 1) * seg_stride - seg_len) * 4, seg_len * 4))
            src = xn.data_ptr()
        be.synchronize()
        chain_want = yp.cpu().numpy()
        whole.free()
        chain_ok = bool(np.array_equal(chain_want.view(np.uint32), chain_got.view(np.uint32))) and \
            bool(np.isfinite(chain_got).all()) and float(np.abs(chain_got).max()) > 0.0
    if n > 1:
        # every rank ended on the same vector
        d = torch.tensor([int(chain_got.view(np.int32).astype(np.int64).sum())], device=dev)
        lo, hi = d.clone(), d.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        chain_ok = chain_ok and bool(torch.equal(lo, hi))
    chained["check_ok"] = chain_ok
    check["chained_ok"] = chain_ok
    check["ok"] = check["ok"] and chain_ok
    note("chained form timed and checked")

    # ---- kernel-only figure for the roofline: the list launch over this GPU's rows with no exchange at all
    plain_batch = vb.GemvBatch(be, [{"w": layers[l], "x": x_dev.data_ptr(), "y": y_local + (l * ROWS + row0) * 4}
                                    for l in range(LAYERS)])

    def time_graph(fn, reps):
        g = capture(fn)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(stream)
        for _ in range(reps):
            g.replay()
        k1.record(stream)
        torch.cuda.synchronize()
        return k0.elapsed_time(k1) * 1e3 / reps      # us per replay

    reps = max(3, args.steps)
    launch_us = time_graph(plain_batch.launch, reps)

    def separate():
        for l in range(LAYERS):
            _lib.check(lib.vx_gemv_q_rows(be._ctx, layers[l]._h, 0, shard, x_dev.data_ptr(), COLS,
                                          y_local + (l * ROWS + row0) * 4, shard, 1))
    separate_us = time_graph(separate, reps) / LAYERS
    shard_bytes = gemv_bytes(shard, COLS)
    list_bytes = LAYERS * shard_bytes
    peak, peak_kind = measured_peak_hbm()
    achieved = list_bytes / (launch_us * 1e-6) / 1e9
    # a read-only pass (vx_checksum_u32: streaming 16-byte loads, nothing written) over one 4 GiB buffer, as a
    # second denominator beside the copy bandwidth; and the weights' own checksums, which must all agree
    probe = torch.empty(1 << 32, device=dev, dtype=torch.uint8)
    probe.fill_(1)
    sums = torch.zeros(LAYERS + 1, device=dev, dtype=torch.int32)

    def read_only():
        _lib.check(lib.vx_checksum_u32(be._ctx, probe.data_ptr(), probe.numel(), sums.data_ptr() + 4 * LAYERS))
    read_us = time_graph(read_only, max(3, min(reps, 10)))
    read_only_gbs = probe.numel() / (read_us * 1e-6) / 1e9
    del probe
    for l in range(LAYERS):
        _lib.check(lib.vx_qweights_checksum(be._ctx, layers[l]._h, sums.data_ptr() + 4 * l))
    check["weights_intact"] = bool((sums[:LAYERS] == sums[0]).all().item())      # 32 uploads of the same bytes
    check["ok"] = check["ok"] and check["weights_intact"]
    note("kernel-only timing done")

    # ---- end to end through the public API with host buffers (vx_gemv_batch_run_host): the step's 32 x vectors
    # (all different) come from pinned host memory and every product goes back to it — rank 0's host reads every
    # product whole, the other ranks' hosts the rows their GPU computed.  The step is cut into E2E_STAGES stages
    # (a list launch each, + barrier at N > 1) so that a stage's copies run beside its neighbours' kernels.
    xs_pin = torch.from_numpy(xs_host).pin_memory()
    ys_pin = torch.empty(LAYERS, ROWS, dtype=torch.float32).pin_memory()
    xs_dev = torch.empty(LAYERS, COLS, device=dev, dtype=torch.float32)
    x_ptrs_e2e = [xs_dev[l].data_ptr() for l in range(LAYERS)]
    e2e_batches, e2e_stages = [], []
    E2E_STAGES = E2E_STAGES_1GPU if n == 1 else E2E_STAGES_MULTI
    per_stage = LAYERS // E2E_STAGES
    for i in range(E2E_STAGES):
        lo, hi = i * per_stage, (i + 1) * per_stage
        e2e_batches.append(gather_list(x_ptrs_e2e, lo, hi))
        first, width = (0, ROWS) if rank == 0 else (row0, shard)
        off = (lo * ROWS + first) * 4
        stage = {"batch": e2e_batches[-1],
                 "up": (xs_dev.data_ptr() + lo * COLS * 4, xs_pin.data_ptr() + lo * COLS * 4, per_stage * COLS * 4),
                 "down": (ys_pin.data_ptr() + off, ROWS * 4, y_local + off, ROWS * 4, width * 4, per_stage)}
        if n > 1:
            stage["barrier"] = (flag_ptrs, rank)
        e2e_stages.append(stage)
    barrier()
    e2e_recorded = True
    try:
        e2e_run = vb.HostStages(be, e2e_stages, recorded=True)     # vx_host_pipeline: the step recorded once, replayed per step
    except vb.VortxError as err:                                   # the immediate form does the same work call by call
        note(f"recording the end-to-end step failed ({err}); running it unrecorded")
        e2e_recorded = False
        e2e_run = vb.HostStages(be, e2e_stages)

    def step_e2e():
        e2e_run.run()

    for _ in range(3):
        step_e2e()
    barrier()
    e2e_steps = max(5, min(args.steps, 20))
    e2e_blocks = []
    for _ in range(5):
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            step_e2e()
        barrier()
        e2e_blocks.append((time.perf_counter() - t0) * 1e3 / e2e_steps)
    e2e_ms = statistics.median(max_over_ranks(e2e_blocks))
    e2e_value = bytes_per_step / (e2e_ms * 1e-3) / 1e9
    # the e2e results too: different x per product, so every product has its own answer
    e2e_rels = []
    if rank == 0:
        for l in CHECKED_PRODUCTS:
            w64, ad = o.gemv_f64(o.Q4_0, blocks, shard, COLS, xs_host[l:l + 1])
            got = ys_pin[l, row0:row0 + shard].numpy()
            diff = np.abs(got.astype(np.float64) - w64[0])
            e2e_rels.append(float(diff.max() / np.abs(w64[0]).max()))
            check["ok"] = check["ok"] and e2e_rels[-1] <= 1e-4 and bool((diff <= 2e-6 * ad[0]).all())
        check["e2e_max_rel"] = max(e2e_rels)
    note("end-to-end timing done")

    extra = {"chained": chained,
             "timed_region": {"blocks": len(per_step), "steps_per_block": args.steps,
                              "ms_per_step_median": ms_per_step, "ms_per_step_min": min(per_step),
                              "ms_per_step_max": max(per_step), "seconds": sum(per_step) * args.steps * 1e-3},
             "read_only_pass": {"GB/s": read_only_gbs, "kernel": "checksum_kernel, one launch over a 4 GiB buffer",
                                "frac_of_copy_peak": read_only_gbs / peak}}
    if n > 1:
        extra["kernels_only"] = {"us_per_list_launch": launch_us, "GB/s_per_gpu": achieved}
        # NCCL's all-gather after every product (the wording of the configuration), launched eagerly: no NCCL
        # kernel is ever captured in a CUDA graph here
        y_t = [torch.empty(ROWS, device=dev, dtype=torch.float32) for _ in range(LAYERS)]

        def step_nccl():
            for l in range(LAYERS):
                _lib.check(lib.vx_gemv_q_rows(be._ctx, layers[l]._h, 0, shard, x_dev.data_ptr(), COLS,
                                              y_t[l].data_ptr() + row0 * 4, shard, 1))
                dist.all_gather_into_tensor(y_t[l], y_t[l][row0:row0 + shard])
        for _ in range(3):
            step_nccl()
        barrier()
        n0, n1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0.record(stream)
        for _ in range(max(3, min(args.steps, 10))):
            step_nccl()
        n1.record(stream)
        barrier()
        nccl_ms = max_over_ranks([n0.elapsed_time(n1)])[0] / max(3, min(args.steps, 10))
        nccl_same = bool(np.array_equal(y_t[5].cpu().numpy().view(np.uint32), y_host[5].view(np.uint32)))
        extra["nccl_all_gather"] = {"ms_per_step": nccl_ms, "GB/s": bytes_per_step / (nccl_ms * 1e-3) / 1e9,
                                    "launch": "eager (no graph)", "same_bits_as_fused": nccl_same}
        check["ok"] = check["ok"] and nccl_same
        note("NCCL form timed")
        # (the headline numbers above must not be lost to a failure in this side measurement: every rank
        # runs the same code, so a library error raises on all of them alike)
        try:
            extra["gemm_tf32_8192_col_sharded"] = sharded_gemm_numbers(be, torch, dist, stream, n, rank, barrier)
        except _lib.VortxError as e:
            extra["gemm_tf32_8192_col_sharded"] = {"failed": str(e)}
    cpu = None
    if rank == 0 and n == 1:
        try:
            extra.update(side_configs(be, lib, torch, stream))
        except (_lib.VortxError, RuntimeError) as e:      # a side configuration must not take the headline line with it
            extra["side_configs_failed"] = str(e)
        try:
            gbs, dt, threads = cpu_gemv_rate(blocks, ROWS, steps=5, warmup=1)
            cpu = {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"5 x {CPU_GEMVS_PER_STEP} GEMVs of {ROWS} x {COLS} Q4_0 (the step has {LAYERS}); "
                             "C++ restatement of the GEMV, not khal"}
            extra["cpu_baselines"] = cpu_side_baselines(o, threads)
        except Exception as e:  # the oracle is test infrastructure; its absence must not hide the GPU numbers
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"unavailable: {e}"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "q4_0 x f32 (24-bit fixed point) -> f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows": ROWS, "cols": COLS, "batch": 1,
                       "gemv_per_step": LAYERS,
                       "sharding": (f"rows/{n} per GPU; every row stored into the y of every GPU by the kernel's epilogue "
                                    "(NVLink stores), one barrier kernel per step") if n > 1 else "none",
                       "dependencies": "32 independent products per step at every N (the chained form: extra.chained)",
                       "l2": "inputs larger than L2: 32 weight copies walked in turn",
                       "launch": "CUDA graph replay; the 32 products of a step are one persistent list launch",
                       "timed": f"median of {len(per_step)} blocks of {args.steps} steps"},
            "check": check,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": LAYERS * COLS * 4, "d2h_bytes_per_step": LAYERS * ROWS * 4,
                    "stages": E2E_STAGES, "recorded_as_graph": e2e_recorded,
                    "what": f"per step, in {E2E_STAGES} stages whose copies overlap the neighbouring stages' kernels: "
                            "32 x vectors up from pinned memory, the list launches"
                            + (" + barrier kernels" if n > 1 else "") + ", every product down to rank 0's host"
                            + (" (the other ranks read back the rows they computed)" if n > 1 else "")},
            "gpu_launches": launches_per_step * args.steps * len(per_step),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"{peak_kind} HBM copy bandwidth (read + write)", "datasheet_peak": 8000.0,
                         "frac_datasheet": achieved / 8000.0, "read_only_peak": read_only_gbs,
                         "frac_read_only": achieved / read_only_gbs, "kernel": "gemv_stream_kernel (list launch)",
                         "bytes_per_launch": list_bytes, "us_per_launch": launch_us, "gemvs_per_launch": LAYERS,
                         "one_gemv_per_launch": {"us_per_launch": separate_us, "bytes_per_launch": shard_bytes,
                                                 "achieved": shard_bytes / (separate_us * 1e-6) / 1e9},
                         "traffic": LAYERS * NCU_TRAFFIC_PER_PRODUCT if n == 1 else None,
                         "traffic_source": "ncu dram__bytes_read + dram__bytes_write of a list launch of 8 products "
                                           "(1060.5 MB) scaled by 32 / 8: every product reads its own matrix once"},
            "clocks": clocks,
            "extra": extra,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        emit(line)

    # ---- leave cleanly: lists and graphs first (a CUDA graph that captured work keeps references alive), then the
    # IPC mappings, then a last barrier with nothing in flight.  The process group is not torn down collectively:
    # every rank is past the barrier, has nothing in flight and holds no NVLS binding, and simply exits.
    e2e_run.free()
    for b in [value_batch, chain_batch, plain_batch] + e2e_batches:
        b.free()
    graphs.clear()
    graph = chain_graph = None
    import gc
    gc.collect()
    torch.cuda.synchronize()
    if n > 1:
        dist.barrier()
        for pb in [y_all, flags] + vecs:
            pb.close()
        barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def cpu_side_baselines(o, threads):
    """The CPU restatement on the other configurations, each a bounded sample with all host threads (reported
    baselines, not targets): the tiled GEMM at 1024^3 and 2048^3, the Q8_0 GEMV 4096^2, the Q4_0 GEMV 8192^2."""
    from vortx_b200 import synth
    out = {"cores": threads, "kind": "port", "note": "C++ restatement of vortx-shaders on the host cores, not khal"}
    for dim, reps in ((1024, 3), (2048, 1)):
        a, b = synth.uniform_matrix(dim, dim, 0), synth.uniform_matrix(dim, dim, 1)
        c = np.zeros(dim * dim, np.float32)
        sh = o.shape_contiguous(1, 1, dim, dim)
        o.gemm_tiled(c, a.ravel(), b.ravel(), sh, sh, sh, nthreads=threads)
        t0 = time.perf_counter()
        for _ in range(reps):
            o.gemm_tiled(c, a.ravel(), b.ravel(), sh, sh, sh, nthreads=threads)
        dt = (time.perf_counter() - t0) / reps
        out[f"gemm_tiled_{dim}"] = {"ms": dt * 1e3, "GFLOP/s": 2 * dim ** 3 / dt / 1e9, "sample": f"{reps} call(s) after one warm-up"}
    out["gemm_tiled_8192"] = "skipped: minutes per call with this SIMT-shaped code"
    for name, qt, dim, bb in (("q8_0_gemv_4096x4096", o.Q8_0, 4096, 34), ("q4_0_gemv_8192x8192", o.Q4_0, 8192, 18)):
        blocks = o.quantize(qt, synth.normal_matrix(dim, dim, seed=0))
        x = synth.normal_vectors(1, dim, seed=1)[0]
        o.gemv(qt, blocks, dim, dim, x, nthreads=threads)
        t0 = time.perf_counter()
        for _ in range(10):
            o.gemv(qt, blocks, dim, dim, x, nthreads=threads)
        dt = (time.perf_counter() - t0) / 10
        out[name] = {"ms": dt * 1e3, "GB/s": gemv_bytes(dim, dim, 1, 1, bb) / dt / 1e9, "sample": "10 calls after one warm-up"}
    # the kernels around the path: a += b and the sum of 4096 x 4096 f32 (the restatements are single-threaded, as
    # the shaders' one-element-per-invocation form is)
    dim = 4096
    a = synth.uniform_matrix(dim, dim, 2).ravel().copy()
    b = synth.uniform_matrix(dim, dim, 3).ravel().copy()
    sh = o.shape_contiguous(1, 1, dim, dim)
    t0 = time.perf_counter()
    o.op_assign(0, a, sh, b, sh)
    dt = time.perf_counter() - t0
    out["op_assign_add_4096x4096"] = {"ms": dt * 1e3, "GB/s": 3 * dim * dim * 4 / dt / 1e9, "cores": 1, "sample": "1 call"}
    t0 = time.perf_counter()
    o.reduce(b, "sum")
    dt = time.perf_counter() - t0
    out["reduce_sum_16Mi"] = {"ms": dt * 1e3, "GB/s": dim * dim * 4 / dt / 1e9, "cores": 1, "sample": "1 call"}
    return out


def sharded_gemm_numbers(be, torch, dist, stream, world, rank, barrier):
    """C = A B at 8192^3 with B and C split by columns over the ranks (A replicated), the full C on every GPU:
    panel compute alone, the peer-store epilogue + barrier kernel, and NCCL all-gather + re-layout.  Device time
    of `iters` back-to-back products, max over ranks; TFLOP/s counts the whole product's flops."""
    from vortx_b200.multi_gpu import ShardedGemm
    import ctypes as C
    from vortx_b200 import _lib
    lib = _lib.load()
    dim, iters = 8192, 5
    g = ShardedGemm(be, dim, dim, dim)
    gen = torch.Generator(device="cuda").manual_seed(5)
    a = torch.rand(dim, dim, device="cuda", generator=gen) * 2 - 1
    b = torch.rand(dim, g.ncols, device="cuda", generator=gen) * 2 - 1       # this rank's columns of B
    local_c = torch.empty(dim, dim, device="cuda")
    sh = g._shapes(dim, g.ncols)

    def compute_only():
        _lib.check(lib.vx_gemm_f32(be._ctx, _lib.VX_GEMM_TF32, local_c.data_ptr() + g.col0 * 4, a.data_ptr(), b.data_ptr(),
                                   C.byref(sh), 0, 0, 0))

    def peer_tile128():
        be.set_option("gemm.tf32.tile_m", 128)      # two accumulator stages: the peer stores run under the next tile's MMAs
        g.dispatch_peer(a.data_ptr(), b.data_ptr(), g.ncols)
        be.set_option("gemm.tf32.tile_m", 0)

    forms = {"compute_only": compute_only,
             "peer_stores": lambda: g.dispatch_peer(a.data_ptr(), b.data_ptr(), g.ncols),
             "peer_stores_tile128": peer_tile128,
             "nccl_all_gather": lambda: g.dispatch_nccl(a.data_ptr(), b.data_ptr(), g.ncols)}
    out = {"m=n=k": dim, "columns_per_gpu": g.ncols, "iters": iters}
    flops = 2.0 * dim ** 3
    for name, fn in forms.items():
        for _ in range(2):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item()) / iters
        out[name] = {"ms": ms, "TFLOP/s": flops / (ms * 1e-3) / 1e12}
    g.close()
    return out


def side_configs(be, lib, torch, stream):
    """The other benchmark configurations, each timed briefly (graph replay, rotating weight copies)."""
    import vortx_b200 as vb
    from vortx_b200 import _lib, synth
    import ctypes as C
    out = {}

    def time_graph(fn, n_launch, reps=5):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            g.replay()
        b.record(stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / (reps * n_launch)

    peak, _ = measured_peak_hbm()
    for name, qt, rows, cols, batches, copies in (("q8_0_gemv_4096x4096", vb.Q8_0, 4096, 4096, (1,), 24),
                                                  ("q4_0_gemv_8192x8192", vb.Q4_0, 8192, 8192, (1, 4, 8), 12),
                                                  # the down-projection shape: rows too long for 8-row tiles
                                                  ("q4_0_gemv_8192x28672", vb.Q4_0, 8192, 28672, (1,), 6)):
        blocks = vb.quantize(qt, synth.normal_matrix(rows, cols, seed=0))
        ws = [vb.QuantizedMatrix(be, qt, blocks, rows, cols) for _ in range(copies)]
        qb = lib.vx_qblock_bytes(qt)
        for b in batches:
            x = torch.randn(b, cols, device="cuda")
            y = torch.empty(b, rows, device="cuda")

            def fn():
                for w in ws:
                    _lib.check(lib.vx_gemv_q_rows(be._ctx, w._h, 0, rows, x.data_ptr(), cols, y.data_ptr(), rows, b))
            us = time_graph(fn, copies)
            byts = gemv_bytes(rows, cols, 1, b, qb)
            out[f"{name}_b{b}"] = {"us": us, "GB/s": byts / us / 1e3, "frac_of_measured_hbm": byts / us / 1e3 / peak}
            if b == 1:
                # the same products as one list launch over the rotating weight copies
                batch = vb.GemvBatch(be, [{"w": w, "x": x.data_ptr(), "y": y.data_ptr()} for w in ws])
                us = time_graph(batch.launch, copies)
                out[f"{name}_b1_list_of_{copies}"] = {"us_per_gemv": us, "GB/s": byts / us / 1e3,
                                                      "frac_of_measured_hbm": byts / us / 1e3 / peak}
                batch.free()
                # hot-L2 variant, reported separately: the same matrix in every entry (fits the 126 MB L2 when
                # the matrix does), so the list runs at the integer pipe's rate, not HBM's
                if byts < 100e6:
                    batch = vb.GemvBatch(be, [{"w": ws[0], "x": x.data_ptr(), "y": y.data_ptr()} for _ in range(copies)])
                    us = time_graph(batch.launch, copies)
                    out[f"{name}_b1_list_hot_l2"] = {"us_per_gemv": us, "GB/s_weights_from_l2": byts / us / 1e3}
                    batch.free()
            if b == 8 and len(ws) >= 8:
                # eight of the matrices times the same eight vectors in one call (vx_gemv_q_multi): the planes of x
                # are made once, one launch walks the matrices
                ys8 = [torch.empty(b, rows, device="cuda") for _ in range(8)]
                gemv = vb.Gemv()

                def fn8():
                    gemv.dispatch_multi(be, None, [t.data_ptr() for t in ys8], ws[:8], x.data_ptr(), batch=b,
                                        x_stride=cols, y_stride=rows)
                us = time_graph(fn8, 8)
                out[f"{name}_b8_multi_of_8"] = {"us_per_matrix": us, "GB/s": byts / us / 1e3,
                                                "frac_of_measured_hbm": byts / us / 1e3 / peak}
        for w in ws:
            w.free()

    # f32 GEMM 1024^3, exact SIMT path (and the TF32 path at 8192^3 when the device has room).
    for name, mode, dim in (("gemm_f32_simt_exact_1024", _lib.VX_GEMM_SIMT_EXACT, 1024),
                            ("gemm_tf32_4096", _lib.VX_GEMM_TF32, 4096),
                            ("gemm_tf32_8192", _lib.VX_GEMM_TF32, 8192)):
        A = torch.rand(dim, dim, device="cuda") * 2 - 1
        B = torch.rand(dim, dim, device="cuda") * 2 - 1
        Cm = torch.empty(dim, dim, device="cuda")
        sh = _lib.VxShapes3()
        for s in (sh.out, sh.lhs, sh.rhs):
            s.n = s.c = 1
            s.h = s.w = dim
            s.n_stride = s.c_stride = dim * dim
            s.h_stride, s.w_stride = dim, 1

        def fn():
            _lib.check(lib.vx_gemm_f32(be._ctx, mode, Cm.data_ptr(), A.data_ptr(), B.data_ptr(), C.byref(sh), 0, 0, 0))
        us = time_graph(fn, 1, reps=3)
        k = C.c_int32()
        lib.vx_gemm_last_kernel(be._ctx, C.byref(k))
        out[name] = {"us": us, "TFLOP/s": 2 * dim ** 3 / us / 1e6, "kernel": int(k.value)}
        # the reference example's own protocol (examples/gemm_bench.rs:11-12, :80-89): 3 warm-up calls, 10 timed
        # calls, a synchronise after each, wall clock
        for _ in range(3):
            fn()
            be.synchronize()
        t0 = time.perf_counter()
        for _ in range(10):
            fn()
            be.synchronize()
        out[name]["reference_protocol_ms"] = (time.perf_counter() - t0) * 1e3 / 10
        if mode == _lib.VX_GEMM_TF32:
            be.set_option("gemm.tf32.tma_store", 0)     # the epilogue warps store C themselves
            us = time_graph(fn, 1, reps=3)
            be.set_option("gemm.tf32.tma_store", 1)
            out[name]["plain_store_epilogue"] = {"us": us, "TFLOP/s": 2 * dim ** 3 / us / 1e6}
            # sustained: the same product back to back for at least a second (the burst figure above is three calls)
            reps = max(10, int(1.2e6 / us))
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(reps):
                fn()
            b.record(stream)
            torch.cuda.synchronize()
            sus = a.elapsed_time(b) * 1e3 / reps
            out[name]["sustained"] = {"us": sus, "TFLOP/s": 2 * dim ** 3 / sus / 1e6, "calls": reps,
                                      "seconds": sus * reps * 1e-6}
            # cuBLAS TF32 on the same inputs (torch.matmul with TF32 allowed): the library figure beside ours
            prev = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = True
            try:
                for _ in range(3):
                    torch.matmul(A, B, out=Cm)
                torch.cuda.synchronize()
                a.record(stream)
                for _ in range(3):
                    torch.matmul(A, B, out=Cm)
                b.record(stream)
                torch.cuda.synchronize()
                cb = a.elapsed_time(b) * 1e3 / 3
                reps_c = max(10, int(1.2e6 / cb))
                a.record(stream)
                for _ in range(reps_c):
                    torch.matmul(A, B, out=Cm)
                b.record(stream)
                torch.cuda.synchronize()
                cs = a.elapsed_time(b) * 1e3 / reps_c
                out[name]["cublas_tf32"] = {"us": cb, "TFLOP/s": 2 * dim ** 3 / cb / 1e6,
                                            "sustained_us": cs, "sustained_TFLOP/s": 2 * dim ** 3 / cs / 1e6}
            finally:
                torch.backends.cuda.matmul.allow_tf32 = prev
        del A, B, Cm

    # The reference example's sweep (examples/gemm_bench.rs:29, :70-115): naive against tiled at every size, 3 warm-up
    # and 10 timed calls with a synchronise after each, wall clock; the tensor-core kernel beside them.
    sweep = []
    for dim in (64, 128, 256, 512, 768, 1024, 1536, 2048, 4096):
        A = torch.rand(dim, dim, device="cuda") * 2 - 1
        B = torch.rand(dim, dim, device="cuda") * 2 - 1
        Cm = torch.empty(dim, dim, device="cuda")
        sh = _lib.VxShapes3()
        for s in (sh.out, sh.lhs, sh.rhs):
            s.n = s.c = 1
            s.h = s.w = dim
            s.n_stride = s.c_stride = dim * dim
            s.h_stride, s.w_stride = dim, 1
        row = {"size": dim}
        for label, mode in (("naive_ms", _lib.VX_GEMM_NAIVE), ("tiled_ms", _lib.VX_GEMM_SIMT_EXACT), ("tf32_ms", _lib.VX_GEMM_TF32)):
            def call():
                _lib.check(lib.vx_gemm_f32(be._ctx, mode, Cm.data_ptr(), A.data_ptr(), B.data_ptr(), C.byref(sh), 0, 0, 0))
                be.synchronize()
            for _ in range(3):
                call()
            t0 = time.perf_counter()
            for _ in range(10):
                call()
            row[label] = (time.perf_counter() - t0) * 1e3 / 10
        row["speedup_tiled_over_naive"] = row["naive_ms"] / row["tiled_ms"]
        sweep.append(row)
        del A, B, Cm
    out["gemm_bench_sweep"] = {"protocol": "3 warm-up + 10 timed calls, synchronise after each, wall clock", "rows": sweep}

    # The kernels around the matmul path (reductions, OpAssign / Contiguous / Repeat) on 8192 x 8192 f32 operands
    # (268 MB each, beyond L2), against the HBM copy peak; algorithmic bytes = every operand element read or
    # written once.
    D = 8192
    cases, keep = elementwise_cases(be, lib, D, big=True)
    ew = {}
    for name, operands, call in cases:
        def fn(call=call):
            _lib.check(call())
        us = time_graph(fn, 1, reps=10)
        byts = int(operands * D * D * 4)
        ew[name] = {"us": us, "GB/s": byts / us / 1e3, "frac_of_measured_hbm": byts / us / 1e3 / peak}
    out["elementwise_and_reduce_8192x8192_f32"] = ew
    del cases, keep
    return out


def elementwise_cases(be, lib, D, big=False):
    """The element-wise and reduction calls timed under `extra` (and launched by the `elementwise_8192` profile
    case): (name, operands of D x D f32 moved, call), and the tensors that must outlive the calls.  `big` adds
    the reductions over 2^30 elements (4 GiB), where launch and tail no longer count."""
    import ctypes as C
    import torch
    from vortx_b200 import _lib
    A = torch.rand(D * D, device="cuda")
    B = torch.rand(D * D, device="cuda") + 1.0
    O = torch.empty(D * D, device="cuda")
    res = torch.zeros(4, device="cuda")

    def shp(n, c, h, w, ns, cs, hs, ws_):
        s_ = _lib.VxShape()
        s_.n, s_.c, s_.h, s_.w, s_.n_stride, s_.c_stride, s_.h_stride, s_.w_stride = n, c, h, w, ns, cs, hs, ws_
        return s_
    dense, transp = shp(1, 1, D, D, D * D, D * D, D, 1), shp(1, 1, D, D, D * D, D * D, 1, D)
    one_row = shp(1, 1, D, D, 0, 0, 0, 1)
    small = shp(1, 1, 64, 64, 4096, 4096, 64, 1)
    vec = shp(1, 1, 1, D * D, D * D, D * D, D * D, 1)
    cases = (
        ("op_assign_add_dense", 3, lambda: lib.vx_op_assign(be._ctx, 0, A.data_ptr(), C.byref(dense), 0, B.data_ptr(), C.byref(dense), 0, 0, 0)),
        ("op_assign_add_row_broadcast", 2, lambda: lib.vx_op_assign(be._ctx, 0, A.data_ptr(), C.byref(dense), 0, B.data_ptr(), C.byref(one_row), 0, 0, 0)),
        ("op_assign_add_transposed_b", 3, lambda: lib.vx_op_assign(be._ctx, 0, A.data_ptr(), C.byref(dense), 0, B.data_ptr(), C.byref(transp), 0, 0, 0)),
        ("contiguous_of_transposed", 2, lambda: lib.vx_contiguous(be._ctx, O.data_ptr(), 0, B.data_ptr(), C.byref(transp), 0, 0)),
        ("repeat_64x64_tile", 1, lambda: lib.vx_repeat(be._ctx, O.data_ptr(), C.byref(dense), 0, B.data_ptr(), C.byref(small), 0)),
        ("reduce_sum_wide", 1, lambda: lib.vx_reduce(be._ctx, 0, 0, 1, B.data_ptr(), C.byref(vec), 0, res.data_ptr())),
        ("reduce_max_wide", 1, lambda: lib.vx_reduce(be._ctx, 3, 0, 1, B.data_ptr(), C.byref(vec), 0, res.data_ptr())),
    )
    keep = [A, B, O, res, dense, transp, one_row, small, vec]
    if big:
        n_big = 1 << 30
        G = torch.rand(n_big, device="cuda")
        vbig = shp(1, 1, 1, n_big, n_big, n_big, n_big, 1)
        keep += [G, vbig]
        cases = cases + (
            ("reduce_sum_wide_1Gi", n_big / (D * D), lambda: lib.vx_reduce(be._ctx, 0, 0, 1, G.data_ptr(), C.byref(vbig), 0, res.data_ptr())),
            ("reduce_max_wide_1Gi", n_big / (D * D), lambda: lib.vx_reduce(be._ctx, 3, 0, 1, G.data_ptr(), C.byref(vbig), 0, res.data_ptr())),
        )
    return cases, keep


PROFILE_CASES = {
    # name: (kind, rows/dim, cols, qtype name, weight copies)
    "gemv_q4_0_28672x8192": ("gemv", 28672, 8192, "Q4_0", 2),
    "gemv_q4_0_8192x8192": ("gemv", 8192, 8192, "Q4_0", 4),
    "gemv_list_q4_0_28672x8192_x8": ("gemv_list", 28672, 8192, "Q4_0", 8),   # one list launch over 8 weight copies
    "gemv_q8_0_4096x4096": ("gemv", 4096, 4096, "Q8_0", 8),
    "gemv_mma_q4_0_8192x8192_b8": ("gemv_batch", 8192, 8192, "Q4_0", 8),     # tensor-core batch kernel, 8 vectors
    "gemv_mma_q4_0_8192x8192_b2": ("gemv_batch", 8192, 8192, "Q4_0", 2),     # its one-MMA form, 2 vectors
    "gemv_mma_q4_0_28672x8192_b8": ("gemv_batch", 28672, 8192, "Q4_0", 8),
    "gemv_mma_q4_0_28672x8192_b2": ("gemv_batch", 28672, 8192, "Q4_0", 2),
    "gemv_mma_q8_0_4096x4096_b8": ("gemv_batch", 4096, 4096, "Q8_0", 8),
    "gemm_simt_exact_1024": ("gemm", 1024, 1024, "SIMT", 0),
    "gemm_tf32_4096": ("gemm", 4096, 4096, "TF32", 0),
    "gemm_tf32_8192": ("gemm", 8192, 8192, "TF32", 0),
    # OpAssign / Contiguous / Repeat / WIDE reductions, the calls `extra` times, twice each on 8192 x 8192 f32
    "elementwise_8192": ("elementwise", 8192, 8192, "f32", 2),
    # not for ncu: the chained list with the kernel's own %globaltimer stamps (a library built with
    # `python -m vortx_b200.build --timeline`); runs on 1 GPU or, under torchrun, on N
    "gemv_chain_timeline": ("chain_timeline", ROWS, COLS, "Q4_0", LAYERS),
    # the same stamps for single launches back to back (12 weight copies in one CUDA graph), one GPU
    "gemv_single_timeline_q4_0_8192x8192": ("single_timeline", 8192, 8192, "Q4_0", 12),
    "gemv_single_timeline_q8_0_4096x4096": ("single_timeline", 4096, 4096, "Q8_0", 24),
}


def run_chain_timeline():
    """Where a chained product's time goes, per thread block, from the list kernel's own %globaltimer stamps:
    the bench's chain (32 dependent 28672 x 8192 Q4_0 products, rows split over the ranks, x of a product = the
    rows every rank computed last in the one before), launched four times; the last launch is stamped."""
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist
    rank, n = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    if n > 1:
        dist.init_process_group("nccl", rank=rank, world_size=n, device_id=torch.device("cuda", local))
    import vortx_b200 as vb
    from vortx_b200 import _lib, synth
    from vortx_b200.multi_gpu import PeerBuffers
    lib = _lib.load()
    be = vb.Backend(local)
    shard, row0 = ROWS // n, rank * (ROWS // n)
    blocks = vb.quantize(vb.Q4_0, slab_matrix(shard, seed=100 + rank))
    layers = [vb.QuantizedMatrix(be, vb.Q4_0, blocks, shard, COLS) for _ in range(LAYERS)]
    x_dev = torch.from_numpy(synth.normal_vectors(1, COLS, seed=1)[0]).cuda()
    if n > 1:
        vecs = [PeerBuffers(be, lib.vx_xvec_bytes(ROWS)) for _ in range(2)]
        vec_ptrs = [v.ptrs for v in vecs]
    else:
        bufs = [torch.zeros(lib.vx_xvec_bytes(ROWS), device="cuda", dtype=torch.uint8) for _ in range(2)]
        vec_ptrs = [[b.data_ptr()] for b in bufs]
    others = [r for r in range(n) if r != rank]
    seg_len, seg_stride = COLS // n, ROWS // n
    entries = []
    for l in range(LAYERS):
        e = {"w": layers[l], "nrows": shard, "y_xvec": vec_ptrs[l % 2][rank],
             "peers": [vec_ptrs[l % 2][r] for r in others], "y_row0": row0, "y_stride": 1}
        if l == 0:
            e["x"] = x_dev.data_ptr()
        else:
            e["x_xvec"] = vec_ptrs[(l - 1) % 2][rank]
            e["x_seg_len"], e["x_seg_stride"], e["x_seg_first"] = seg_len, seg_stride, seg_stride - seg_len
        entries.append(e)
    chain = vb.GemvBatch(be, entries)
    sms = torch.cuda.get_device_properties(local).multi_processor_count
    stamps = torch.zeros(sms * LAYERS * 8, dtype=torch.int64, device="cuda")

    def sync():
        be.synchronize()
        if n > 1:
            dist.barrier()

    for it in range(4):
        sync()
        be.set_option("debug.timeline_ptr", stamps.data_ptr() if it == 3 else 0)
        chain.launch()
    sync()
    d = stamps.cpu().numpy().reshape(sms, LAYERS, 8).astype(np.float64)
    d = d[d[:, 1, 0] > 0]
    if d.shape[0] == 0:
        text = f"rank {rank}: no stamps — the library was not built with `python -m vortx_b200.build --timeline`"
    else:
        def stat(a):
            return f"{np.median(a) / 1e3:6.2f} (min {a.min() / 1e3:5.2f}, max {a.max() / 1e3:5.2f})"
        o = slice(4, LAYERS)
        begin, waited, conv, first, last, st_last = (d[:, o, i] for i in range(6))
        prev_last = d[:, 3:LAYERS - 1, 4]
        prev_store = d[:, 3:LAYERS - 1, 5].max(axis=0, keepdims=True)
        spread = d[:, o, 5].max(axis=0) - d[:, o, 5].min(axis=0)
        text = "\n".join([
            f"rank {rank} of {n}: {d.shape[0]} thread blocks, products 4..{LAYERS - 1}, per block, microseconds: median (min, max)",
            f"  product period (last tile to last tile)              {stat(last - prev_last)}",
            f"  last tile of product l-1 -> product l begins         {stat(begin - prev_last)}",
            f"  the block's wait for x (block-wait form only)        {stat(waited - begin)}",
            f"  x read (the threads' own waits included), converted  {stat(conv - waited)}",
            f"  this GPU's last store of l-1 -> x converted here     {stat(conv - prev_store)}",
            f"  first tile present after the conversion              {stat(first - conv)}",
            f"  first tile -> last tile computed                     {stat(last - first)}",
            f"  last tile computed -> its rows stored                {stat(st_last - last)}",
            f"  spread of the blocks' last stores of a product       {np.median(spread) / 1e3:6.2f} (max {spread.max() / 1e3:5.2f})"])
    if n > 1:
        gathered = [None] * n
        dist.all_gather_object(gathered, text)
        if rank == 0:
            print("\n".join(gathered), flush=True)
    else:
        print(text, flush=True)
    chain.free()
    sync()
    sys.stdout.flush()
    os._exit(0)   # past the final barrier with nothing in flight; no communicator teardown


def run_single_timeline(rows: int, cols: int, what: str, copies: int):
    """Where a single-launch GEMV's time goes: `copies` launches (one weight copy each) in one CUDA graph, every
    launch stamping its own buffer; times are relative to the last store of the launch before."""
    import torch
    import vortx_b200 as vb
    from vortx_b200 import _lib, synth
    lib = _lib.load()
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    be = vb.Backend(0, stream=stream.cuda_stream)
    qt = vb.Q4_0 if what == "Q4_0" else vb.Q8_0
    blocks = vb.quantize(qt, synth.normal_matrix(rows, cols, seed=0))
    ws = [vb.QuantizedMatrix(be, qt, blocks, rows, cols) for _ in range(copies)]
    x = torch.randn(1, cols, device="cuda")
    y = torch.empty(1, rows, device="cuda")
    max_blocks = 4 * torch.cuda.get_device_properties(0).multi_processor_count
    bufs = [torch.zeros(max_blocks * 8, dtype=torch.int64, device="cuda") for _ in range(copies)]
    for pdl in (1, 0):
        be.set_option("gemv.pdl", pdl)

        def fn():
            for i, w in enumerate(ws):
                be.set_option("debug.timeline_ptr", bufs[i].data_ptr())
                _lib.check(lib.vx_gemv_q_rows(be._ctx, w._h, 0, rows, x.data_ptr(), cols, y.data_ptr(), rows, 1))
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
        for _ in range(4):
            g.replay()
        torch.cuda.synchronize()
        for bf in bufs:
            bf.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        g.replay()
        b.record(stream)
        torch.cuda.synchronize()
        per = a.elapsed_time(b) * 1e3 / copies
        d = [bf.cpu().numpy().reshape(max_blocks, 8).astype(np.float64) for bf in bufs]
        d = [t[t[:, 7] > 0] for t in d]
        if d[0].shape[0] == 0:
            print("no stamps — the library was not built with `python -m vortx_b200.build --timeline`", flush=True)
            break
        table = []
        for l in range(3, copies - 1):
            end = d[l - 1][:, 5].max()
            t = d[l]
            table.append([np.median(t[:, 7]) - end, np.median(t[:, 0]) - end, np.median(t[:, 1]) - end, np.median(t[:, 2]) - end,
                          np.median(t[:, 3]) - end, np.median(t[:, 4]) - end, t[:, 5].min() - end, t[:, 5].max() - end])
        m = np.median(np.array(table), axis=0) / 1e3
        print(f"{what} {rows} x {cols}, programmatic dependent launch {'on' if pdl else 'off'}: {per:.2f} us per launch, "
              f"{d[4].shape[0]} thread blocks; microseconds after the last store of the launch before (median block, "
              f"median launch): block starts {m[0]:.2f}, past griddepcontrol.wait {m[1]:.2f}, first of x here {m[2]:.2f}, "
              f"x converted {m[3]:.2f}, first tile present {m[4]:.2f}, last tile computed {m[5]:.2f}, "
              f"first block's last store {m[6]:.2f}, last block's last store {m[7]:.2f}", flush=True)
    g = None
    for w in ws:
        w.free()
    be.synchronize()


def run_profile_case(name: str):
    """A handful of plain launches of one kernel on a small footprint, for `ncu` captures.
    Prints what it ran; nothing printed here is a benchmark value."""
    import ctypes as C
    import vortx_b200 as vb
    from vortx_b200 import _lib
    kind, rows, cols, what, copies = PROFILE_CASES[name]
    if kind == "chain_timeline":
        return run_chain_timeline()
    if kind == "single_timeline":
        return run_single_timeline(rows, cols, what, copies)
    be = vb.Backend(0)
    lib = _lib.load()
    rng = np.random.Generator(np.random.Philox(1))
    if kind == "elementwise":
        cases, keep = elementwise_cases(be, lib, rows)
        for _ in range(copies):
            for _name, _operands, call in cases:
                _lib.check(call())
        be.synchronize()
        emit({"profile_case": name, "kernels_launched": be.launch_count(), "order": [c[0] for c in cases]})
        del cases, keep
        be.close()
        return
    if kind == "gemv_batch":
        # `copies` is the batch here; four copies of the weights so that they come from HBM
        batch, copies = copies, 4
    if kind in ("gemv", "gemv_list", "gemv_batch"):
        qt = vb.Q4_0 if what == "Q4_0" else vb.Q8_0
        bb = lib.vx_qblock_bytes(qt)
        nblocks = rows * cols // 32
        # random quants with sane f16 scales: the kernel's work does not depend on the values
        blocks = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
        sc = (rng.random(nblocks, dtype=np.float32) * 0.01 + 0.001).astype(np.float16).view(np.uint16)
        blocks[:, 0] = sc & 0xFF
        blocks[:, 1] = sc >> 8
        ws = [vb.QuantizedMatrix(be, qt, blocks.ravel(), rows, cols) for _ in range(copies)]
        nvec = batch if kind == "gemv_batch" else 1
        x = be.init_buffer(rng.standard_normal(nvec * cols, dtype=np.float32))
        y = be.uninit_buffer(nvec * rows)
        if kind == "gemv_batch":
            for _ in range(3):
                for w in ws:
                    vb.Gemv().dispatch(be, None, y, w, x, batch=nvec)
        elif kind == "gemv_list":
            batch = vb.GemvBatch(be, [{"w": w, "x": x.ptr, "y": y.ptr} for w in ws])
            for _ in range(3):
                batch.launch()
        else:
            for _ in range(3):
                for w in ws:
                    vb.Gemv().dispatch(be, None, y, w, x)
    else:
        mode = _lib.VX_GEMM_SIMT_EXACT if what == "SIMT" else _lib.VX_GEMM_TF32
        a = be.init_buffer(rng.random(rows * cols, dtype=np.float32) * 2 - 1)
        b = be.init_buffer(rng.random(rows * cols, dtype=np.float32) * 2 - 1)
        c = be.uninit_buffer(rows * cols)
        sh = _lib.VxShapes3()
        for s in (sh.out, sh.lhs, sh.rhs):
            s.n = s.c = 1
            s.h = s.w = rows
            s.n_stride = s.c_stride = rows * cols
            s.h_stride, s.w_stride = cols, 1
        for _ in range(4):
            _lib.check(lib.vx_gemm_f32(be._ctx, mode, c.ptr, a.ptr, b.ptr, C.byref(sh), 0, 0, 0))
    be.synchronize()
    emit({"profile_case": name, "kernels_launched": be.launch_count()})
    be.close()


_REAL_STDOUT = None


def isolate_stdout():
    """Libraries (NCCL's version banner, for one) write to file descriptor 1.  Point it at stderr for the
    run and keep the original for the one JSON line."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


EXCHANGE_TEXT = {
    "peer": "chain of dependent GEMVs in one persistent launch per GPU: rows stored as {value, generation} pairs into "
            "every GPU's exchange vector from the kernel epilogue; the next GEMV's x is the END of every rank's slab "
            "in that vector (the rows computed last: it cannot start before the previous one is complete everywhere), "
            "awaited pair by pair",
    "peer-launches": "flagged pairs with one launch per GEMV and rows dealt out in turn; x is the vector's first 8192 "
                     "elements (rows computed early: a looser dependency than 'peer')",
    "separate": "N = 1 only: one launch per GEMV instead of the list launch",
    "peer-barrier": "peer stores from the kernel epilogue + a barrier kernel after every GEMV",
    "nccl": "NCCL all-gather after every GEMV",
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--exchange", choices=sorted(EXCHANGE_TEXT), default="peer",
                    help="N > 1: how the slabs of y reach every GPU")
    ap.add_argument("--profile-case", choices=sorted(PROFILE_CASES), default=None,
                    help="run a few launches of one kernel on a small footprint (for ncu) and exit")
    args = ap.parse_args()
    isolate_stdout()
    if args.profile_case:
        run_profile_case(args.profile_case)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
