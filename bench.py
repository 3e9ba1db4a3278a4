#!/usr/bin/env python
"""Benchmark of the block-quantised GEMV hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("q4_0_gemv_28672x8192_x32"): the Q4_0 GEMV y = W x with W 28672 x 8192 (the FFN
up-projection shape of the multi-GPU configuration), x f32 of length 8192, W ~ N(0, 0.02)
before quantisation, x ~ N(0, 1), all seeded and synthetic.  One STEP is a pass over 32
such matrices held at 32 different addresses (4.2 GB of weights at N = 1, far beyond the
126 MB L2), i.e. 32 dependent GEMV launches replayed from one CUDA graph.  With N > 1 the rows
of every matrix are split into N contiguous slabs (strong scaling: total work fixed), each
rank computes its slab straight into its slice of y and the slices are all-gathered with NCCL.

The line printed by rank 0:
  value      algorithmic bytes per step / device time per step, weights resident in HBM
             (bytes per GEMV = 132 120 576 of blocks + 32 768 n of x + 114 688 of y)
  e2e        the same through the public API with host buffers: per GEMV the activation is
             copied from pinned host memory, the product is read back to the host
  roofline   the streaming GEMV kernel against the measured HBM copy bandwidth
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


def make_weights(rows: int, cols: int, seed: int) -> np.ndarray:
    """One Q4_0 block stream for a rows x cols matrix ~ N(0, 0.02), quantised by the library's host quantiser."""
    import vortx_b200 as vb
    from vortx_b200 import synth
    return vb.quantize(vb.Q4_0, synth.normal_matrix(rows, cols, seed))


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
    built here, so this arm times the CPU oracle's GEMV, the stand-in the parity tests use."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    blocks = make_weights(ROWS, COLS, seed=100)
    gbs, dt, threads = cpu_gemv_rate(blocks, ROWS, args.steps, args.warmup)
    sample = (f"each step is {CPU_GEMVS_PER_STEP} of the workload's {LAYERS} GEMVs ({ROWS} x {COLS} Q4_0), "
              f"{threads} host threads; C++ restatement of the GEMV, not khal")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "q4_0 x f32 -> f32", "data": "synthetic",
        "config": {"workload": "q4_0_gemv_28672x8192_x32", "rows": ROWS, "cols": COLS, "batch": 1,
                   "sampled": sample},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------ GPU arm ----

def run_ours(args):
    import torch
    import torch.distributed as dist
    import vortx_b200 as vb
    from vortx_b200 import _lib, synth

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
    assert ROWS % n == 0
    shard = ROWS // n
    row0 = rank * shard

    # One quantised shard, uploaded LAYERS times to distinct addresses (identical bytes are still
    # distinct cache lines, and the step walks all of them before coming back).
    blocks = make_weights(shard, COLS, seed=100 + rank)
    layers = [vb.QuantizedMatrix(be, vb.Q4_0, blocks, shard, COLS) for _ in range(LAYERS)]
    x_host = synth.normal_vectors(1, COLS, seed=1)[0]
    x_dev = torch.from_numpy(x_host).to(dev)
    y_full = torch.zeros(LAYERS, ROWS, device=dev, dtype=torch.float32)  # one y per layer

    # N > 1: how the rows of y reach every GPU.
    #   "peer" (default): the step is a CHAIN in one persistent launch per GPU.  Each rank owns a contiguous slab
    #       of rows; the GEMV's epilogue stores each row as a {value, generation} pair into an exchange vector on
    #       every GPU over NVLink (a tile's rows leave as one contiguous store), and the next GEMV takes its x from
    #       the END of every rank's slab in that vector (COLS / N elements each: the rows every rank computes last,
    #       so the GEMV cannot start before the previous one is complete on every GPU), re-reading pairs that have
    #       not arrived yet while its weights already stream.  GEMV 0 of a step reads the plain x;
    #       the step ends by unpacking the last vector to plain f32.
    #   "peer-launches": the same dependency with one launch per GEMV and rows dealt out in turn.
    #   "peer-barrier": plain peer stores from the epilogue + a one-warp barrier kernel after every GEMV.
    #   "nccl": all-gather after every GEMV.
    scatter = chain = None
    if n > 1:
        from vortx_b200.multi_gpu import PeerScatterGemv
        scatter = PeerScatterGemv(be, ROWS, COLS, LAYERS, vectors=0)
        chain = PeerScatterGemv(be, ROWS, COLS, 1, vectors=2, cyclic=True)      # "peer-launches": rows dealt out in turn
        chain_w = PeerScatterGemv(be, ROWS, COLS, 1, vectors=2)                  # "peer": contiguous slabs, windowed x

    def gemv(layer: int, xptr: int):
        yptr = y_full[layer].data_ptr() + row0 * 4
        st = lib.vx_gemv_q_rows(be._ctx, layers[layer]._h, 0, shard, xptr, COLS, yptr, shard, 1)
        if st != 0:
            raise RuntimeError(_lib.last_error())

    # The step's 32 products as ONE persistent launch (a GEMV list): plain and independent at N = 1 and for
    # the kernel-only figure; chained through the exchange vectors for "peer".
    plain_batch = vb.GemvBatch(be, [{"w": layers[l], "x": x_dev.data_ptr(), "y": y_full[l].data_ptr() + row0 * 4}
                                    for l in range(LAYERS)])
    if os.environ.get("VX_GEMV_BLOCK_WAIT"):     # 0 / 1 overrides the library's choice of how blocks wait for x
        be.set_option("gemv.block_wait", int(os.environ["VX_GEMV_BLOCK_WAIT"]))
    chain_batch = chain_w.chain_batch(layers, x_dev.data_ptr(), window=True) if n > 1 else None

    def step_device(exchange=args.exchange):
        if n == 1 and exchange != "separate":
            plain_batch.launch()
            return
        if n > 1 and exchange == "peer":
            chain_batch.launch()
            chain_w.unpack((LAYERS - 1) % 2, chain_w.y_ptr(0))
            return
        if n > 1 and exchange == "peer-launches":      # the same chain, one launch per GEMV
            chain.dispatch_chained(layers[0], 0, x_ptr=x_dev.data_ptr())
            for l in range(1, LAYERS):
                chain.dispatch_chained(layers[l], l % 2, x_vec=(l - 1) % 2)
            chain.unpack((LAYERS - 1) % 2, chain.y_ptr(0))
            return
        for l in range(LAYERS):
            if n > 1 and exchange == "peer-barrier":
                scatter.dispatch(layers[l], x_dev.data_ptr(), l)
            else:
                gemv(l, x_dev.data_ptr())
                if n > 1 and exchange == "nccl":
                    dist.all_gather_into_tensor(y_full[l], y_full[l, row0:row0 + shard])

    note("weights uploaded")
    # Warm-up outside the graph (also sizes NCCL's buffers), then capture one step.
    launches_before = be.launch_count()
    step_device()
    launches_per_step = be.launch_count() - launches_before
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        step_device()
    torch.cuda.synchronize()

    note("step captured")
    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        graph.replay()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        graph.replay()
    e1.record(stream)
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    bytes_per_step = LAYERS * gemv_bytes(ROWS, COLS, n)
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9

    note("timed region done")
    # Kernel-only figure for the roofline: the step's products on this GPU's rows without any exchange
    # (N = 1: the step itself), timed live with CUDA events on the launching stream.  The dominant kernel is
    # the list launch: LAYERS products per launch.
    def time_graph(fn, reps):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
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
    separate_us = time_graph(lambda: [gemv(l, x_dev.data_ptr()) for l in range(LAYERS)], reps) / LAYERS
    shard_bytes = gemv_bytes(shard, COLS)
    list_bytes = LAYERS * shard_bytes
    peak, peak_kind = measured_peak_hbm()
    achieved = list_bytes / (launch_us * 1e-6) / 1e9

    note("kernel-only timing done")
    # End to end through the public API with host buffers: the step's 32 x vectors go up from pinned host
    # memory in one copy, the step runs (each product reads its own x), and the 32 y vectors come back in one
    # copy.  N > 1: every rank uploads x and reads back the whole y of every product, gathered on the device
    # (one list launch whose epilogue stores the rows on every GPU + one barrier kernel; or NCCL).
    xs_pin = torch.from_numpy(np.tile(x_host, (LAYERS, 1))).pin_memory()
    ys_pin = torch.empty(LAYERS, ROWS, dtype=torch.float32).pin_memory()
    xs_dev = torch.empty(LAYERS, COLS, device=dev, dtype=torch.float32)
    e2e_batch = vb.GemvBatch(be, [{"w": layers[l], "x": xs_dev[l].data_ptr(), "y": y_full[l].data_ptr() + row0 * 4}
                                  for l in range(LAYERS)])

    e2e_scatter = scatter.scatter_batch(layers, [xs_dev[l].data_ptr() for l in range(LAYERS)]) if n > 1 else None

    def step_e2e():
        _lib.check(lib.vx_upload(be._ctx, xs_dev.data_ptr(), xs_pin.data_ptr(), LAYERS * COLS * 4))
        if n == 1:
            e2e_batch.launch()
            src = y_full.data_ptr()
        elif args.exchange.startswith("peer"):
            e2e_scatter.launch()      # rows of all 32 products stored here and on every peer ...
            scatter.finish()          # ... and one arrival barrier for the step
            src = scatter.y_ptr(0)
        else:
            e2e_batch.launch()
            for l in range(LAYERS):
                dist.all_gather_into_tensor(y_full[l], y_full[l, row0:row0 + shard])
            src = y_full.data_ptr()
        _lib.check(lib.vx_download(be._ctx, ys_pin.data_ptr(), src, LAYERS * ROWS * 4))

    for _ in range(2):
        step_e2e()
    barrier()
    e2e_steps = max(2, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    if n > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    e2e_value = bytes_per_step / (e2e_ms * 1e-3) / 1e9

    note("end-to-end timing done")
    extra = {}
    if n > 1:
        # the other ways of exchanging y, timed the same way, for comparison
        for other in ("peer", "peer-launches", "peer-barrier", "nccl"):
            if other == args.exchange:
                continue
            step_device(other)
            torch.cuda.synchronize()
            og = torch.cuda.CUDAGraph()
            with torch.cuda.graph(og, stream=stream):
                step_device(other)
            for _ in range(3):
                og.replay()
            barrier()
            o0, o1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            o0.record(stream)
            for _ in range(args.steps):
                og.replay()
            o1.record(stream)
            barrier()
            t = torch.tensor([o0.elapsed_time(o1)], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            other_ms = float(t.item()) / args.steps
            extra[f"exchange_{other}"] = {"ms_per_step": other_ms, "GB/s": bytes_per_step / (other_ms * 1e-3) / 1e9}
        extra["kernels_only"] = {"us_per_list_launch": launch_us, "GB/s_per_gpu": achieved}
        note("exchange variants timed")
        # (the headline numbers above must not be lost to a failure in this side measurement: every rank
        # runs the same code, so a library error raises on all of them alike)
        try:
            extra["gemm_tf32_8192_col_sharded"] = sharded_gemm_numbers(be, torch, dist, stream, n, rank, barrier)
        except _lib.VortxError as e:
            extra["gemm_tf32_8192_col_sharded"] = {"failed": str(e)}
    cpu = None
    if rank == 0 and n == 1:
        try:
            extra = side_configs(be, lib, torch, stream)
        except _lib.VortxError as e:
            extra = {"side_configs_failed": str(e)}
        try:
            gbs, dt, threads = cpu_gemv_rate(blocks, ROWS, steps=5, warmup=1)
            cpu = {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
                   "sample": f"5 x {CPU_GEMVS_PER_STEP} GEMVs of {ROWS} x {COLS} Q4_0 (the step has {LAYERS}); "
                             "C++ restatement of the GEMV, not khal"}
        except Exception as e:  # the oracle is test infrastructure; its absence must not hide the GPU numbers
            cpu = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"unavailable: {e}"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "q4_0 x f32 (24-bit fixed point) -> f32",
            "data": "synthetic",
            "config": {"workload": "q4_0_gemv_28672x8192_x32", "rows": ROWS, "cols": COLS, "batch": 1,
                       "gemv_per_step": LAYERS,
                       "sharding": (f"rows/{n} per GPU; y exchanged by " + EXCHANGE_TEXT[args.exchange]) if n > 1 else "none",
                       "l2": "inputs larger than L2: 32 weight copies walked in turn",
                       "launch": "CUDA graph replay; the 32 products of a step are one persistent list launch"},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": LAYERS * COLS * 4, "d2h_bytes_per_step": LAYERS * ROWS * 4},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"{peak_kind} HBM copy bandwidth", "datasheet_peak": 8000.0,
                         "frac_datasheet": achieved / 8000.0, "kernel": "gemv_stream_kernel",
                         "bytes_per_launch": list_bytes, "us_per_launch": launch_us, "gemvs_per_launch": LAYERS,
                         "one_gemv_per_launch": {"us_per_launch": separate_us, "bytes_per_launch": shard_bytes,
                                                 "achieved": shard_bytes / (separate_us * 1e-6) / 1e9},
                         "traffic": LAYERS * 135_400_000 if n == 1 else None,
                         "traffic_source": "ncu dram__bytes_read + write of one 28672 x 8192 product (135.4 MB, profiles/gemv_stream_q4_0_28672x8192.md) x the 32 products of the list launch"},
            "clocks": clocks,
            "extra": extra,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        emit(line)
    if n > 1:
        # NCCL's communicator teardown was seen to hang on this pool's boxes after all work had
        # completed; every rank has synchronised and rank 0 has printed, so leave without it.
        barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


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
    return out


PROFILE_CASES = {
    # name: (kind, rows/dim, cols, qtype name, weight copies)
    "gemv_q4_0_28672x8192": ("gemv", 28672, 8192, "Q4_0", 2),
    "gemv_q4_0_8192x8192": ("gemv", 8192, 8192, "Q4_0", 4),
    "gemv_list_q4_0_28672x8192_x8": ("gemv_list", 28672, 8192, "Q4_0", 8),   # one list launch over 8 weight copies
    "gemv_q8_0_4096x4096": ("gemv", 4096, 4096, "Q8_0", 8),
    "gemm_simt_exact_1024": ("gemm", 1024, 1024, "SIMT", 0),
    "gemm_tf32_4096": ("gemm", 4096, 4096, "TF32", 0),
    "gemm_tf32_8192": ("gemm", 8192, 8192, "TF32", 0),
}


def run_profile_case(name: str):
    """A handful of plain launches of one kernel on a small footprint, for `ncu` captures.
    Prints what it ran; nothing printed here is a benchmark value."""
    import ctypes as C
    import vortx_b200 as vb
    from vortx_b200 import _lib
    kind, rows, cols, what, copies = PROFILE_CASES[name]
    be = vb.Backend(0)
    lib = _lib.load()
    rng = np.random.Generator(np.random.Philox(1))
    if kind in ("gemv", "gemv_list"):
        qt = vb.Q4_0 if what == "Q4_0" else vb.Q8_0
        bb = lib.vx_qblock_bytes(qt)
        nblocks = rows * cols // 32
        # random quants with sane f16 scales: the kernel's work does not depend on the values
        blocks = rng.integers(0, 256, size=(nblocks, bb), dtype=np.uint8)
        sc = (rng.random(nblocks, dtype=np.float32) * 0.01 + 0.001).astype(np.float16).view(np.uint16)
        blocks[:, 0] = sc & 0xFF
        blocks[:, 1] = sc >> 8
        ws = [vb.QuantizedMatrix(be, qt, blocks.ravel(), rows, cols) for _ in range(copies)]
        x = be.init_buffer(rng.standard_normal(cols, dtype=np.float32))
        y = be.uninit_buffer(rows)
        if kind == "gemv_list":
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
