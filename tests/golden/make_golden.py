"""Writes tests/golden/*.npz: small seeded inputs with the outputs of the CPU oracle.

The reference (dimforge/vortx v0.3.0) holds no golden vectors for GEMM and has no quantised
code, and it cannot be built or imported here (Rust, with its kernels compiled by rust-gpu), so
these fixtures pin the ORACLE: they freeze its outputs at the commit that wrote them, and the
tests check both the oracle (on CPU) and the CUDA path (on a GPU) against them.

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle as o  # noqa: E402
from vortx_b200 import synth  # noqa: E402

OUT = Path(__file__).resolve().parent


def gemm_case(m, k, n, seed):
    A = synth.uniform_matrix(m, k, seed)
    B = synth.uniform_matrix(k, n, seed + 1)
    out = np.zeros(m * n, np.float32)
    o.gemm_dispatch(out, A.ravel(), B.ravel(), o.shape_contiguous(1, 1, m, n), o.shape_contiguous(1, 1, m, k),
                    o.shape_contiguous(1, 1, k, n), 1)
    return {"A": A, "B": B, "C": out.reshape(m, n)}


def gemv_case(qt, rows, cols, batch, seed):
    w = synth.normal_matrix(rows, cols, seed)
    x = synth.normal_vectors(batch, cols, seed + 1)
    blocks = o.quantize(qt, w)
    y64, absdot = o.gemv_f64(qt, blocks, rows, cols, x)
    return {"w": w, "x": x, "blocks": blocks, "dequant": o.dequantize(qt, blocks, rows, cols),
            "y_f32": o.gemv(qt, blocks, rows, cols, x), "y_f64": y64, "absdot": absdot}


def main():
    np.savez_compressed(OUT / "gemm_f32.npz", **{f"{name}_{k}": v for name, case in {
        "m33k65n31": gemm_case(33, 65, 31, 10), "m64k16n64": gemm_case(64, 16, 64, 20),
        "m5k7n3": gemm_case(5, 7, 3, 30), "m130k40n70": gemm_case(130, 40, 70, 40)}.items() for k, v in case.items()})
    np.savez_compressed(OUT / "gemv_q8_0.npz", **{f"{name}_{k}": v for name, case in {
        "r17c96b1": gemv_case(o.Q8_0, 17, 96, 1, 50), "r64c256b4": gemv_case(o.Q8_0, 64, 256, 4, 60)}.items()
        for k, v in case.items()})
    np.savez_compressed(OUT / "gemv_q4_0.npz", **{f"{name}_{k}": v for name, case in {
        "r17c96b1": gemv_case(o.Q4_0, 17, 96, 1, 70), "r64c256b4": gemv_case(o.Q4_0, 64, 256, 4, 80)}.items()
        for k, v in case.items()})
    # f16 conversion table: every half value and its float
    halves = np.arange(65536, dtype=np.uint16)
    np.savez_compressed(OUT / "f16_table.npz", f32=halves.view(np.float16).astype(np.float32))
    print("wrote", sorted(p.name for p in OUT.glob("*.npz")))


if __name__ == "__main__":
    main()
