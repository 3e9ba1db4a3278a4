"""Builds libvortx_b200.so in-tree with nvcc for sm_100a.

    python -m vortx_b200.build [--force] [--verbose]

Every translation unit under csrc/ is compiled to an object next to it (build/) and
linked into vortx_b200/libvortx_b200.so.  Cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libvortx_b200.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--extended-lambda",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; libvortx_b200.so needs the CUDA toolkit to build")
    return exe


def _sources() -> list[Path]:
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp")))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, timeline: bool = False) -> Path:
    """Compiles what is out of date and links the library.  `timeline`: the list GEMV kernel with its
    %globaltimer stamps compiled in (-DVX_TIMELINE, for `bench.py --profile-case gemv_chain_timeline`); the next
    build without it compiles that file again, so the product never carries the stamps by accident."""
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    jobs = []
    for src in _sources():
        obj = OBJ / (src.stem + ".o")
        extra = ["-DVX_TIMELINE"] if timeline and src.name == "vx_gemv_stream.cu" else []
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-x", "cu", "-c", str(src), "-o", str(obj)]
        line = OBJ / (src.stem + ".cmd")            # the command the object was made with
        same_cmd = line.exists() and line.read_text() == " ".join(cmd)
        if force or not same_cmd or _stale(obj, [src, Path(__file__)] + headers):
            jobs.append((src, obj, cmd))

    def run(job):
        src, obj, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        (OBJ / (src.stem + ".log")).write_text(r.stdout + r.stderr)
        if r.returncode == 0:
            (OBJ / (src.stem + ".cmd")).write_text(" ".join(cmd))
        return src, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, r in ex.map(run, jobs):
            if verbose or r.returncode != 0:
                sys.stderr.write(f"--- {src.name}\n{r.stdout}{r.stderr}\n")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")

    objs = [OBJ / (s.stem + ".o") for s in _sources()]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-gencode",
               "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("linking libvortx_b200.so failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--timeline", action="store_true",
                    help="compile the list GEMV kernel with its %%globaltimer stamps (profiling builds only)")
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.timeline))
