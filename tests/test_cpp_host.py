"""The C++ host mirror (include/vortx_b200.hpp): compiled against the shared library with g++, its layout
checks run on the CPU, and on a GPU the whole program replays the reference's gpu_gemm_generic test and the
other operators through the C++ types."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def host_mirror_binary(tmp_path_factory):
    import vortx_b200
    vortx_b200.load()                                   # fails loudly if the library has not been built
    lib_dir = ROOT / "vortx_b200"
    out = tmp_path_factory.mktemp("cpp") / "host_mirror_test"
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", f"-I{ROOT / 'include'}",
           str(ROOT / "tests" / "cpp" / "host_mirror_test.cpp"), "-o", str(out),
           f"-L{lib_dir}", "-lvortx_b200", f"-Wl,-rpath,{lib_dir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def test_cpp_layout_algebra_on_cpu(host_mirror_binary):
    res = subprocess.run([str(host_mirror_binary), "layout"], capture_output=True, text=True, timeout=60)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout + res.stderr


@pytest.mark.gpu
def test_cpp_host_mirror_on_gpu(host_mirror_binary):
    res = subprocess.run([str(host_mirror_binary), "gpu"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout + res.stderr


@pytest.fixture(scope="module")
def group_binary(tmp_path_factory):
    import vortx_b200
    vortx_b200.load()
    lib_dir = ROOT / "vortx_b200"
    out = tmp_path_factory.mktemp("cpp") / "group_test"
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-Werror", f"-I{ROOT / 'include'}",
           str(ROOT / "tests" / "cpp" / "group_test.cpp"), "-o", str(out),
           f"-L{lib_dir}", "-lvortx_b200", f"-Wl,-rpath,{lib_dir}"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return out


def test_group_program_compiles(group_binary):
    """The torch-free multi-GPU driver builds against the C ABI alone (its runs need GPUs)."""
    assert group_binary.exists()


def _gpus():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_group_through_the_c_abi_without_torch(group_binary, tmp_path, world):
    """One process per GPU, nothing but the C ABI: group create over NCCL, all-gather, broadcast, the row-sharded
    GEMV and the column-sharded GEMM, each checked against the unsharded product."""
    import os
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    id_file = tmp_path / "nccl_id"
    procs = [subprocess.Popen([str(group_binary), str(world), str(r), str(id_file)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True, env=env) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()                       # the exact child started above
            out, _ = p.communicate()
            out += "\n(timed out)"
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and out.strip().endswith("ok"), f"rank {r}:\n{out}"
