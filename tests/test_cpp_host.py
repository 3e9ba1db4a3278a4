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
