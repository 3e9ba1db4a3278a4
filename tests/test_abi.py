"""The C ABI without a GPU: the shared library loads, exports every symbol the headers declare,
and its host-only entry points (errors, quantisers, layouts) behave."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    names = set()
    for h in (ROOT / "include").glob("*.h"):
        names |= set(re.findall(r"VX_API\s+[\w\s\*]+?\b(vx_\w+)\s*\(", h.read_text()))
    return names


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _declared()
    assert len(declared) >= 50
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    # and the Python binding types exactly that set
    assert declared == set(_lib.SIGNATURES), (declared ^ set(_lib.SIGNATURES))


def test_struct_layouts_match_the_reference_abi():
    # vortx-shaders/src/linalg/shape.rs:9-29: 8 x u32 = 32 bytes; Shapes3 = 96 bytes
    assert C.sizeof(_lib.VxShape) == 32 and C.sizeof(_lib.VxShapes3) == 96
    assert [f for f, _ in _lib.VxShape._fields_] == ["n", "c", "h", "w", "n_stride", "c_stride", "h_stride", "w_stride"]
    assert C.sizeof(_lib.VxLayout) == 40


def test_no_device_is_reported_not_hidden():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(vb.VortxError) as e:
        vb.Backend(0)
    assert e.value.status == _lib.VX_ERR_NO_DEVICE


def test_error_paths_and_messages():
    lib = _lib.load()
    assert lib.vx_version().startswith(b"vortx_b200")
    assert lib.vx_synchronize(None) == _lib.VX_ERR_INVALID_ARGUMENT
    assert b"null context" in lib.vx_last_error()
    assert lib.vx_qblock_bytes(_lib.VX_Q8_0) == 34 and lib.vx_qblock_bytes(_lib.VX_Q4_0) == 18
    assert lib.vx_qblock_bytes(7) == 0
    w = np.zeros((2, 48), np.float32)
    out = np.zeros(64, np.uint8)
    st = lib.vx_quantize(_lib.VX_Q4_0, w.ctypes.data, 2, 48, out.ctypes.data)
    assert st == _lib.VX_ERR_INVALID_ARGUMENT and b"multiple of 32" in lib.vx_last_error()
    assert lib.vx_quantize(5, w.ctypes.data, 2, 64, out.ctypes.data) == _lib.VX_ERR_INVALID_ARGUMENT
    assert lib.vx_gemm_f32(None, 0, None, None, None, None, 0, 0, 0) == _lib.VX_ERR_INVALID_ARGUMENT
    assert lib.vx_free(None, None) == _lib.VX_ERR_INVALID_ARGUMENT
    assert lib.vx_gemv_batch_run_host(None, None, 1) == _lib.VX_ERR_INVALID_ARGUMENT
    assert lib.vx_context_destroy(None) == _lib.VX_OK


def test_host_quantise_round_trip():
    rng = np.random.Generator(np.random.Philox(0))
    w = (rng.standard_normal((8, 128)) * 0.02).astype(np.float32)
    for qt, levels in ((vb.Q8_0, 127), (vb.Q4_0, 7)):
        blocks = vb.quantize(qt, w)
        deq = vb.dequantize_host(qt, blocks, 8, 128)
        step = np.abs(w).reshape(8, 4, 32).max(axis=2, keepdims=True) / levels
        assert (np.abs(deq - w).reshape(8, 4, 32) <= 0.501 * step + 1e-9).all()


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libvortx_b200.so")
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()
