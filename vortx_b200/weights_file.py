"""Packed-weight files: GGUF containers of GGML tensors (vx_wfile_* of the C ABI), and a writer for them.

vortx keeps GGML's dimension convention in its layout helpers (GGML_IDS, permute_ggml; src/shapes.rs:15-18,
:261-265): a GGML tensor lists its innermost dimension first, so a rows x cols weight matrix has ne = [cols, rows].
GGML's Q4_0 / Q8_0 blocks are byte for byte this library's host block stream, so a quantised matrix goes from
the mapped file to the device without a conversion pass.
"""
from __future__ import annotations

import ctypes as C
import struct
from typing import Dict, Iterable, List, Optional, Tuple

import numpy as np

from . import _lib

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q8_0 = 0, 1, 2, 8
_BLOCK = {GGML_F32: (4, 1), GGML_F16: (2, 1), GGML_Q4_0: (18, 32), GGML_Q8_0: (34, 32)}   # bytes, elements per block
QTYPE_OF_GGML = {GGML_Q4_0: _lib.VX_Q4_0, GGML_Q8_0: _lib.VX_Q8_0}
GGML_OF_QTYPE = {v: k for k, v in QTYPE_OF_GGML.items()}


class WeightFile:
    """A mapped GGUF file.  `tensors()` lists (name, ggml_type, ne, bytes); `load(backend, name)` uploads a
    Q4_0 / Q8_0 matrix as a QuantizedMatrix; `array(name)` views an F32 / F16 tensor, `raw(name)` any sized one."""

    def __init__(self, path: str):
        h = C.c_void_p()
        _lib.check(_lib.load().vx_wfile_open(str(path).encode(), C.byref(h)))
        self._h = h

    def close(self) -> None:
        if self._h:
            _lib.load().vx_wfile_close(self._h)
        self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __len__(self) -> int:
        n = C.c_size_t()
        _lib.check(_lib.load().vx_wfile_count(self._h, C.byref(n)))
        return int(n.value)

    def tensor(self, index: int) -> Tuple[str, int, Tuple[int, ...], int]:
        name = C.create_string_buffer(256)
        t, nd, b = C.c_uint32(), C.c_uint32(), C.c_uint64()
        ne = (C.c_uint64 * 4)()
        _lib.check(_lib.load().vx_wfile_tensor(self._h, index, name, 256, C.byref(t), C.byref(nd), ne, C.byref(b)))
        return name.value.decode(), int(t.value), tuple(int(v) for v in ne[:nd.value]), int(b.value)

    def tensors(self) -> List[Tuple[str, int, Tuple[int, ...], int]]:
        return [self.tensor(i) for i in range(len(self))]

    def index(self, name: str) -> int:
        i = C.c_size_t()
        _lib.check(_lib.load().vx_wfile_find(self._h, name.encode(), C.byref(i)))
        return int(i.value)

    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes, copied out of the mapping."""
        p, n = C.c_void_p(), C.c_uint64()
        _lib.check(_lib.load().vx_wfile_data(self._h, self.index(name), C.byref(p), C.byref(n)))
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(int(n.value),)).copy()

    def array(self, name: str) -> np.ndarray:
        _, t, ne, _ = self.tensor(self.index(name))
        if t not in (GGML_F32, GGML_F16):
            raise TypeError(f"'{name}' has GGML type {t}; array() reads F32 and F16")
        return self.raw(name).view(np.float32 if t == GGML_F32 else np.float16).reshape(tuple(reversed(ne)))

    def load(self, backend, name: str):
        """A Q4_0 / Q8_0 matrix as device weights: rows = ne[1], columns = ne[0]."""
        from .linalg import QuantizedMatrix
        i = self.index(name)
        _, t, ne, _ = self.tensor(i)
        h = C.c_void_p()
        _lib.check(_lib.load().vx_wfile_load_qweights(backend._ctx, self._h, i, C.byref(h)))
        qm = QuantizedMatrix.__new__(QuantizedMatrix)
        qm.backend, qm.qtype = backend, QTYPE_OF_GGML[t]
        qm.rows, qm.cols = (ne[1] if len(ne) > 1 else 1), ne[0]
        qm._h = h
        return qm


def _gguf_string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path: str, tensors: Iterable[Tuple[str, int, Tuple[int, ...], np.ndarray]],
               metadata: Optional[Dict[str, object]] = None, alignment: int = 32, version: int = 3) -> None:
    """Writes a GGUF file.  `tensors`: (name, ggml_type, ne, data) with `ne` innermost dimension first and `data`
    the tensor's bytes (a block stream for Q4_0 / Q8_0, as `quantize` returns it).  `metadata`: str, int (u32),
    float (f32) or list-of-str values."""
    tensors = list(tensors)
    md = dict(metadata or {})
    md.setdefault("general.alignment", alignment)
    out = bytearray(struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(md)))
    for k, v in md.items():
        out += _gguf_string(k)
        if isinstance(v, str):
            out += struct.pack("<I", 8) + _gguf_string(v)
        elif isinstance(v, bool):
            out += struct.pack("<IB", 7, int(v))
        elif isinstance(v, int):
            out += struct.pack("<II", 4, v)
        elif isinstance(v, float):
            out += struct.pack("<If", 6, v)
        elif isinstance(v, (list, tuple)):
            out += struct.pack("<IIQ", 9, 8, len(v))
            for e in v:
                out += _gguf_string(str(e))
        else:
            raise TypeError(f"metadata value of '{k}'")
    blobs, offset = [], 0
    for name, t, ne, data in tensors:
        raw = np.ascontiguousarray(data).view(np.uint8).ravel()
        bb, be = _BLOCK[t]
        count = int(np.prod(ne))
        if ne[0] % be or raw.size != count // be * bb:
            raise ValueError(f"'{name}': {raw.size} bytes do not hold ne = {ne} of GGML type {t}")
        out += _gguf_string(name) + struct.pack("<I", len(ne)) + struct.pack(f"<{len(ne)}Q", *ne)
        out += struct.pack("<IQ", t, offset)
        blobs.append((offset, raw))
        offset = (offset + raw.size + alignment - 1) // alignment * alignment
    out += b"\0" * ((-len(out)) % alignment)
    start = len(out)
    for off, raw in blobs:
        out += b"\0" * (start + off - len(out))
        out += raw.tobytes()
    with open(path, "wb") as f:
        f.write(out)
