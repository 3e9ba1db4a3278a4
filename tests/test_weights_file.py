"""Packed-weight files (GGUF containers of GGML tensors): the reader of the C ABI against files written here.

On the CPU: header, metadata of every value type, alignment, tensor records, the bytes of every tensor, and
the refusals.  On the GPU: a Q4_0 and a Q8_0 matrix loaded from a file give the very weights
vx_qweights_upload gives from the same block stream (dequantised planes and GEMV outputs bit-identical)."""
import struct

import numpy as np
import pytest

import vortx_b200 as vb
from vortx_b200 import _lib, synth
from vortx_b200.weights_file import GGML_F16, GGML_F32, GGML_Q4_0, GGML_Q8_0, WeightFile, write_gguf


def _model(tmp_path, alignment=32, version=3):
    rng = np.random.Generator(np.random.Philox(5))
    w4 = synth.normal_matrix(48, 256, seed=1)
    w8 = synth.normal_matrix(33, 512, seed=2)
    norm = rng.standard_normal(256).astype(np.float32)
    emb = rng.standard_normal((7, 64)).astype(np.float16)
    tensors = [("blk.0.ffn_up.weight", GGML_Q4_0, (256, 48), vb.quantize(vb.Q4_0, w4)),
               ("blk.0.attn_norm.weight", GGML_F32, (256,), norm),
               ("blk.0.ffn_down.weight", GGML_Q8_0, (512, 33), vb.quantize(vb.Q8_0, w8)),
               ("token_embd.weight", GGML_F16, (64, 7), emb)]
    path = tmp_path / "model.gguf"
    write_gguf(str(path), tensors, metadata={"general.architecture": "llama", "llama.block_count": 1,
                                             "llama.rope.freq_base": 10000.0, "tokenizer.ggml.tokens": ["a", "bc", "d"],
                                             "general.file_type": 2}, alignment=alignment, version=version)
    return path, tensors, (w4, w8, norm, emb)


@pytest.mark.parametrize("alignment,version", [(32, 3), (64, 2), (4096, 3)])
def test_reader_lists_and_returns_every_tensor(tmp_path, alignment, version):
    path, tensors, (w4, w8, norm, emb) = _model(tmp_path, alignment, version)
    with WeightFile(str(path)) as f:
        assert len(f) == 4
        listed = f.tensors()
        for (name, t, ne, data), got in zip(tensors, listed):
            assert got[0] == name and got[1] == t and got[2] == tuple(ne)
            raw = np.ascontiguousarray(data).view(np.uint8).ravel()
            assert got[3] == raw.size
            assert np.array_equal(f.raw(name), raw)
        assert np.array_equal(f.array("blk.0.attn_norm.weight"), norm)
        assert np.array_equal(f.array("token_embd.weight"), emb)          # ne = (64, 7): 7 rows of 64
        assert f.index("blk.0.ffn_down.weight") == 2
        with pytest.raises(_lib.VortxError):
            f.index("missing")
        # the blocks in the file are the library's own host block stream
        deq = vb.dequantize_host(vb.Q4_0, f.raw("blk.0.ffn_up.weight"), 48, 256)
        assert np.abs(deq - w4).max() <= np.abs(w4).max() / 7 * 0.51


def test_reader_refuses_what_it_cannot_read(tmp_path):
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(_lib.VortxError, match="GGUF"):
        WeightFile(str(bad))
    bad.write_bytes(struct.pack("<IIQQ", 0x46554747, 9, 0, 0))
    with pytest.raises(_lib.VortxError, match="version 9"):
        WeightFile(str(bad))
    with pytest.raises(_lib.VortxError, match="cannot open"):
        WeightFile(str(tmp_path / "nothing.gguf"))
    # a tensor record that points beyond the end of the file
    path, _, _ = _model(tmp_path)
    data = path.read_bytes()
    (tmp_path / "cut.gguf").write_bytes(data[:len(data) - 100])
    with pytest.raises(_lib.VortxError, match="does not lie inside"):
        WeightFile(str(tmp_path / "cut.gguf"))
    # a type this library cannot size is listed (bytes 0) but has no data view
    other = tmp_path / "other.gguf"
    hdr = bytearray(struct.pack("<IIQQ", 0x46554747, 3, 1, 0))
    name = b"x.weight"
    hdr += struct.pack("<Q", len(name)) + name + struct.pack("<IQQIQ", 2, 256, 4, 12, 0)     # GGML type 12
    hdr += b"\0" * ((-len(hdr)) % 32) + b"\0" * 1024
    other.write_bytes(bytes(hdr))
    with WeightFile(str(other)) as f:
        assert f.tensor(0) == ("x.weight", 12, (256, 4), 0)
        with pytest.raises(_lib.VortxError, match="cannot size"):
            f.raw("x.weight")


@pytest.mark.gpu
def test_matrices_loaded_from_a_file_equal_uploaded_ones(tmp_path, backend):
    path, tensors, _ = _model(tmp_path)
    with WeightFile(str(path)) as f:
        for name, qt, rows, cols in (("blk.0.ffn_up.weight", vb.Q4_0, 48, 256), ("blk.0.ffn_down.weight", vb.Q8_0, 33, 512)):
            from_file = f.load(backend, name)
            assert (from_file.rows, from_file.cols, from_file.qtype) == (rows, cols, qt)
            blocks = next(t[3] for t in tensors if t[0] == name)
            uploaded = vb.QuantizedMatrix(backend, qt, blocks, rows, cols)
            assert from_file.checksum() == uploaded.checksum()          # the same bytes on the device
            x = synth.normal_vectors(1, cols, seed=3)
            xd = backend.init_buffer(x.ravel())
            ys = []
            for qm in (from_file, uploaded):
                out = backend.uninit_buffer(rows * cols)
                qm.dequantize(out)
                deq = np.empty(rows * cols, np.float32)
                backend.slow_read_buffer(out, deq)
                yd = backend.init_buffer(np.full(rows, np.nan, np.float32))
                vb.Gemv().dispatch(backend, None, yd, qm, xd)
                y = np.empty(rows, np.float32)
                backend.slow_read_buffer(yd, y)
                ys.append((deq, y))
            assert np.array_equal(ys[0][0].view(np.uint32), ys[1][0].view(np.uint32))
            assert np.array_equal(ys[0][1].view(np.uint32), ys[1][1].view(np.uint32))
            from_file.free()
            uploaded.free()
        with pytest.raises(_lib.VortxError) as e:
            f.load(backend, "blk.0.attn_norm.weight")
        assert e.value.status == _lib.VX_ERR_UNSUPPORTED


@pytest.mark.gpu
def test_checksum_matches_the_same_fold_on_the_host(backend):
    """vx_checksum_u32: XOR of all 32-bit words, word j of every 16-byte group rotated left by 8 j bits."""
    import ctypes as C
    lib = _lib.load()
    rng = np.random.Generator(np.random.Philox(9))
    for n16 in (1, 7, 1000, 70001):
        host = rng.integers(0, 2 ** 32, size=4 * n16, dtype=np.uint64).astype(np.uint32)
        w = host.reshape(n16, 4)
        rot = lambda v, r: ((v << np.uint32(r)) | (v >> np.uint32(32 - r))) if r else v
        want = np.bitwise_xor.reduce(w[:, 0] ^ rot(w[:, 1], 8) ^ rot(w[:, 2], 16) ^ rot(w[:, 3], 24))
        d = backend.init_buffer(host)
        out = backend.init_buffer(np.zeros(1, np.uint32))
        _lib.check(lib.vx_checksum_u32(backend._ctx, d.ptr, host.nbytes, out.ptr))
        got = np.zeros(1, np.uint32)
        backend.slow_read_buffer(out, got)
        assert int(got[0]) == int(want), n16
    assert lib.vx_checksum_u32(backend._ctx, d.ptr, 24, out.ptr) == _lib.VX_ERR_INVALID_ARGUMENT
