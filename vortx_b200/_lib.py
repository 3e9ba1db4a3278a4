"""ctypes binding of libvortx_b200.so (the C ABI declared in include/vortx_b200*.h).

The library is the product; there is no Python or CPU fallback.  If the shared object is
missing, `load()` raises with the build command instead of degrading.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libvortx_b200.so"

VX_OK = 0
VX_ERR_INVALID_ARGUMENT = 1
VX_ERR_SHAPE = 2
VX_ERR_OUT_OF_BOUNDS = 3
VX_ERR_CUDA = 4
VX_ERR_OUT_OF_MEMORY = 5
VX_ERR_UNSUPPORTED = 6
VX_ERR_DEVICE_TIMEOUT = 7
VX_ERR_NO_DEVICE = 8
VX_ERR_COLLECTIVE = 9

VX_GEMM_AUTO, VX_GEMM_NAIVE, VX_GEMM_SIMT_EXACT, VX_GEMM_TF32 = 0, 1, 2, 3
VX_DISPATCH, VX_DISPATCH_NAIVE, VX_DISPATCH_TILED, VX_DISPATCH_TF32 = 0, 1, 2, 3
VX_Q8_0, VX_Q4_0 = 0, 1


class VxShape(C.Structure):
    """vortx-shaders/src/linalg/shape.rs:9-29."""

    _fields_ = [(n, C.c_uint32) for n in
                ("n", "c", "h", "w", "n_stride", "c_stride", "h_stride", "w_stride")]

    def astuple(self):
        return tuple(getattr(self, f) for f, _ in self._fields_)


class VxShapes3(C.Structure):
    _fields_ = [("out", VxShape), ("lhs", VxShape), ("rhs", VxShape)]


class VxLayout(C.Structure):
    """src/shapes.rs:49-60."""

    _fields_ = [("size", C.c_uint32 * 4), ("stride", C.c_uint32 * 4),
                ("rank", C.c_uint32), ("offset", C.c_uint32)]


class VxGemvOp(C.Structure):
    """vx_gemv_op: one entry of a GEMV list."""

    _fields_ = [("w", C.c_void_p), ("row0", C.c_size_t), ("nrows", C.c_size_t), ("x_xvec", C.c_void_p),
                ("x", C.c_void_p), ("y", C.c_void_p), ("y_xvec", C.c_void_p), ("peer_y_xvec", C.POINTER(C.c_void_p)),
                ("n_peers", C.c_size_t), ("y_row0", C.c_size_t), ("y_stride", C.c_size_t),
                ("peer_y", C.POINTER(C.c_void_p)), ("n_peer_y", C.c_size_t),
                ("x_seg_len", C.c_size_t), ("x_seg_stride", C.c_size_t), ("x_seg_first", C.c_size_t)]


class VxHostStage(C.Structure):
    """vx_host_stage: one stage of vx_gemv_batch_run_host."""

    _fields_ = [("batch", C.c_void_p), ("up_device", C.c_void_p), ("up_host", C.c_void_p), ("up_bytes", C.c_size_t),
                ("down_host", C.c_void_p), ("down_host_pitch", C.c_size_t), ("down_device", C.c_void_p),
                ("down_device_pitch", C.c_size_t), ("down_width_bytes", C.c_size_t), ("down_rows", C.c_size_t),
                ("barrier_flags", C.POINTER(C.c_void_p)), ("world", C.c_size_t), ("rank", C.c_size_t)]


class VortxError(RuntimeError):
    """A non-zero vx_status; `.status` holds the code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"vortx_b200 status {status}: {message}")
        self.status = status
        self.message = message


class ShapeMismatch(VortxError, AssertionError):
    """VX_ERR_SHAPE — where the reference's assert_eq! would panic (src/linalg/gemm.rs:70-104)."""


class LayoutError(VortxError, ValueError):
    """VX_ERR_INVALID_ARGUMENT from the layout algebra — where the reference panics."""


_P = C.c_void_p
_LP = C.POINTER(VxLayout)
_U32P = C.POINTER(C.c_uint32)

# name -> (restype, argtypes).  Everything declared in include/vortx_b200.h and
# include/vortx_b200_host.h is listed here; tests check the two stay in step.
SIGNATURES = {
    "vx_last_error": (C.c_char_p, []),
    "vx_version": (C.c_char_p, []),
    "vx_context_create": (C.c_int32, [C.c_int32, C.POINTER(_P)]),
    "vx_context_create_on_stream": (C.c_int32, [C.c_int32, _P, C.POINTER(_P)]),
    "vx_context_destroy": (C.c_int32, [_P]),
    "vx_synchronize": (C.c_int32, [_P]),
    "vx_context_device": (C.c_int32, [_P, C.POINTER(C.c_int32)]),
    "vx_context_stream": (C.c_int32, [_P, C.POINTER(_P)]),
    "vx_context_launch_count": (C.c_int32, [_P, C.POINTER(C.c_uint64)]),
    "vx_alloc": (C.c_int32, [_P, C.c_size_t, C.POINTER(_P)]),
    "vx_free": (C.c_int32, [_P, _P]),
    "vx_upload": (C.c_int32, [_P, _P, _P, C.c_size_t]),
    "vx_download": (C.c_int32, [_P, _P, _P, C.c_size_t]),
    "vx_copy": (C.c_int32, [_P, _P, _P, C.c_size_t]),
    "vx_memset": (C.c_int32, [_P, _P, C.c_int, C.c_size_t]),
    "vx_host_alloc": (C.c_int32, [C.c_size_t, C.POINTER(_P)]),
    "vx_host_free": (C.c_int32, [_P]),
    "vx_gemm_f32": (C.c_int32, [_P, C.c_int, _P, _P, _P, C.POINTER(VxShapes3),
                                C.c_uint64, C.c_uint64, C.c_uint64]),
    "vx_gemm_last_kernel": (C.c_int32, [_P, C.POINTER(C.c_int32)]),
    "vx_qblock_bytes": (C.c_size_t, [C.c_int]),
    "vx_quantize": (C.c_int32, [C.c_int, _P, C.c_size_t, C.c_size_t, _P]),
    "vx_dequantize_host": (C.c_int32, [C.c_int, _P, C.c_size_t, C.c_size_t, _P]),
    "vx_qweights_upload": (C.c_int32, [_P, C.c_int, _P, C.c_size_t, C.c_size_t, C.POINTER(_P)]),
    "vx_qweights_from_device": (C.c_int32, [_P, C.c_int, _P, C.c_size_t, C.c_size_t, C.c_size_t, C.POINTER(_P)]),
    "vx_qweights_free": (C.c_int32, [_P, _P]),
    "vx_qweights_info": (C.c_int32, [_P, C.POINTER(C.c_int32), C.POINTER(C.c_size_t),
                                     C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "vx_dequantize": (C.c_int32, [_P, _P, _P]),
    "vx_gemv_q": (C.c_int32, [_P, _P, _P, C.c_size_t, _P, C.c_size_t, C.c_size_t]),
    "vx_gemv_q_rows": (C.c_int32, [_P, _P, C.c_size_t, C.c_size_t, _P, C.c_size_t, _P,
                                   C.c_size_t, C.c_size_t]),
    "vx_gemv_q_multi": (C.c_int32, [_P, C.POINTER(_P), C.c_size_t, _P, C.c_size_t, C.POINTER(_P), C.c_size_t, C.c_size_t]),
    "vx_ipc_export": (C.c_int32, [_P, _P, _P]),
    "vx_ipc_import": (C.c_int32, [_P, _P, C.POINTER(_P)]),
    "vx_ipc_release": (C.c_int32, [_P, _P]),
    "vx_gemv_q_rows_scatter": (C.c_int32, [_P, _P, C.c_size_t, C.c_size_t, _P, _P, C.POINTER(_P), C.c_size_t]),
    "vx_xvec_bytes": (C.c_size_t, [C.c_size_t]),
    "vx_gemv_q_rows_exchange": (C.c_int32, [_P, _P, C.c_size_t, C.c_size_t, _P, _P, _P, _P, C.POINTER(_P),
                                            C.c_size_t, C.c_size_t, C.c_size_t]),
    "vx_xvec_unpack": (C.c_int32, [_P, _P, C.c_size_t, _P]),
    "vx_gemv_batch_create": (C.c_int32, [_P, _P, C.c_size_t, C.POINTER(_P)]),
    "vx_gemv_batch_launch": (C.c_int32, [_P, _P]),
    "vx_gemv_batch_free": (C.c_int32, [_P, _P]),
    "vx_gemv_batch_run_host": (C.c_int32, [_P, _P, C.c_size_t]),
    "vx_host_pipeline_create": (C.c_int32, [_P, _P, C.c_size_t, C.POINTER(_P)]),
    "vx_host_pipeline_run": (C.c_int32, [_P]),
    "vx_host_pipeline_free": (C.c_int32, [_P]),
    "vx_gemm_tf32_scatter": (C.c_int32, [_P, _P, _P, _P, C.POINTER(VxShapes3), C.POINTER(_P), C.c_size_t]),
    "vx_peer_barrier": (C.c_int32, [_P, C.POINTER(_P), C.c_size_t, C.c_size_t]),
    "vx_group_unique_id": (C.c_int32, [_P]),
    "vx_group_create": (C.c_int32, [_P, C.c_size_t, C.c_size_t, _P, C.POINTER(_P)]),
    "vx_group_destroy": (C.c_int32, [_P]),
    "vx_group_info": (C.c_int32, [_P, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "vx_group_all_gather": (C.c_int32, [_P, _P, _P, C.c_size_t]),
    "vx_group_broadcast": (C.c_int32, [_P, _P, C.c_size_t, C.c_size_t]),
    "vx_group_barrier": (C.c_int32, [_P]),
    "vx_group_peer_alloc": (C.c_int32, [_P, C.c_size_t, C.POINTER(_P)]),
    "vx_group_peer_free": (C.c_int32, [_P, C.POINTER(_P)]),
    "vx_group_gemv_q": (C.c_int32, [_P, _P, C.c_size_t, _P, C.POINTER(_P), C.c_size_t]),
    "vx_group_gemm_tf32": (C.c_int32, [_P, _P, _P, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                       C.c_size_t, C.POINTER(_P)]),
    "vx_reduce": (C.c_int32, [_P, C.c_int, C.c_int, C.c_int, _P, C.POINTER(VxShape), C.c_uint64, _P]),
    "vx_reduce_static": (C.c_int32, [C.c_int32, _P, C.c_int, C.c_int, _P, C.POINTER(VxShape), _P]),
    "vx_op_assign": (C.c_int32, [_P, C.c_int, _P, C.POINTER(VxShape), C.c_uint64, _P, C.POINTER(VxShape), C.c_uint64,
                                 C.c_uint32, C.c_uint32]),
    "vx_contiguous": (C.c_int32, [_P, _P, C.c_uint64, _P, C.POINTER(VxShape), C.c_uint64, C.c_uint32]),
    "vx_repeat": (C.c_int32, [_P, _P, C.POINTER(VxShape), C.c_uint64, _P, C.POINTER(VxShape), C.c_uint64]),
    "vx_op_assign_dispatch": (C.c_int32, [_P, C.c_int, C.c_int32, _P, _LP, C.c_uint64, _P, _LP, C.c_uint64]),
    "vx_wfile_open": (C.c_int32, [C.c_char_p, C.POINTER(_P)]),
    "vx_wfile_close": (C.c_int32, [_P]),
    "vx_wfile_count": (C.c_int32, [_P, C.POINTER(C.c_size_t)]),
    "vx_wfile_tensor": (C.c_int32, [_P, C.c_size_t, C.c_char_p, C.c_size_t, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                    C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "vx_wfile_find": (C.c_int32, [_P, C.c_char_p, C.POINTER(C.c_size_t)]),
    "vx_wfile_data": (C.c_int32, [_P, C.c_size_t, C.POINTER(_P), C.POINTER(C.c_uint64)]),
    "vx_wfile_load_qweights": (C.c_int32, [_P, _P, C.c_size_t, C.POINTER(_P)]),
    "vx_checksum_u32": (C.c_int32, [_P, _P, C.c_size_t, _P]),
    "vx_qweights_checksum": (C.c_int32, [_P, _P, _P]),
    "vx_download_2d": (C.c_int32, [_P, _P, C.c_size_t, _P, C.c_size_t, C.c_size_t, C.c_size_t]),
    "vx_set_option": (C.c_int32, [_P, C.c_char_p, C.c_int64]),
    "vx_get_option": (C.c_int32, [_P, C.c_char_p, C.POINTER(C.c_int64)]),
    # host mirror
    "vx_layout_contiguous": (C.c_int32, [_U32P, C.c_uint32, _LP]),
    "vx_layout_to_shape": (C.c_int32, [_LP, C.POINTER(VxShape)]),
    "vx_layout_canonicalize": (C.c_int32, [_LP, _LP]),
    "vx_layout_unsqueeze_to_rank": (C.c_int32, [_LP, C.c_uint32, _LP]),
    "vx_layout_unsqueeze": (C.c_int32, [_LP, C.c_uint32, _LP]),
    "vx_layout_squeeze_axis": (C.c_int32, [_LP, C.c_uint32, _LP]),
    "vx_layout_squeeze": (C.c_int32, [_LP, _LP]),
    "vx_layout_index": (C.c_int32, [_LP, C.c_uint32, _LP]),
    "vx_layout_transpose": (C.c_int32, [_LP, C.c_uint32, C.c_uint32, _LP]),
    "vx_layout_transpose_last_dims": (C.c_int32, [_LP, _LP]),
    "vx_layout_permute": (C.c_int32, [_LP, _U32P, _LP]),
    "vx_layout_permute_ggml": (C.c_int32, [_LP, _U32P, _LP]),
    "vx_layout_is_contiguous": (C.c_int32, [_LP]),
    "vx_layout_broadcast": (C.c_int32, [_LP, _LP, _LP, _LP]),
    "vx_layout_broadcast_assign": (C.c_int32, [_LP, _LP, _LP, _LP]),
    "vx_layout_view": (C.c_int32, [_LP, C.c_uint32, _U32P, C.c_uint32, _U32P,
                                   C.POINTER(C.c_uint8), C.c_uint32, _LP]),
    "vx_layout_reshape": (C.c_int32, [_LP, _U32P, C.c_uint32, _LP]),
    "vx_layout_narrow": (C.c_int32, [_LP, C.c_uint32, C.c_uint32, C.c_uint32, _LP]),
    "vx_layout_matrix": (C.c_int32, [_LP, C.c_uint32, _LP]),
    "vx_layout_columns": (C.c_int32, [_LP, C.c_uint32, C.c_uint32, _LP]),
    "vx_layout_rows": (C.c_int32, [_LP, C.c_uint32, C.c_uint32, _LP]),
    "vx_layout_f32_to_vec4": (C.c_int32, [_LP, _LP]),
    "vx_layout_len": (C.c_uint64, [_LP]),
    "vx_layout_span": (C.c_uint64, [_LP]),
    "vx_gemm_dispatch": (C.c_int32, [_P, C.c_int, _P, _LP, C.c_uint64, _P, _LP, C.c_uint64,
                                     _P, _LP, C.c_uint64]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the shared library once and types every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. "
            "Run `python -m vortx_b200.build` (needs nvcc); there is no fallback path.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().vx_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raises the exception that corresponds to a non-zero status."""
    if status == VX_OK:
        return
    msg = last_error()
    if status == VX_ERR_SHAPE:
        raise ShapeMismatch(status, msg)
    raise VortxError(status, msg)
