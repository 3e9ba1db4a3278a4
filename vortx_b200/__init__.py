"""vortx_b200 — the B200 (sm_100a) matmul path of vortx behind vortx's own interface.

The package is a thin host mirror (Tensor / TensorLayout / Gemm with the reference's names)
over libvortx_b200.so, a C-ABI library of hand-written CUDA.  Importing the package does
not load the library; the first call does, and fails loudly if it has not been built.
"""
from ._lib import (LayoutError, ShapeMismatch, VortxError, load, LIB_PATH)
from .backend import Backend, BufferUsages, GpuBuffer, GpuBufferSlice, GpuEncoder, GpuPass
from .shapes import GGML_IDS, TensorLayout, TensorLayoutBuffers
from .tensor import Tensor, TensorBuilder, TensorMut, TensorRef
from .weights_file import WeightFile, write_gguf
from .linalg import (Contiguous, Gemm, Gemv, GemvBatch, HostStages, MatrixMode, N, OpAssign, OpAssignVariant, Q4_0, Q8_0, QuantizedMatrix,
                     Reduce, ReduceVariant, Repeat, T, dequantize_host, quantize)

__all__ = [
    "Backend", "BufferUsages", "GpuBuffer", "GpuBufferSlice", "GpuEncoder", "GpuPass",
    "GGML_IDS", "TensorLayout", "TensorLayoutBuffers", "Tensor", "TensorBuilder", "TensorMut",
    "TensorRef", "Gemm", "Gemv", "GemvBatch", "HostStages", "Reduce", "ReduceVariant", "OpAssign", "OpAssignVariant", "Contiguous", "Repeat",
    "MatrixMode", "N", "T", "Q4_0", "Q8_0", "QuantizedMatrix",
    "quantize", "dequantize_host", "WeightFile", "write_gguf", "LayoutError", "ShapeMismatch", "VortxError", "load", "LIB_PATH",
]
