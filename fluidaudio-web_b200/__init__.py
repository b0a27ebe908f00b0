"""CUDA (sm_100a) compute backend for fluidaudio-web's quantized matrix-product path.

`CudaContext` implements the reference's ComputeContext operator interface
(src/gpu/compute.d.ts:106-255) for the hot path - matmul / matmulInt8 / matmulNBits and
the glue ops its encoder/decoder forwards call between them - on top of the C-ABI
library `libfa_cuda.so` (include/fa_cuda.h).  There is no CPU fallback: importing works
anywhere, creating a context without the built library or without a B200 raises.
"""
from .context import ACT, CudaContext, CudaError, PackedBytes, StagedRead, Tensor, create_context
from ._lib import library_path, load_library

__all__ = ["ACT", "CudaContext", "CudaError", "PackedBytes", "StagedRead", "Tensor", "create_context",
           "library_path", "load_library"]
