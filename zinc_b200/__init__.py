"""zinc_b200: B200 (sm_100a) quantized-matmul path behind the ZINC engine's DMMV dispatch interface.

The product is the CUDA shared library `libzinc_b200.so` (C ABI in
include/zinc_cuda.h). This package is its thin host-side mirror of the
reference's dispatch layer plus seeded synthetic inputs for tests and the
benchmark. It has no CPU compute path.
"""
from ._lib import (BF16, F16, F32, MXFP4, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0, TYPE_NAMES,
                   ROUTE_SOFTMAX_ALL_RENORM, ROUTE_TOPK_THEN_SOFTMAX, SHARED_EXPERT, SKIP_EXPERT, SO_PATH)
from .dispatch import (Buffer, Context, CudaError, DeviceTimeout, DmmvDispatch, InvalidArgument, OutOfMemory,
                       PipelineNotLoaded, UnsupportedQuantType, ZincError, block_size, bytes_per_block,
                       expert_slice_bytes, row_bytes, tensor_size_bytes)

__all__ = [
    "BF16", "F16", "F32", "MXFP4", "Q4_K", "Q5_0", "Q5_1", "Q5_K", "Q6_K", "Q8_0", "TYPE_NAMES",
    "ROUTE_SOFTMAX_ALL_RENORM", "ROUTE_TOPK_THEN_SOFTMAX", "SHARED_EXPERT", "SKIP_EXPERT", "SO_PATH",
    "Buffer", "Context", "CudaError", "DeviceTimeout", "DmmvDispatch", "InvalidArgument", "OutOfMemory",
    "PipelineNotLoaded", "UnsupportedQuantType", "ZincError", "block_size", "bytes_per_block",
    "expert_slice_bytes", "row_bytes", "tensor_size_bytes",
]
