"""ctypes binding of libzinc_b200.so (the C ABI declared in include/zinc_cuda.h).

The library is the product; this module only loads it and declares argument
types. There is no fallback: if the shared library is missing the import
raises, and every compute call needs a CUDA device of compute capability 10.x.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libzinc_b200.so")

OK, ERR_UNSUPPORTED_TYPE, ERR_NOT_LOADED, ERR_INVALID_ARG, ERR_OOM, ERR_CUDA, ERR_TIMEOUT = range(7)

# GGML type ids (src/model/gguf.zig:38-69 of the reference project)
F32, F16, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, BF16, MXFP4 = 0, 1, 6, 7, 8, 12, 13, 14, 30, 39
TYPE_NAMES = {F32: "f32", F16: "f16", Q5_0: "q5_0", Q5_1: "q5_1", Q8_0: "q8_0", Q4_K: "q4_k",
              Q5_K: "q5_k", Q6_K: "q6_k", BF16: "bf16", MXFP4: "mxfp4"}

ROUTE_SOFTMAX_ALL_RENORM, ROUTE_TOPK_THEN_SOFTMAX = 0, 1
# routing ids with a meaning of their own: no expert in this slot on this rank / the shared expert
SKIP_EXPERT, SHARED_EXPERT = 0xFFFFFFFF, 0xFFFFFFFE

_u32, _u64, _i32, _vp = C.c_uint32, C.c_uint64, C.c_int32, C.c_void_p

# name -> argument types after the leading zc_ctx* (all return int32 status)
_OPS = {
    "zc_dmmv": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u64, _u64, _u32],
    "zc_dmmv_push": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u64, _u64, _u32],
    "zc_dmmv_fused_gate_up_swiglu": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32,
                                     _u64, _u64, _u64, _u64],
    "zc_dmmv_sigmoid_acc": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u64, _u64, _u32],
    "zc_rms_norm_dmmv_f32": [_vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, C.c_float],
    "zc_mul_mm_block_scaled": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _u32, _u32, _u64, _u64, _u64, _vp,
                               _u64],
    "zc_dmmv_o_proj_merge": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u64, _u32, _u32, _u32, _u32,
                             _u32],
    "zc_moe_gate_up_act_ex": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64,
                              _vp, _u64, _u32, _u32, _u64, _u32, _u64, _u64, _u32],
    "zc_moe_down_acc_ex": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u32,
                           _u32, _u64, _u64],
    "zc_moe_router_topk": [_vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32,
                           _u32, _u32, C.c_float, _u32, _u32, _u32, _u32],
    "zc_rms_norm_dmmv_alpha_beta": [_vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32,
                                    C.c_float],
    "zc_dmmv_multi": [_u32, _u32, C.POINTER(_vp), C.POINTER(_u64), C.POINTER(_u64), _vp, _u64, _u64,
                      C.POINTER(_vp), C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u32), _u32, _u32],
    "zc_dmmv_batch": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u64, _u64, _u32],
    "zc_mul_mm": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _u32, _u32, _u64, _u64, _u64, _u32],
    "zc_moe_dmmv": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u32, _u32, _u64, _u64],
    "zc_moe_fused_gate_up": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64,
                             _u32, _u32, _u64, _u32, _u32, _u64, _u64],
    "zc_moe_fused_down_acc": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u32, _u32,
                              _u64, _u64],
    "zc_moe_fused_gate_up_act": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u32,
                                 _u32, _u64, _u64, _u32],
    "zc_moe_dmmv_batched_pair": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32,
                                 _u64, _u32, _u32, _u32, _u32, _u32],
    "zc_moe_dmmv_batched": [_u32, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u32, _u32, _u32,
                            _u32, _u32],
    "zc_softmax_topk": [_vp, _u64, _vp, _vp, _u64, _u32, _u32, _u32, _u32, _u32, _u32],
    "zc_moe_weighted_acc": [_vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32],
    "zc_swiglu": [_vp, _vp, _vp, _u32],
    "zc_swiglu_oai": [_vp, _vp, _vp, _u32],
    "zc_bias_add": [_vp, _u64, _vp, _u64, _u32, _u32],
    "zc_moe_bias_act": [_vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _u32],
    "zc_moe_weighted_bias_acc": [_vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32],
    "zc_set_wait_limit": [_u32],
    "zc_comm_connect_local": [_u32, _vp, _u64],
    "zc_moe_ep_filter": [_vp, _u64, _vp, _u64, _u32, _u32, _u32, _u32, _u32, _u32],
    "zc_count_experts": [_vp, _u64, _vp, _u64, _u32, _u32, _u32, _u32, _u32, _u64],
    "zc_moe_route_pack": [_vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _u32, _u32],
    "zc_moe_route_scatter": [_vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u32, _u32],
    "zc_dequant_rows": [_u32, _vp, _u64, _vp, _u64, _u64, _u32, _u32, _u64],
    "zc_alloc": [_u64, C.POINTER(_vp)],
    "zc_free": [_vp],
    "zc_upload": [_vp, _u64, _vp, _u64],
    "zc_download": [_vp, _vp, _u64, _u64],
    "zc_memset": [_vp, _u64, _i32, _u64],
    "zc_set_stream": [_vp],
    "zc_use_own_stream": [],
    "zc_set_workspace": [_vp, _u64],
    "zc_comm_init": [_u32, _u32, _vp],
    "zc_comm_connect": [_vp],
    "zc_allreduce_sum_f32": [_vp, _u64, _u64, _u32],
    "zc_allgather_f32": [_vp, _u64, _u64, _vp, _u64, _u64, _u32],
    "zc_comm_destroy": [],
    "zc_begin_record": [],
    "zc_end_record": [C.POINTER(_vp)],
    "zc_replay": [_vp],
    "zc_free_recording": [_vp],
    "zc_barrier": [],
    "zc_submit_and_wait": [],
    "zc_destroy": [],
}

# every symbol include/zinc_cuda.h declares
EXPORTS = sorted(list(_OPS) + [
    "zc_init", "zc_get_stream", "zc_last_error", "zc_status_string", "zc_launch_count",
    "zc_block_size", "zc_bytes_per_block", "zc_tensor_size_bytes", "zc_expert_slice_bytes",
    "zc_dmmv_supported", "zc_moe_dmmv_supported", "zc_dmmv_q4k_static_scratch", "zc_moe_grouped_workspace_bytes",
    "zc_comm_buffer_bytes", "zc_mul_mm_workspace_bytes",
])

_lib = None


def lib() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise ImportError(
                f"{SO_PATH} is missing: build it with `python -m zinc_b200.build` "
                "(nvcc, sm_100a). There is no CPU fallback.")
        L = C.CDLL(SO_PATH)
        for name, args in _OPS.items():
            fn = getattr(L, name)
            fn.restype = _i32
            fn.argtypes = [_vp] + args
        L.zc_init.restype = _i32
        L.zc_init.argtypes = [_i32, C.POINTER(_vp)]
        L.zc_get_stream.restype = _vp
        L.zc_get_stream.argtypes = [_vp]
        L.zc_last_error.restype = C.c_char_p
        L.zc_last_error.argtypes = [_vp]
        L.zc_status_string.restype = C.c_char_p
        L.zc_status_string.argtypes = [_i32]
        L.zc_launch_count.restype = _u64
        L.zc_launch_count.argtypes = [_vp]
        for name in ("zc_block_size", "zc_bytes_per_block"):
            getattr(L, name).restype = _u32
            getattr(L, name).argtypes = [_u32]
        L.zc_comm_buffer_bytes.restype = _u64
        L.zc_comm_buffer_bytes.argtypes = []
        L.zc_mul_mm_workspace_bytes.restype = _u64
        L.zc_mul_mm_workspace_bytes.argtypes = [_u32, _u32, _u32]
        L.zc_moe_grouped_workspace_bytes.restype = _u64
        L.zc_moe_grouped_workspace_bytes.argtypes = [_u32, _u32, _u32, _u32]
        L.zc_tensor_size_bytes.restype = _u64
        L.zc_tensor_size_bytes.argtypes = [_u32, _u64]
        L.zc_expert_slice_bytes.restype = _u64
        L.zc_expert_slice_bytes.argtypes = [_u32, _u32, _u32]
        L.zc_dmmv_supported.restype = _i32
        L.zc_dmmv_supported.argtypes = [_u32]
        L.zc_moe_dmmv_supported.restype = _i32
        L.zc_moe_dmmv_supported.argtypes = [_u32]
        L.zc_dmmv_q4k_static_scratch.restype = _i32
        L.zc_dmmv_q4k_static_scratch.argtypes = [_vp, _vp, _u64, _vp, _u64, _vp, _u64, _u32, _u32, _u64, _u64, _u64,
                                                 _u32, _vp, C.c_char_p, _u64]
        _lib = L
    return _lib
