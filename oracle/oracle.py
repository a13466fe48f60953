"""ctypes binding of the CPU oracle (oracle/zinc_oracle.cpp).

TEST INFRASTRUCTURE ONLY. The oracle restates the reference's CPU math for the
quantized matmul path; tests, the smoke check and the benchmark's CPU-baseline
legs load it to check or to time against. The product package never imports
this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libzinc_oracle.so")

F32, F16, Q5_0, Q5_1, Q8_0, Q4_K, Q5_K, Q6_K, MXFP4 = 0, 1, 6, 7, 8, 12, 13, 14, 39


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile if the .so is missing or stale."""
    src = os.path.join(_HERE, "zinc_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libzinc_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = C.CDLL(_SO)
        u8p, f32p, f64p, u32p = (C.POINTER(C.c_uint8), C.POINTER(C.c_float),
                                 C.POINTER(C.c_double), C.POINTER(C.c_uint32))
        L.zo_block_size.restype = C.c_uint32
        L.zo_bytes_per_block.restype = C.c_uint32
        L.zo_tensor_size_bytes.restype = C.c_uint64
        L.zo_tensor_size_bytes.argtypes = [C.c_uint32, C.c_uint64]
        L.zo_expert_slice_bytes.restype = C.c_uint32
        L.zo_expert_slice_bytes.argtypes = [C.c_uint32] * 3
        L.zo_dmmv_bytes_model.restype = C.c_uint64
        L.zo_dmmv_bytes_model.argtypes = [C.c_uint32] * 3
        L.zo_get_scale_min_k4.argtypes = [C.c_uint32, u8p, u8p, u8p]
        L.zo_dequant_row.argtypes = [u8p, C.c_uint64, C.c_uint32, C.c_uint32, f32p]
        L.zo_dequant_rows.argtypes = [u8p, C.c_uint64, C.c_uint32, C.c_uint32, f32p]
        L.zo_dmmv_f32seq.argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32, f32p, f32p, C.c_uint32]
        L.zo_dmmv_f64.argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32, f32p, f64p]
        L.zo_gemm_f64.argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32, f32p, C.c_uint32, f64p, C.c_uint32]
        L.zo_dmmv_shader_order.argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32, f32p, f32p,
                                           C.c_uint32, C.c_int32]
        L.zo_topk_softmax.argtypes = [f32p, C.c_uint32, C.c_uint32, u32p, f32p]
        L.zo_topk_softmax_weight.argtypes = [f32p, C.c_uint32, C.c_uint32, u32p, f32p]
        L.zo_rms_norm_dmmv_f32.argtypes = [f32p, f32p, f32p, f32p, C.POINTER(C.c_double), C.c_uint32, C.c_uint32,
                                           C.c_float]
        L.zo_attn_merge.argtypes = [f32p, f32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]
        L.zo_swiglu.argtypes = [f32p, f32p, f32p, C.c_uint32]
        L.zo_swiglu_oai.argtypes = [f32p, f32p, f32p, C.c_uint32]
        L.zo_moe_weighted_acc.argtypes = [f32p, f32p, u32p, C.c_uint32, C.c_uint32, C.c_uint32]
        L.zo_count_experts.argtypes = [u32p, u32p] + [C.c_uint32] * 6
        L.zo_moe_route_pack.argtypes = [u32p] + [C.c_uint32] * 5 + [u32p, u32p]
        L.zo_moe_route_scatter.argtypes = [u32p, f32p, f32p] + [C.c_uint32] * 4
        L.zo_moe_dmmv_f64.argtypes = [u8p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint64, u32p,
                                      C.c_uint32, C.c_uint32, f32p, f64p]
        _lib = L
    return _lib


def _p(a: np.ndarray, ct):
    return a.ctypes.data_as(C.POINTER(ct))


def _u8(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def block_size(t: int) -> int:
    return lib().zo_block_size(t)


def bytes_per_block(t: int) -> int:
    return lib().zo_bytes_per_block(t)


def tensor_size_bytes(t: int, n: int) -> int:
    return lib().zo_tensor_size_bytes(t, n)


def expert_slice_bytes(t: int, rows: int, cols: int) -> int:
    return lib().zo_expert_slice_bytes(t, rows, cols)


def dmmv_bytes_model(t: int, M: int, K: int) -> int:
    return lib().zo_dmmv_bytes_model(t, M, K)


def get_scale_min_k4(j: int, scales) -> tuple[int, int]:
    s = _u8(np.asarray(scales, dtype=np.uint8))
    sc, m = C.c_uint8(), C.c_uint8()
    lib().zo_get_scale_min_k4(j, _p(s, C.c_uint8), C.byref(sc), C.byref(m))
    return sc.value, m.value


def dequant_row(raw, row: int, cols: int, t: int) -> np.ndarray:
    raw = _u8(raw)
    out = np.empty(cols, dtype=np.float32)
    lib().zo_dequant_row(_p(raw, C.c_uint8), row, cols, t, _p(out, C.c_float))
    return out


def dequant_rows(raw, rows: int, cols: int, t: int) -> np.ndarray:
    raw = _u8(raw)
    out = np.empty((rows, cols), dtype=np.float32)
    rc = lib().zo_dequant_rows(_p(raw, C.c_uint8), rows, cols, t, _p(out, C.c_float))
    if rc != 0:
        raise ValueError(f"oracle: unsupported type {t}")
    return out


def dmmv_f32seq(raw, t: int, M: int, K: int, x, y0=None) -> np.ndarray:
    raw = _u8(raw)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.zeros(M, dtype=np.float32) if y0 is None else np.array(y0, dtype=np.float32)
    lib().zo_dmmv_f32seq(_p(raw, C.c_uint8), t, M, K, _p(x, C.c_float), _p(y, C.c_float),
                         0 if y0 is None else 1)
    return y


def dmmv_f64(raw, t: int, M: int, K: int, x) -> np.ndarray:
    raw = _u8(raw)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(M, dtype=np.float64)
    rc = lib().zo_dmmv_f64(_p(raw, C.c_uint8), t, M, K, _p(x, C.c_float), _p(y, C.c_double))
    if rc != 0:
        raise ValueError(f"oracle: unsupported type {t}")
    return y


def gemm_f64(raw, t: int, M: int, K: int, X, round_bf16: bool = False) -> np.ndarray:
    """Y[c][M] = W X[c][K], f64 accumulate; X is [T][K] f32."""
    raw = _u8(raw)
    X = np.ascontiguousarray(X, dtype=np.float32)
    T = X.shape[0]
    Y = np.empty((T, M), dtype=np.float64)
    rc = lib().zo_gemm_f64(_p(raw, C.c_uint8), t, M, K, _p(X, C.c_float), T, _p(Y, C.c_double),
                           1 if round_bf16 else 0)
    if rc != 0:
        raise ValueError(f"oracle: unsupported type {t}")
    return Y


def dmmv_shader_order(raw, t: int, M: int, K: int, x, n_threads: int = 0) -> np.ndarray:
    raw = _u8(raw)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.zeros(M, dtype=np.float32)
    rc = lib().zo_dmmv_shader_order(_p(raw, C.c_uint8), t, M, K, _p(x, C.c_float), _p(y, C.c_float),
                                    0, n_threads)
    if rc != 0:
        raise ValueError(f"oracle: unsupported type {t}")
    return y


def max_threads() -> int:
    return lib().zo_max_threads()


def topk_softmax(logits, k: int):
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    ids = np.empty(k, dtype=np.uint32)
    w = np.empty(k, dtype=np.float32)
    lib().zo_topk_softmax(_p(lg, C.c_float), lg.size, k, _p(ids, C.c_uint32), _p(w, C.c_float))
    return ids, w


def topk_softmax_weight(logits, k: int):
    lg = np.ascontiguousarray(logits, dtype=np.float32)
    ids = np.empty(k, dtype=np.uint32)
    w = np.empty(k, dtype=np.float32)
    lib().zo_topk_softmax_weight(_p(lg, C.c_float), lg.size, k, _p(ids, C.c_uint32), _p(w, C.c_float))
    return ids, w


def rms_norm_dmmv_f32(x, norm_w, W, M: int, K: int, eps: float):
    """(normalised vector f32 [K], router logits f64 [M]) of the fused RMS norm + f32 router matvec."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(norm_w, dtype=np.float32)
    Wm = np.ascontiguousarray(W, dtype=np.float32)
    xn = np.empty(K, dtype=np.float32)
    logits = np.empty(M, dtype=np.float64)
    lib().zo_rms_norm_dmmv_f32(_p(x, C.c_float), _p(w, C.c_float), _p(Wm, C.c_float), _p(xn, C.c_float),
                               _p(logits, C.c_double), M, K, eps)
    return xn, logits


def attn_merge(partial, sinks, n_heads: int, n_chunks: int, head_dim: int, sink_offset: int = 0) -> np.ndarray:
    """Attention output [n_heads * head_dim] merged from split-K partials + their LSE region (sinks: f32 array,
    NaN = none, or None)."""
    p = np.ascontiguousarray(partial, dtype=np.float32)
    out = np.empty(n_heads * head_dim, dtype=np.float32)
    s = None if sinks is None else np.ascontiguousarray(sinks, dtype=np.float32)
    lib().zo_attn_merge(_p(p, C.c_float), None if s is None else _p(s, C.c_float), _p(out, C.c_float), n_heads,
                        n_chunks, head_dim, sink_offset)
    return out


def swiglu(gate, up, oai: bool = False) -> np.ndarray:
    g = np.ascontiguousarray(gate, dtype=np.float32)
    u = np.ascontiguousarray(up, dtype=np.float32)
    out = np.empty_like(g)
    fn = lib().zo_swiglu_oai if oai else lib().zo_swiglu
    fn(_p(g, C.c_float), _p(u, C.c_float), _p(out, C.c_float), g.size)
    return out


def moe_weighted_acc(a, b, routing, n: int, n_used: int, src_stride: int) -> np.ndarray:
    a = np.array(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    r = np.ascontiguousarray(routing, dtype=np.uint32)
    lib().zo_moe_weighted_acc(_p(a, C.c_float), _p(b, C.c_float), _p(r, C.c_uint32), n, n_used, src_stride)
    return a


def count_experts(a, n_experts: int, ne00: int, ne01: int, nb00: int, nb01: int, a_offset: int) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint32)
    out = np.empty(n_experts, dtype=np.uint32)
    lib().zo_count_experts(_p(a, C.c_uint32), _p(out, C.c_uint32), n_experts, ne00, ne01, nb00, nb01, a_offset)
    return out


def moe_route_pack(routing, n_tokens: int, n_experts: int, k: int, routing_stride: int, ids_stride: int):
    r = np.ascontiguousarray(routing, dtype=np.uint32)
    counts = np.zeros(n_experts, dtype=np.uint32)
    ids = np.full(n_experts * ids_stride, 0xFFFFFFFF, dtype=np.uint32)
    lib().zo_moe_route_pack(_p(r, C.c_uint32), n_tokens, n_experts, k, routing_stride, ids_stride,
                            _p(counts, C.c_uint32), _p(ids, C.c_uint32))
    return counts, ids.reshape(n_experts, ids_stride)


def moe_route_scatter(routing, src, dst, n_tokens: int, hidden: int, k: int, routing_stride: int) -> np.ndarray:
    r = np.ascontiguousarray(routing, dtype=np.uint32)
    s = np.ascontiguousarray(src, dtype=np.float32)
    d = np.array(dst, dtype=np.float32)
    lib().zo_moe_route_scatter(_p(r, C.c_uint32), _p(s, C.c_float), _p(d, C.c_float), n_tokens, hidden, k,
                               routing_stride)
    return d


def moe_dmmv_f64(raw, t: int, M: int, K: int, expert_stride: int, routing_ids, x_expert_stride: int, x):
    raw = _u8(raw)
    ids = np.ascontiguousarray(routing_ids, dtype=np.uint32)
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty((ids.size, M), dtype=np.float64)
    rc = lib().zo_moe_dmmv_f64(_p(raw, C.c_uint8), t, M, K, expert_stride, _p(ids, C.c_uint32), ids.size,
                               x_expert_stride, _p(x, C.c_float), _p(y, C.c_double))
    if rc != 0:
        raise ValueError(f"oracle: unsupported type {t}")
    return y
