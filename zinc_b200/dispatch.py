"""Host-side mirror of the reference's DMMV dispatch layer over the C ABI.

`DmmvDispatch` keeps the method names, argument order, units and error
behaviour of `DmmvDispatch` in the reference (src/compute/dmmv.zig:161-1094)
and of the engine-side wrappers that call it (src/compute/forward.zig:
8147-8540, 4135-4210), so a call site of the reference translates line by
line. Where the reference binds buffers through a descriptor set, the methods
here take `Buffer` objects (device pointer + byte size) in binding order.

Everything computes on the GPU through libzinc_b200.so; nothing here touches
tensor data on the host.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any, Optional

from . import _lib
from ._lib import (BF16, F16, F32, MXFP4, Q4_K, Q5_0, Q5_1, Q5_K, Q6_K, Q8_0,  # noqa: F401 (re-exported)
                   ROUTE_SOFTMAX_ALL_RENORM, ROUTE_TOPK_THEN_SOFTMAX)


class ZincError(RuntimeError):
    status = -1


class UnsupportedQuantType(ZincError):  # error.UnsupportedQuantType
    status = _lib.ERR_UNSUPPORTED_TYPE


class PipelineNotLoaded(ZincError):  # error.PipelineNotLoaded
    status = _lib.ERR_NOT_LOADED


class InvalidArgument(ZincError):  # error.InvalidArgument
    status = _lib.ERR_INVALID_ARG


class OutOfMemory(ZincError):
    status = _lib.ERR_OOM


class CudaError(ZincError):
    status = _lib.ERR_CUDA


class DeviceTimeout(ZincError):
    status = _lib.ERR_TIMEOUT


_ERRORS = {c.status: c for c in (UnsupportedQuantType, PipelineNotLoaded, InvalidArgument, OutOfMemory,
                                 CudaError, DeviceTimeout)}


@dataclass
class Buffer:
    """A borrowed device allocation: pointer + byte size (the reference's Buffer.handle/size)."""
    ptr: int
    size: int
    owner: Any = None  # keeps the backing object (torch tensor / context allocation) alive

    @staticmethod
    def from_torch(t) -> "Buffer":
        if not t.is_cuda:
            raise InvalidArgument("Buffer.from_torch needs a CUDA tensor")
        if not t.is_contiguous():
            raise InvalidArgument("Buffer.from_torch needs a contiguous tensor")
        return Buffer(t.data_ptr(), t.numel() * t.element_size(), t)


def _buf(b) -> Buffer:
    if isinstance(b, Buffer):
        return b
    if hasattr(b, "data_ptr"):
        return Buffer.from_torch(b)
    raise InvalidArgument(f"expected a Buffer or CUDA tensor, got {type(b).__name__}")


class Context:
    """One device + one stream: the unit the reference calls an engine's command buffer."""

    def __init__(self, device: int = 0, stream: Optional[int] = None):
        self._lib = _lib.lib()
        h = C.c_void_p()
        rc = self._lib.zc_init(device, C.byref(h))
        if rc != _lib.OK:
            raise _ERRORS.get(rc, ZincError)(
                f"zc_init(device={device}) failed: {self._lib.zc_status_string(rc).decode()}")
        self._h = h
        self.device = device
        if stream is not None:
            self.set_stream(stream)

    # -- plumbing --------------------------------------------------------------------------
    def call(self, name: str, *args) -> None:
        rc = getattr(self._lib, name)(self._h, *args)
        if rc != _lib.OK:
            msg = self._lib.zc_last_error(self._h).decode()
            raise _ERRORS.get(rc, ZincError)(f"{name}: {msg}")

    def set_stream(self, stream: Optional[int]) -> None:
        """Launch on the given cudaStream_t handle (0 / None = CUDA's default stream)."""
        self.call("zc_set_stream", C.c_void_p(stream or 0))

    def use_own_stream(self) -> None:
        self.call("zc_use_own_stream")

    @property
    def stream(self) -> int:
        return self._lib.zc_get_stream(self._h) or 0

    @property
    def launch_count(self) -> int:
        return int(self._lib.zc_launch_count(self._h))

    def alloc(self, nbytes: int) -> Buffer:
        p = C.c_void_p()
        self.call("zc_alloc", nbytes, C.byref(p))
        return Buffer(p.value, nbytes, self)

    def free(self, b: Buffer) -> None:
        self.call("zc_free", C.c_void_p(b.ptr))
        b.ptr, b.size = 0, 0

    def upload(self, dst: Buffer, host, dst_offset: int = 0) -> None:
        """host: any object with the buffer protocol (numpy array, bytes)."""
        mv = memoryview(host).cast("B")
        src = (C.c_uint8 * len(mv)).from_buffer_copy(mv) if mv.readonly else (C.c_uint8 * len(mv)).from_buffer(mv)
        self.call("zc_upload", C.c_void_p(dst.ptr), dst_offset, C.cast(src, C.c_void_p), len(mv))
        self.submit_and_wait()

    def download(self, src: Buffer, nbytes: int, src_offset: int = 0) -> bytes:
        out = (C.c_uint8 * nbytes)()
        self.call("zc_download", C.cast(out, C.c_void_p), C.c_void_p(src.ptr), src_offset, nbytes)
        self.submit_and_wait()
        return bytes(out)

    def upload_from_ptr(self, dst: Buffer, host_ptr: int, nbytes: int, dst_offset: int = 0) -> None:
        """Asynchronous copy from (pinned) host memory; ordered on the context's stream."""
        self.call("zc_upload", C.c_void_p(dst.ptr), dst_offset, C.c_void_p(host_ptr), nbytes)

    def download_to_ptr(self, host_ptr: int, src: Buffer, nbytes: int, src_offset: int = 0) -> None:
        """Asynchronous copy to (pinned) host memory; complete after submit_and_wait()."""
        self.call("zc_download", C.c_void_p(host_ptr), C.c_void_p(src.ptr), src_offset, nbytes)

    def memset(self, dst: Buffer, value: int, nbytes: Optional[int] = None, dst_offset: int = 0) -> None:
        self.call("zc_memset", C.c_void_p(dst.ptr), dst_offset, value, dst.size - dst_offset if nbytes is None else nbytes)

    def barrier(self) -> None:  # computeBarrier (src/vulkan/command.zig:345-425): stream order already holds
        self.call("zc_barrier")

    def submit_and_wait(self) -> None:  # submitAndWait (src/vulkan/command.zig:477)
        self.call("zc_submit_and_wait")

    # -- pre-recorded sequences (a command buffer recorded once and submitted per token) ------
    def begin_record(self) -> None:
        self.call("zc_begin_record")

    def end_record(self) -> int:
        h = C.c_void_p()
        self.call("zc_end_record", C.byref(h))
        return h.value

    def replay(self, recording: int) -> None:
        self.call("zc_replay", C.c_void_p(recording))

    def free_recording(self, recording: int) -> None:
        self.call("zc_free_recording", C.c_void_p(recording))

    # -- tensor-parallel exchange ------------------------------------------------------------
    def comm_init(self, rank: int, world: int) -> bytes:
        """Allocate this rank's receive buffer; returns its 64-byte IPC handle for the other ranks."""
        h = (C.c_uint8 * 64)()
        self.call("zc_comm_init", rank, world, C.cast(h, C.c_void_p))
        return bytes(h)

    def comm_connect(self, handles: "list[bytes]") -> None:
        """Map the receive buffers of all ranks (handles in rank order, this rank's own included)."""
        blob = b"".join(handles)
        arr = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        self.call("zc_comm_connect", C.cast(arr, C.c_void_p))

    def allreduce_sum(self, buf, n: int, offset: int = 0) -> None:
        b = _buf(buf)
        self.call("zc_allreduce_sum_f32", b.ptr, b.size, offset, n)

    def allgather(self, src, dst, n: int, src_offset: int = 0, dst_offset: int = 0) -> None:
        a, b = _buf(src), _buf(dst)
        self.call("zc_allgather_f32", a.ptr, a.size, src_offset, b.ptr, b.size, dst_offset, n)

    def comm_connect_local(self, rank: int, receive_buffer) -> None:
        """Lend the receive buffer of a rank that lives in this process (a device pointer, no IPC handle)."""
        b = _buf(receive_buffer)
        self.call("zc_comm_connect_local", rank, b.ptr, b.size)

    @staticmethod
    def comm_buffer_bytes() -> int:
        return int(_lib.lib().zc_comm_buffer_bytes())

    def set_wait_limit(self, polls: int) -> None:
        """Polls after which a device-side wait gives up (0 = defaults); see zc_set_wait_limit."""
        self.call("zc_set_wait_limit", polls)

    def comm_destroy(self) -> None:
        self.call("zc_comm_destroy")

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.zc_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ---- layout helpers (src/model/gguf.zig:75-122, 222-229; src/compute/forward.zig:650-656) ----
def block_size(t: int) -> int:
    return _lib.lib().zc_block_size(t)


def bytes_per_block(t: int) -> int:
    return _lib.lib().zc_bytes_per_block(t)


def tensor_size_bytes(t: int, n_elements: int) -> int:
    return _lib.lib().zc_tensor_size_bytes(t, n_elements)


def expert_slice_bytes(t: int, rows: int, cols: int) -> int:
    return _lib.lib().zc_expert_slice_bytes(t, rows, cols)


def row_bytes(t: int, K: int) -> int:
    return (K // block_size(t)) * bytes_per_block(t)


class DmmvDispatch:
    """Mirror of DmmvDispatch (src/compute/dmmv.zig:161-297): one object per context."""

    def __init__(self, ctx: Context):
        self.ctx = ctx

    # pipelineForType / moePipelineForType (src/compute/dmmv.zig:678-703)
    def pipelineForType(self, quant_type: int) -> bool:
        return bool(_lib.lib().zc_dmmv_supported(quant_type))

    def moePipelineForType(self, quant_type: int) -> bool:
        return bool(_lib.lib().zc_moe_dmmv_supported(quant_type))

    # recordDispatch (src/compute/dmmv.zig:806-874); buffers in binding order A, x, y
    def recordDispatch(self, quant_type, A, x, y, M, K, a_offset=0, x_offset=0, y_offset=0, acc_mode=0):
        A, x, y = _buf(A), _buf(x), _buf(y)
        self.ctx.call("zc_dmmv", quant_type, A.ptr, A.size, x.ptr, x.size, y.ptr, y.size, M, K,
                      a_offset, x_offset, y_offset, acc_mode)

    # recordDispatch for a K-sharded projection on N GPUs: the partial result is pushed to every rank and
    # summed into dst by the next call on the context (no counterpart in the single-GPU reference)
    def recordDispatchPush(self, quant_type, A, x, dst, M, K, a_offset=0, x_offset=0, dst_offset=0, acc_mode=0):
        A, x, dst = _buf(A), _buf(x), _buf(dst)
        self.ctx.call("zc_dmmv_push", quant_type, A.ptr, A.size, x.ptr, x.size, dst.ptr, dst.size, M, K,
                      a_offset, x_offset, dst_offset, acc_mode)

    # recordBatchDispatchPush (src/compute/dmmv.zig:880-926) + dispatchProjectionBatched chunk loop
    def recordDispatchMulti(self, quant_type, As, x, ys, Ms, K, a_offsets=None, x_offset=0, y_offsets=None,
                            acc_mode=0):
        """Several recordDispatch calls on the same input (the reference's Q, K, V sequence,
        src/compute/forward.zig:4530-4564) as one call: y_i (+)= W_i x."""
        n = len(As)
        if not (n == len(ys) == len(Ms)) or not 1 <= n <= 3:
            raise InvalidArgument("recordDispatchMulti needs 1..3 matrices with matching outputs and row counts")
        Ab, yb, xb = [_buf(a) for a in As], [_buf(y) for y in ys], _buf(x)
        a_offsets = a_offsets or [0] * n
        y_offsets = y_offsets or [0] * n
        vp, u64, u32 = C.c_void_p * n, C.c_uint64 * n, C.c_uint32 * n
        self.ctx.call("zc_dmmv_multi", quant_type, n, vp(*[b.ptr for b in Ab]), u64(*[b.size for b in Ab]),
                      u64(*a_offsets), xb.ptr, xb.size, x_offset, vp(*[b.ptr for b in yb]),
                      u64(*[b.size for b in yb]), u64(*y_offsets), u32(*Ms), K, acc_mode)

    def recordBatchDispatchPush(self, quant_type, A, X, Y, M, K, a_offset, x_offset, y_offset, num_cols):
        A, X, Y = _buf(A), _buf(X), _buf(Y)
        self.ctx.call("zc_dmmv_batch", quant_type, A.ptr, A.size, X.ptr, X.size, Y.ptr, Y.size, M, K,
                      a_offset, x_offset, y_offset, num_cols)

    # recordMoeDispatch (src/compute/dmmv.zig:709-739); bindings A, x, y, routing
    def recordMoeDispatch(self, quant_type, A, x, y, routing, M, K, expert_stride, n_experts_y,
                          x_expert_stride, x_offset=0, y_offset=0):
        A, x, y, routing = _buf(A), _buf(x), _buf(y), _buf(routing)
        self.ctx.call("zc_moe_dmmv", quant_type, A.ptr, A.size, x.ptr, x.size, y.ptr, y.size,
                      routing.ptr, routing.size, M, K, expert_stride, n_experts_y, x_expert_stride,
                      x_offset, y_offset)

    # recordMoeBatchedDispatch (src/compute/dmmv.zig:746-792)
    def recordMoeBatchedDispatch(self, quant_type, A, X, Y, routing, M, K, expert_stride, n_experts,
                                 n_experts_used, n_tokens, x_token_stride, y_token_stride):
        A, X, Y, routing = _buf(A), _buf(X), _buf(Y), _buf(routing)
        self.ctx.call("zc_moe_dmmv_batched", quant_type, A.ptr, A.size, X.ptr, X.size, Y.ptr, Y.size,
                      routing.ptr, routing.size, M, K, expert_stride, n_experts, n_experts_used, n_tokens,
                      x_token_stride, y_token_stride)

    # gate and up of a prefill batch on one grouping (the prefill counterpart of dispatchMoeFusedGateUp)
    def recordMoeBatchedDispatchPair(self, quant_type, Wg, Wu, X, Yg, Yu, routing, M, K, expert_stride, n_experts,
                                     n_experts_used, n_tokens, x_token_stride, y_token_stride):
        Wg, Wu, X, Yg, Yu, routing = map(_buf, (Wg, Wu, X, Yg, Yu, routing))
        self.ctx.call("zc_moe_dmmv_batched_pair", quant_type, Wg.ptr, Wg.size, Wu.ptr, Wu.size, X.ptr, X.size,
                      Yg.ptr, Yg.size, Yu.ptr, Yu.size, routing.ptr, routing.size, M, K, expert_stride, n_experts,
                      n_experts_used, n_tokens, x_token_stride, y_token_stride)

    # Lend the library scratch for the grouped MoE prefill path (no counterpart in the reference's
    # DmmvDispatch; its Metal path owns route_ids / route_counts buffers). None removes it.
    def setWorkspace(self, workspace=None):
        if workspace is None:
            self.ctx.call("zc_set_workspace", None, 0)
        else:
            w = _buf(workspace)
            self.ctx.call("zc_set_workspace", w.ptr, w.size)
        self._workspace = workspace  # keep the tensor alive while the library may use it

    # recordMulMm for MXFP4 weights on the block-scaled FP4 tensor-core path (weights as stored, bf16 activations
    # as two exact FP8 terms in `workspace`)
    def recordMulMmBlockScaled(self, quant_type, a_buf, b_buf, d_buf, M, N, K, stride_b, stride_d, workspace,
                               a_offset=0, b_offset=0, d_offset=0):
        a, b, d, w = map(_buf, (a_buf, b_buf, d_buf, workspace))
        self.ctx.call("zc_mul_mm_block_scaled", quant_type, a.ptr, a.size, b.ptr, b.size, d.ptr, d.size, M, N, K,
                      stride_b, stride_d, a_offset, b_offset, d_offset, w.ptr, w.size)

    @staticmethod
    def mulMmWorkspaceBytes(quant_type, N, K) -> int:
        from ._lib import lib
        return int(lib().zc_mul_mm_workspace_bytes(quant_type, N, K))

    @staticmethod
    def moeGroupedWorkspaceBytes(n_tokens, n_experts_used, K, n_experts) -> int:
        from ._lib import lib
        return int(lib().zc_moe_grouped_workspace_bytes(n_tokens, n_experts_used, K, n_experts))

    # recordCountExperts (src/compute/dmmv.zig:981-1028)
    def recordCountExperts(self, routing, counts, n_tokens, n_layers, layer, n_experts_used, n_experts,
                           d_offset_bytes=0):
        routing, counts = _buf(routing), _buf(counts)
        self.ctx.call("zc_count_experts", routing.ptr, routing.size, counts.ptr, counts.size, n_tokens, n_layers,
                      layer, n_experts_used, n_experts, d_offset_bytes)

    # recordMulMmQ4K (src/compute/dmmv.zig:1045-1094), widened to every type and to bf16 activations
    def recordMulMm(self, quant_type, A, B, D, M, N, K, stride_b, stride_d, a_offset=0, b_offset=0, d_offset=0,
                    act_type=F32):
        A, B, D = _buf(A), _buf(B), _buf(D)
        self.ctx.call("zc_mul_mm", quant_type, A.ptr, A.size, B.ptr, B.size, D.ptr, D.size, M, N, K,
                      stride_b, stride_d, a_offset, b_offset, d_offset, act_type)

    def recordMulMmQ4K(self, A, B, D, M, N, K, stride_b, stride_d, a_offset=0, b_offset=0, d_offset=0):
        self.recordMulMm(Q4_K, A, B, D, M, N, K, stride_b, stride_d, a_offset, b_offset, d_offset, F32)

    # ---- engine-side wrappers (src/compute/forward.zig) ---------------------------------------
    # dispatchDmmvFusedGateUpSwiglu (forward.zig:8237-8313)
    def dispatchDmmvFusedGateUpSwiglu(self, quant_type, Wg, Wu, x, out, M, K, gate_offset=0, up_offset=0,
                                      x_offset=0, out_offset=0):
        Wg, Wu, x, out = _buf(Wg), _buf(Wu), _buf(x), _buf(out)
        self.ctx.call("zc_dmmv_fused_gate_up_swiglu", quant_type, Wg.ptr, Wg.size, Wu.ptr, Wu.size, x.ptr, x.size,
                      out.ptr, out.size, M, K, gate_offset, up_offset, x_offset, out_offset)

    # dispatchDmmvQ8_0SigmoidAcc (forward.zig:8321-8359)
    def dispatchDmmvSigmoidAcc(self, quant_type, A, x, y, gate, M, K, a_offset=0, x_offset=0, y_offset=0,
                               gate_index=0):
        A, x, y, gate = _buf(A), _buf(x), _buf(y), _buf(gate)
        self.ctx.call("zc_dmmv_sigmoid_acc", quant_type, A.ptr, A.size, x.ptr, x.size, y.ptr, y.size,
                      gate.ptr, gate.size, M, K, a_offset, x_offset, y_offset, gate_index)

    # fused gate+up MoE dispatch (forward.zig:6206-6222)
    def dispatchMoeFusedGateUp(self, quant_type, Wg, Wu, x, y_gate, y_up, routing, M, K, expert_stride, n_used,
                               x_expert_stride, x_offset=0, y_offset=0):
        Wg, Wu, x, y_gate, y_up, routing = map(_buf, (Wg, Wu, x, y_gate, y_up, routing))
        self.ctx.call("zc_moe_fused_gate_up", quant_type, Wg.ptr, Wg.size, Wu.ptr, Wu.size, x.ptr, x.size,
                      y_gate.ptr, y_gate.size, y_up.ptr, y_up.size, routing.ptr, routing.size, M, K,
                      expert_stride, n_used, x_expert_stride, x_offset, y_offset)

    # the same with SwiGLU (or the GPT-OSS form) applied in the epilogue: one launch for the reference's
    # fused gate+up dispatch and its activation dispatch (forward.zig:6206-6240)
    def dispatchMoeFusedGateUpAct(self, quant_type, Wg, Wu, x, y, routing, M, K, expert_stride, n_used,
                                  x_expert_stride, oai=False, x_offset=0, y_offset=0):
        Wg, Wu, x, y, routing = map(_buf, (Wg, Wu, x, y, routing))
        self.ctx.call("zc_moe_fused_gate_up_act", quant_type, Wg.ptr, Wg.size, Wu.ptr, Wu.size, x.ptr, x.size,
                      y.ptr, y.size, routing.ptr, routing.size, M, K, expert_stride, n_used, x_expert_stride,
                      x_offset, y_offset, 1 if oai else 0)

    # One launch for the routed gate + up dispatch, the shared expert's gate + up (a slot with the id
    # SHARED_EXPERT), the per-expert gate / up biases and the activation (forward.zig:6206-6240, 6455-6500,
    # 6841-6849). shared = (gate, up) matrices or None; biases = (gate_bias, up_bias) [n_experts][M] or None.
    def dispatchMoeGateUpActEx(self, quant_type, Wg, Wu, x, y, routing, M, K, expert_stride, n_used, shared=None,
                               biases=None, oai=False, x_offset=0, y_offset=0):
        Wg, Wu, x, y, routing = map(_buf, (Wg, Wu, x, y, routing))
        none = Buffer(None, 0)
        sg, su = map(_buf, shared) if shared is not None else (none, none)
        bg, bu = map(_buf, biases) if biases is not None else (none, none)
        self.ctx.call("zc_moe_gate_up_act_ex", quant_type, Wg.ptr, Wg.size, Wu.ptr, Wu.size, sg.ptr, sg.size,
                      su.ptr, su.size, bg.ptr, bg.size, bu.ptr, bu.size, x.ptr, x.size, y.ptr, y.size,
                      routing.ptr, routing.size, M, K, expert_stride, n_used, x_offset, y_offset, 1 if oai else 0)

    # fused down + weighted accumulate with the shared expert's down matrix as one more slot and the per-expert
    # down bias inside the weighted sum (forward.zig:6362-6389, 6501-6545, 6923-6927)
    def dispatchMoeDownAccEx(self, quant_type, A, x, y, routing, M, K, expert_stride, n_used, x_expert_stride,
                             shared=None, bias=None, x_offset=0, y_offset=0):
        A, x, y, routing = map(_buf, (A, x, y, routing))
        none = Buffer(None, 0)
        sd = _buf(shared) if shared is not None else none
        bd = _buf(bias) if bias is not None else none
        self.ctx.call("zc_moe_down_acc_ex", quant_type, A.ptr, A.size, sd.ptr, sd.size, bd.ptr, bd.size, x.ptr,
                      x.size, y.ptr, y.size, routing.ptr, routing.size, M, K, expert_stride, n_used,
                      x_expert_stride, x_offset, y_offset)

    # router DMMV (optionally behind the RMS norm) + softmax_topk (+ the expert-parallel filter) in one launch
    # (forward.zig:6139-6190). routing = [k + shared_slot ids][k + shared_slot weights].
    def dispatchMoeRouterTopk(self, hidden, router_weights, logits, routing, n_experts, K, k,
                              rule=ROUTE_TOPK_THEN_SOFTMAX, bias=None, norm_weights=None, norm_out=None, eps=0.0,
                              shared_slot=False, routing_local=None, e_lo=0, e_hi=0, local_shared=False):
        h, w, lg, rt = map(_buf, (hidden, router_weights, logits, routing))
        none = Buffer(None, 0)
        b = _buf(bias) if bias is not None else none
        nw = _buf(norm_weights) if norm_weights is not None else none
        no = _buf(norm_out) if norm_out is not None else none
        rl = _buf(routing_local) if routing_local is not None else none
        self.ctx.call("zc_moe_router_topk", h.ptr, h.size, nw.ptr, nw.size, w.ptr, w.size, b.ptr, b.size, no.ptr,
                      no.size, lg.ptr, lg.size, rt.ptr, rt.size, rl.ptr, rl.size, n_experts, K, k, rule,
                      C.c_float(eps), 1 if shared_slot else 0, e_lo, e_hi if routing_local is not None else 0,
                      1 if local_shared else 0)

    # fused down + weighted accumulate (forward.zig:6362-6389)
    def dispatchMoeFusedDownAcc(self, quant_type, A, x, y, routing, M, K, expert_stride, n_used, x_expert_stride,
                                x_offset=0, y_offset=0):
        A, x, y, routing = map(_buf, (A, x, y, routing))
        self.ctx.call("zc_moe_fused_down_acc", quant_type, A.ptr, A.size, x.ptr, x.size, y.ptr, y.size,
                      routing.ptr, routing.size, M, K, expert_stride, n_used, x_expert_stride, x_offset, y_offset)

    # dispatchSoftmaxTopk (forward.zig:4135-4210) and the CPU routers (forward.zig:496-571)
    def dispatchSoftmaxTopk(self, logits, out, n_experts, k, rule=ROUTE_TOPK_THEN_SOFTMAX, n_tokens=1,
                            logits_stride=None, out_stride=None, bias=None):
        logits, out = _buf(logits), _buf(out)
        bias_ptr = _buf(bias).ptr if bias is not None else None
        self.ctx.call("zc_softmax_topk", logits.ptr, logits.size, bias_ptr, out.ptr, out.size, n_experts, k, rule,
                      n_tokens, n_experts if logits_stride is None else logits_stride,
                      2 * k if out_stride is None else out_stride)

    # fused RMS norm + f32 router DMMV (src/shaders/rms_norm_dmmv_f32.comp; src/compute/forward.zig:3469)
    def dispatchRmsNormDmmvF32(self, hidden, norm_weights, router_weights, norm_out, logits, M, K, eps):
        h, w, r, lg = _buf(hidden), _buf(norm_weights), _buf(router_weights), _buf(logits)
        no = _buf(norm_out) if norm_out is not None else Buffer(None, 0)
        self.ctx.call("zc_rms_norm_dmmv_f32", h.ptr, h.size, w.ptr, w.size, r.ptr, r.size, no.ptr, no.size,
                      lg.ptr, lg.size, M, K, C.c_float(eps))

    # dispatchDmmvOprojMerge (src/compute/forward.zig:8360-8411): split-K attention merge + O projection
    def dispatchDmmvOprojMerge(self, quant_type, o_tensor, partial_buf, sinks_buf, hidden_buf, M, K, n_heads,
                               n_i_chunks, sink_offset, head_dim, acc_mode=1, a_offset=0, y_offset=0):
        A, p, y = map(_buf, (o_tensor, partial_buf, hidden_buf))
        s = _buf(sinks_buf) if sinks_buf is not None else Buffer(None, 0)
        self.ctx.call("zc_dmmv_o_proj_merge", quant_type, A.ptr, A.size, p.ptr, p.size, y.ptr, y.size, s.ptr, s.size,
                      M, K, a_offset, y_offset, acc_mode, n_heads, n_i_chunks, sink_offset, head_dim)

    # fused RMS norm + alpha / beta SSM projections (src/shaders/rms_norm_dmmv_q4k_alpha_beta.comp)
    def dispatchRmsNormDmmvAlphaBeta(self, hidden, norm_weights, alpha_weights, beta_weights, norm_out, alpha_out,
                                     beta_out, M, K, eps):
        h, w, a, b, ao, bo = map(_buf, (hidden, norm_weights, alpha_weights, beta_weights, alpha_out, beta_out))
        no = _buf(norm_out) if norm_out is not None else Buffer(None, 0)
        self.ctx.call("zc_rms_norm_dmmv_alpha_beta", h.ptr, h.size, w.ptr, w.size, a.ptr, a.size, b.ptr, b.size,
                      no.ptr, no.size, ao.ptr, ao.size, bo.ptr, bo.size, M, K, C.c_float(eps))

    # dispatchMoeWeightedAcc (src/shaders/moe_weighted_acc.comp:23-33)
    def dispatchMoeWeightedAcc(self, a, b, routing, n, n_used, src_stride):
        a, b, routing = map(_buf, (a, b, routing))
        self.ctx.call("zc_moe_weighted_acc", a.ptr, a.size, b.ptr, b.size, routing.ptr, routing.size, n, n_used,
                      src_stride)

    # dispatchFfnActivation (forward.zig:3620-3727): swiglu / swiglu_oai
    def dispatchSwiglu(self, gate, up, y, n, oai=False):
        gate, up, y = map(_buf, (gate, up, y))
        need = n * 4
        if gate.size < need or up.size < need or y.size < need:
            raise InvalidArgument("dispatchSwiglu: buffer smaller than n floats")
        self.ctx.call("zc_swiglu_oai" if oai else "zc_swiglu", gate.ptr, up.ptr, y.ptr, n)

    # dispatchBiasAddSlice (forward.zig:3875-3913): out[i] += bias[element_offset + i]
    def dispatchBiasAddSlice(self, out, bias, element_offset, n_elements):
        out, bias = _buf(out), _buf(bias)
        self.ctx.call("zc_bias_add", out.ptr, out.size, bias.ptr, bias.size, n_elements, element_offset)

    # per-expert gate / up biases + activation for all selected slots (forward.zig:6841-6860)
    def dispatchMoeBiasAct(self, gate, up, gate_bias, up_bias, routing, y, M, n_used, n_experts, oai=False):
        gate, up, routing, y = map(_buf, (gate, up, routing, y))
        gb = _buf(gate_bias) if gate_bias is not None else Buffer(None, 0)
        ub = _buf(up_bias) if up_bias is not None else Buffer(None, 0)
        self.ctx.call("zc_moe_bias_act", gate.ptr, gate.size, up.ptr, up.size, gb.ptr, gb.size, ub.ptr, ub.size,
                      routing.ptr, routing.size, y.ptr, y.size, M, n_used, n_experts, 1 if oai else 0)

    # per-expert down bias inside the weighted sum (forward.zig:6923-6927)
    def dispatchMoeWeightedBiasAcc(self, a, bias, routing, n, n_used, n_experts):
        a, bias, routing = map(_buf, (a, bias, routing))
        self.ctx.call("zc_moe_weighted_bias_acc", a.ptr, a.size, bias.ptr, bias.size, routing.ptr, routing.size,
                      n, n_used, n_experts)

    # expert parallelism: keep (and renumber) the slots whose expert lies in [expert_lo, expert_hi)
    def dispatchMoeEpFilter(self, routing, out, k, expert_lo, expert_hi, n_tokens=1, routing_stride=None, out_stride=None):
        routing, out = _buf(routing), _buf(out)
        self.ctx.call("zc_moe_ep_filter", routing.ptr, routing.size, out.ptr, out.size, k, n_tokens,
                      2 * k if routing_stride is None else routing_stride, 2 * k if out_stride is None else out_stride,
                      expert_lo, expert_hi)

    # grouped-by-expert prefill helpers (src/shaders/metal/moe_route_pack.metal, moe_route_scatter.metal)
    def dispatchMoeRoutePack(self, routing, counts, ids, n_tokens, n_experts, k, routing_stride, ids_stride):
        routing, counts, ids = map(_buf, (routing, counts, ids))
        self.ctx.call("zc_moe_route_pack", routing.ptr, routing.size, counts.ptr, counts.size, ids.ptr, ids.size,
                      n_tokens, n_experts, k, routing_stride, ids_stride)

    def dispatchMoeRouteScatter(self, routing, src, dst, n_tokens, hidden_dim, k, routing_stride):
        routing, src, dst = map(_buf, (routing, src, dst))
        self.ctx.call("zc_moe_route_scatter", routing.ptr, routing.size, src.ptr, src.size, dst.ptr, dst.size,
                      n_tokens, hidden_dim, k, routing_stride)

    # dequantRow on the device (forward.zig:242-465), bit-exact
    def dequantRows(self, quant_type, A, out, first_row, n_rows, K, a_offset=0):
        A, out = _buf(A), _buf(out)
        self.ctx.call("zc_dequant_rows", quant_type, A.ptr, A.size, out.ptr, out.size, first_row, n_rows, K,
                      a_offset)
