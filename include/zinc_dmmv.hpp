// C++ host mirror of the reference's DMMV dispatch layer (DmmvDispatch, src/compute/dmmv.zig:305-1098)
// over the C ABI of zinc_cuda.h. Header-only; link against libzinc_b200.so.
//
// The method names, argument order, units and error cases are the reference's:
//   * offsets a_offset / x_offset / y_offset and expert_stride are in bytes, x_expert_stride and the
//     token strides in elements (src/compute/dmmv.zig:21-66);
//   * error.UnsupportedQuantType / error.PipelineNotLoaded / error.InvalidArgument become
//     zinc::Error values (returned, never thrown; zinc::check() turns them into exceptions);
//   * what the reference binds through a descriptor set (a buffer handle plus its size) is a
//     zinc::Buffer {device pointer, size in bytes} here, in the reference's binding order A, x, y(, routing);
//   * the command buffer `cmd` of the reference is the context's stream: calls are enqueued in order.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>

#include "zinc_cuda.h"

namespace zinc {

enum class Error : int32_t {
    None = ZC_OK,
    UnsupportedQuantType = ZC_ERR_UNSUPPORTED_TYPE,  // error.UnsupportedQuantType
    PipelineNotLoaded = ZC_ERR_NOT_LOADED,           // error.PipelineNotLoaded
    InvalidArgument = ZC_ERR_INVALID_ARG,            // error.InvalidArgument
    OutOfMemory = ZC_ERR_OOM,
    CudaFailure = ZC_ERR_CUDA,
    DeviceTimeout = ZC_ERR_TIMEOUT,
};

// GGMLType ids the path supports (src/model/gguf.zig:38-69)
enum class GGMLType : uint32_t {
    f32 = ZC_F32, f16 = ZC_F16, q5_0 = ZC_Q5_0, q5_1 = ZC_Q5_1, q8_0 = ZC_Q8_0,
    q4_k = ZC_Q4_K, q5_k = ZC_Q5_K, q6_k = ZC_Q6_K, bf16 = ZC_BF16, mxfp4 = ZC_MXFP4,
};

struct Buffer {
    void* ptr = nullptr;
    uint64_t size = 0;
};

// Push-constant blocks of the reference, kept as plain structs so call sites port 1:1.
struct DmmvPushConstants {  // src/compute/dmmv.zig:21-28
    uint32_t M, K, a_offset, x_offset, y_offset, acc_mode = 0;
};
struct BatchDmmvPushConstants {  // src/compute/dmmv.zig:31-38
    uint32_t M, K, a_offset, x_offset, y_offset, num_cols;
};
struct MoeDmmvPushConstants {  // src/compute/dmmv.zig:42-49
    uint32_t M, K, expert_stride, x_expert_stride, x_offset, y_offset;
};
struct MoeBatchedDmmvPushConstants {  // src/compute/dmmv.zig:55-62
    uint32_t M, K, expert_stride, n_experts_used, x_token_stride, y_token_stride;
};
struct OprojMergePushConstants {  // src/compute/dmmv.zig:76-93
    uint32_t M, K, a_offset = 0, x_offset = 0, y_offset = 0, acc_mode = 1, n_heads, n_i_chunks, sink_offset, head_dim;
};

class DmmvDispatch {
public:
    // DmmvDispatch.init (src/compute/dmmv.zig:305): one device, one in-order stream
    static Error init(int device, DmmvDispatch& out) {
        out.deinit();
        return static_cast<Error>(zc_init(device, &out.ctx_));
    }
    DmmvDispatch() = default;
    DmmvDispatch(const DmmvDispatch&) = delete;
    DmmvDispatch& operator=(const DmmvDispatch&) = delete;
    ~DmmvDispatch() { deinit(); }
    void deinit() {  // src/compute/dmmv.zig:1098
        if (ctx_) zc_destroy(ctx_);
        ctx_ = nullptr;
    }

    zc_ctx* context() const { return ctx_; }
    std::string lastError() const { return ctx_ ? zc_last_error(ctx_) : "no context"; }
    Error setStream(void* cuda_stream) { return static_cast<Error>(zc_set_stream(ctx_, cuda_stream)); }

    // pipelineForType / moePipelineForType (src/compute/dmmv.zig:678-703): false <=> the reference returns null
    static bool pipelineForType(GGMLType t) { return zc_dmmv_supported(static_cast<uint32_t>(t)) != 0; }
    static bool moePipelineForType(GGMLType t) { return zc_moe_dmmv_supported(static_cast<uint32_t>(t)) != 0; }

    // recordDispatch (src/compute/dmmv.zig:806-874); acc_mode as in DmmvPushConstants
    Error recordDispatch(GGMLType quant_type, Buffer A, Buffer x, Buffer y, uint32_t M, uint32_t K, uint32_t a_offset,
                         uint32_t x_offset, uint32_t y_offset, uint32_t acc_mode = 0) {
        return static_cast<Error>(zc_dmmv(ctx_, static_cast<uint32_t>(quant_type), A.ptr, A.size, x.ptr, x.size, y.ptr,
                                          y.size, M, K, a_offset, x_offset, y_offset, acc_mode));
    }
    Error recordDispatch(GGMLType quant_type, Buffer A, Buffer x, Buffer y, const DmmvPushConstants& pc) {
        return recordDispatch(quant_type, A, x, y, pc.M, pc.K, pc.a_offset, pc.x_offset, pc.y_offset, pc.acc_mode);
    }

    // The fused split-K attention merge + O projection dispatch (src/compute/forward.zig:8360-8411): bindings
    // W_o, partials (+ LSE region), hidden, sinks (an empty Buffer: no sinks)
    Error recordOprojMerge(GGMLType quant_type, Buffer o_tensor, Buffer partial_buf, Buffer hidden_buf, Buffer sinks_buf,
                           const OprojMergePushConstants& pc) {
        return static_cast<Error>(zc_dmmv_o_proj_merge(
            ctx_, static_cast<uint32_t>(quant_type), o_tensor.ptr, o_tensor.size, partial_buf.ptr, partial_buf.size,
            hidden_buf.ptr, hidden_buf.size, sinks_buf.ptr, sinks_buf.size, pc.M, pc.K, pc.a_offset, pc.y_offset,
            pc.acc_mode, pc.n_heads, pc.n_i_chunks, pc.sink_offset, pc.head_dim));
    }

    // recordBatchDispatchPush (src/compute/dmmv.zig:880-926)
    Error recordBatchDispatchPush(GGMLType quant_type, Buffer a_buf, Buffer x_buf, Buffer y_buf, uint32_t M, uint32_t K,
                                  uint32_t a_offset, uint32_t x_offset, uint32_t y_offset, uint32_t num_cols) {
        return static_cast<Error>(zc_dmmv_batch(ctx_, static_cast<uint32_t>(quant_type), a_buf.ptr, a_buf.size,
                                                x_buf.ptr, x_buf.size, y_buf.ptr, y_buf.size, M, K, a_offset, x_offset,
                                                y_offset, num_cols));
    }

    // recordMoeDispatch (src/compute/dmmv.zig:709-739); bindings A, x, y, routing
    Error recordMoeDispatch(GGMLType quant_type, Buffer A, Buffer x, Buffer y, Buffer routing, uint32_t M, uint32_t K,
                            uint32_t expert_stride, uint32_t n_experts_y, uint32_t x_expert_stride, uint32_t x_offset,
                            uint32_t y_offset) {
        return static_cast<Error>(zc_moe_dmmv(ctx_, static_cast<uint32_t>(quant_type), A.ptr, A.size, x.ptr, x.size,
                                              y.ptr, y.size, routing.ptr, routing.size, M, K, expert_stride,
                                              n_experts_y, x_expert_stride, x_offset, y_offset));
    }

    // recordMoeBatchedDispatch (src/compute/dmmv.zig:746-792)
    Error recordMoeBatchedDispatch(GGMLType quant_type, Buffer a_buf, Buffer x_buf, Buffer y_buf, Buffer routing_buf,
                                   uint32_t M, uint32_t K, uint32_t expert_stride, uint32_t n_experts,
                                   uint32_t n_experts_used, uint32_t n_tokens, uint32_t x_token_stride,
                                   uint32_t y_token_stride) {
        return static_cast<Error>(zc_moe_dmmv_batched(ctx_, static_cast<uint32_t>(quant_type), a_buf.ptr, a_buf.size,
                                                      x_buf.ptr, x_buf.size, y_buf.ptr, y_buf.size, routing_buf.ptr,
                                                      routing_buf.size, M, K, expert_stride, n_experts, n_experts_used,
                                                      n_tokens, x_token_stride, y_token_stride));
    }

    // Gate and up of a prefill batch on one grouping (no single counterpart in the reference: two
    // recordMoeBatchedDispatch calls, src/compute/dmmv.zig:746-792)
    Error recordMoeBatchedDispatchPair(GGMLType quant_type, Buffer wg_buf, Buffer wu_buf, Buffer x_buf, Buffer yg_buf,
                                       Buffer yu_buf, Buffer routing_buf, uint32_t M, uint32_t K, uint32_t expert_stride,
                                       uint32_t n_experts, uint32_t n_experts_used, uint32_t n_tokens,
                                       uint32_t x_token_stride, uint32_t y_token_stride) {
        return static_cast<Error>(zc_moe_dmmv_batched_pair(
            ctx_, static_cast<uint32_t>(quant_type), wg_buf.ptr, wg_buf.size, wu_buf.ptr, wu_buf.size, x_buf.ptr,
            x_buf.size, yg_buf.ptr, yg_buf.size, yu_buf.ptr, yu_buf.size, routing_buf.ptr, routing_buf.size, M, K,
            expert_stride, n_experts, n_experts_used, n_tokens, x_token_stride, y_token_stride));
    }

    // Lend the library scratch for the grouped-by-expert prefill form of recordMoeBatchedDispatch (no
    // counterpart in the reference's DmmvDispatch; its Metal path owns route_ids / route_counts buffers).
    // An empty Buffer removes it.
    Error setWorkspace(Buffer workspace) {
        return static_cast<Error>(zc_set_workspace(ctx_, workspace.ptr, workspace.size));
    }
    static uint64_t moeGroupedWorkspaceBytes(uint32_t n_tokens, uint32_t n_experts_used, uint32_t K, uint32_t n_experts) {
        return zc_moe_grouped_workspace_bytes(n_tokens, n_experts_used, K, n_experts);
    }

    // recordCountExperts (src/compute/dmmv.zig:981-1028)
    Error recordCountExperts(Buffer routing_buf, Buffer counts_buf, uint32_t n_tokens, uint32_t n_layers, uint32_t layer,
                             uint32_t n_experts_used, uint32_t n_experts, uint64_t d_offset_bytes) {
        return static_cast<Error>(zc_count_experts(ctx_, routing_buf.ptr, routing_buf.size, counts_buf.ptr,
                                                   counts_buf.size, n_tokens, n_layers, layer, n_experts_used, n_experts,
                                                   d_offset_bytes));
    }

    // recordMulMmQ4K (src/compute/dmmv.zig:1045-1094): f32 activations, offsets in elements of B and D
    Error recordMulMmQ4K(Buffer a_buf, Buffer b_buf, Buffer d_buf, uint32_t M, uint32_t N, uint32_t K, uint32_t stride_b,
                         uint32_t stride_d, uint32_t a_offset, uint32_t b_offset, uint32_t d_offset) {
        return recordMulMm(GGMLType::q4_k, a_buf, b_buf, d_buf, M, N, K, stride_b, stride_d, a_offset, b_offset, d_offset,
                           GGMLType::f32);
    }
    // the same for any weight type and bf16 activations (the tensor-core path)
    Error recordMulMm(GGMLType quant_type, Buffer a_buf, Buffer b_buf, Buffer d_buf, uint32_t M, uint32_t N, uint32_t K,
                      uint32_t stride_b, uint32_t stride_d, uint64_t a_offset, uint64_t b_offset, uint64_t d_offset,
                      GGMLType act_type) {
        return static_cast<Error>(zc_mul_mm(ctx_, static_cast<uint32_t>(quant_type), a_buf.ptr, a_buf.size, b_buf.ptr,
                                            b_buf.size, d_buf.ptr, d_buf.size, M, N, K, stride_b, stride_d, a_offset,
                                            b_offset, d_offset, static_cast<uint32_t>(act_type)));
    }

    // computeBarrier / submitAndWait of the command buffer (src/vulkan/command.zig:345, 477)
    Error computeBarrier() { return static_cast<Error>(zc_barrier(ctx_)); }
    Error submitAndWait() { return static_cast<Error>(zc_submit_and_wait(ctx_)); }

private:
    zc_ctx* ctx_ = nullptr;
};

// Zig's `try`: throw on any error, with the library's message.
inline void check(Error e, const DmmvDispatch& d) {
    if (e != Error::None) throw std::runtime_error("zinc_b200: " + d.lastError());
}

}  // namespace zinc
