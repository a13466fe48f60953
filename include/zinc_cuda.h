/*
 * zinc_cuda.h - C ABI of the B200 (sm_100a) quantized-matmul library for the
 * ZINC inference engine's compute-op interface.
 *
 * The library replaces the engine's DMMV dispatch layer and the kernels
 * behind it: the decode dequant-matvec over GGUF blocks, the batched-prefill
 * dequant-GEMM, the MoE expert matmuls and the routing / activation / combine
 * steps either side of them. Every entry point below names the reference
 * interface it stands in for, as <path in the reference project>:<lines>.
 *
 * Conventions (shared by all entry points)
 *  - Every pointer named A, x, y, X, Y, routing, ... is a DEVICE pointer owned
 *    by the caller; the library borrows it for the call and never frees it.
 *    `*_size` is the byte size of the caller's buffer behind that pointer and
 *    is used for bounds validation only (the role of the descriptor range in
 *    the reference).
 *  - Offsets keep the reference's units: a_offset / x_offset / y_offset and
 *    expert_stride are BYTES, x_expert_stride and token strides are ELEMENTS
 *    (src/compute/dmmv.zig:21-62, 801-803). They are widened to 64 bit.
 *  - Weight layout is the raw GGUF block stream, row-major by output row,
 *    K/block_size blocks per row (src/model/gguf.zig:75-122).
 *  - Work is enqueued on the context's CUDA stream in call order, so a later
 *    call sees the results of an earlier one; nothing is guaranteed complete
 *    until zc_submit_and_wait returns (record / submit model of
 *    src/vulkan/command.zig:222-320, 477).
 *  - Every function returns a zc_status. No exception crosses the ABI. A
 *    context is thread-compatible, not thread-safe (one recording thread, as
 *    in the reference).
 *  - There is no CPU fallback: a call on a machine without a usable CUDA
 *    device fails with ZC_ERR_CUDA.
 */
#ifndef ZINC_CUDA_H
#define ZINC_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error model. Mirrors the Zig error set of the dispatch layer:
 * error.UnsupportedQuantType (src/compute/dmmv.zig:722, 822, 899-901),
 * error.PipelineNotLoaded (766, 943, 1000, 1064), error.InvalidArgument
 * (767, 944, 1001-1006, 1065-1066). */
typedef enum zc_status {
    ZC_OK = 0,
    ZC_ERR_UNSUPPORTED_TYPE = 1,
    ZC_ERR_NOT_LOADED = 2,
    ZC_ERR_INVALID_ARG = 3,
    ZC_ERR_OOM = 4,
    ZC_ERR_CUDA = 5,
    ZC_ERR_TIMEOUT = 6
} zc_status;

/* GGML tensor type ids (src/model/gguf.zig:38-69). */
typedef enum zc_type {
    ZC_F32 = 0,
    ZC_F16 = 1,
    ZC_Q5_0 = 6,
    ZC_Q5_1 = 7,
    ZC_Q8_0 = 8,
    ZC_Q4_K = 12,
    ZC_Q5_K = 13,
    ZC_Q6_K = 14,
    ZC_BF16 = 30,
    ZC_MXFP4 = 39
} zc_type;

/* MoE routing rules (src/compute/forward.zig:496-571). Both select the k
 * largest logits (ties to the lowest index) and give softmax weights over the
 * selected set; they differ only in rounding order. */
typedef enum zc_routing_rule {
    ZC_ROUTE_SOFTMAX_ALL_RENORM = 0, /* topKSoftmax: softmax over all, pick, renormalise */
    ZC_ROUTE_TOPK_THEN_SOFTMAX = 1   /* topKSoftmaxWeight / softmax_topk.comp */
} zc_routing_rule;

typedef struct zc_ctx zc_ctx;

/* ---- context ------------------------------------------------------------
 * Replaces Instance.init + DmmvDispatch.init / deinit
 * (src/compute/dmmv.zig:305-671, 1098-1129). */
int32_t zc_init(int32_t device, zc_ctx** out_ctx);
int32_t zc_destroy(zc_ctx* ctx);
/* Use a caller-owned cudaStream_t (e.g. the framework's current stream); NULL is
 * CUDA's default stream. zc_use_own_stream goes back to the stream the context
 * created for itself (the initial state). */
int32_t zc_set_stream(zc_ctx* ctx, void* cuda_stream);
int32_t zc_use_own_stream(zc_ctx* ctx);
void* zc_get_stream(zc_ctx* ctx);
/* Text of the last error recorded on this context (never NULL). */
const char* zc_last_error(zc_ctx* ctx);
const char* zc_status_string(int32_t status);
/* Number of kernels this context has launched so far. */
uint64_t zc_launch_count(zc_ctx* ctx);

/* ---- buffers --------------------------------------------------------------
 * Replaces Buffer.initDeviceLocal / initStaging / upload
 * (src/vulkan/buffer.zig:102-149). Optional: any device pointer works. */
int32_t zc_alloc(zc_ctx* ctx, uint64_t bytes, void** out_dptr);
int32_t zc_free(zc_ctx* ctx, void* dptr);
int32_t zc_upload(zc_ctx* ctx, void* dst, uint64_t dst_offset, const void* host_src, uint64_t bytes);
int32_t zc_download(zc_ctx* ctx, void* host_dst, const void* src, uint64_t src_offset, uint64_t bytes);
int32_t zc_memset(zc_ctx* ctx, void* dst, uint64_t dst_offset, int32_t byte_value, uint64_t bytes);

/* ---- ordering ---------------------------------------------------------------
 * zc_barrier replaces computeBarrier / computeBufferBarrier
 * (src/vulkan/command.zig:345-425): a CUDA stream is already ordered, so it
 * only exists to let call sites port one to one. zc_submit_and_wait replaces
 * submitAndWait (src/vulkan/command.zig:477): it blocks until the stream is
 * idle and returns the first deferred device-side error, if any. */
int32_t zc_barrier(zc_ctx* ctx);
int32_t zc_submit_and_wait(zc_ctx* ctx);
/* Device-side errors are deferred to zc_submit_and_wait, as the reference's are to submitAndWait:
 *  - a bounded wait inside a kernel gave up (a split-K hand-off or a peer's flag): ZC_ERR_TIMEOUT. The
 *    results of the calls since the last zc_submit_and_wait are invalid; the context stays usable (its
 *    hand-off flags are cleared), a communicator whose exchange gave up refuses further collectives
 *    until zc_comm_destroy + zc_comm_init on every rank;
 *  - a routing buffer named an expert the weight buffer does not hold: ZC_ERR_INVALID_ARG (the id is
 *    replaced by expert 0 or the pair is skipped, so no kernel reads outside the buffer).
 * zc_set_wait_limit sets the number of polls after which such a wait gives up (0 = the defaults,
 * 2^26 for split-K hand-offs and 2^24 for peer flags, i.e. seconds). No counterpart in the reference
 * (Vulkan reports a lost device instead). */
int32_t zc_set_wait_limit(zc_ctx* ctx, uint32_t polls);

/* ---- pre-recorded op sequences ----------------------------------------------
 * The reference records a token's dispatches into a command buffer and
 * submits it once (src/vulkan/command.zig:222-320, 477). The counterpart here
 * is a CUDA graph: calls made between zc_begin_record and zc_end_record are
 * captured instead of executed; zc_replay enqueues the whole sequence with one
 * launch. Buffers, sizes and offsets are baked in at record time. Host copies
 * recorded this way must use page-locked host memory. */
int32_t zc_begin_record(zc_ctx* ctx);
int32_t zc_end_record(zc_ctx* ctx, void** out_recording);
int32_t zc_replay(zc_ctx* ctx, void* recording);
int32_t zc_free_recording(zc_ctx* ctx, void* recording);

/* ---- layout helpers ---------------------------------------------------------
 * GGMLType.blockSize / bytesPerBlock (src/model/gguf.zig:75-122),
 * TensorInfo.sizeBytes (src/model/gguf.zig:222-229),
 * expertSliceBytes (src/compute/forward.zig:650-656). */
uint32_t zc_block_size(uint32_t type);
uint32_t zc_bytes_per_block(uint32_t type);
uint64_t zc_tensor_size_bytes(uint32_t type, uint64_t n_elements);
uint64_t zc_expert_slice_bytes(uint32_t type, uint32_t rows, uint32_t cols);
/* 1 if the type has a DMMV kernel: pipelineForType (src/compute/dmmv.zig:678-691). */
int32_t zc_dmmv_supported(uint32_t type);
/* 1 if the type has a MoE DMMV kernel: moePipelineForType (src/compute/dmmv.zig:694-703). */
int32_t zc_moe_dmmv_supported(uint32_t type);

/* ---- decode matvec ------------------------------------------------------------
 * y[M] (+)= W[M x K] . x[K].  acc_mode 0: y = result, 1: y += result.
 * Replaces DmmvDispatch.recordDispatch (src/compute/dmmv.zig:806-874) together
 * with the variant policy of dispatchDmmvInner (src/compute/forward.zig:8414-8540):
 * the tall-M and batch-shader special cases there are an internal choice here.
 * Types: q4_k, q5_k, q6_k, q8_0, mxfp4, q5_0, q5_1, f16, f32; any other type
 * returns ZC_ERR_UNSUPPORTED_TYPE. K must be a multiple of the block size;
 * x + x_offset must be 16-byte aligned (src/shaders/dmmv_q6k.comp:24-27). */
int32_t zc_dmmv(zc_ctx* ctx, uint32_t type,
                const void* A, uint64_t a_size, const void* x, uint64_t x_size,
                void* y, uint64_t y_size,
                uint32_t M, uint32_t K,
                uint64_t a_offset, uint64_t x_offset, uint64_t y_offset, uint32_t acc_mode);

/* Fused RMS norm + f32 router matvec (src/shaders/rms_norm_dmmv_f32.comp:68-127, push block
 * RmsNormDmmvF32Push src/compute/elementwise.zig:177-181): rms_inv = 1/sqrt(mean(hidden^2) + eps),
 * norm_out[i] = norm_weights[i] * (hidden[i] * rms_inv) (optional; must not alias hidden),
 * logits[m] = sum_i router_weights[m][i] * norm_out[i]. All f32; K a multiple of 4. */
int32_t zc_rms_norm_dmmv_f32(zc_ctx* ctx, const void* hidden, uint64_t hidden_size,
                             const void* norm_weights, uint64_t norm_size,
                             const void* router_weights, uint64_t router_size,
                             void* norm_out, uint64_t norm_out_size,
                             void* logits, uint64_t logits_size,
                             uint32_t M, uint32_t K, float eps);

/* The same with two M x K f32 matrices on one normalised vector, one launch: alpha_out = W_alpha xn,
 * beta_out = W_beta xn, xn also written to norm_out when given. Replaces the fused RMS norm + alpha / beta
 * SSM projection dispatch (src/shaders/rms_norm_dmmv_q4k_alpha_beta.comp:64-133; f32 weights, as its callers
 * ship them). */
int32_t zc_rms_norm_dmmv_alpha_beta(zc_ctx* ctx, const void* hidden, uint64_t hidden_size,
                                    const void* norm_weights, uint64_t norm_size,
                                    const void* alpha_weights, uint64_t alpha_size,
                                    const void* beta_weights, uint64_t beta_size,
                                    void* norm_out, uint64_t norm_out_size,
                                    void* alpha_out, uint64_t alpha_out_size,
                                    void* beta_out, uint64_t beta_out_size,
                                    uint32_t M, uint32_t K, float eps);

/* Grouped matvec: y_i (+)= W_i x for n = 1..3 matrices of one type that share x and K, e.g. the Q, K
 * and V projections the reference records as three dispatches on the same input
 * (src/compute/forward.zig:4530-4564). One kernel launch when the matrices are Q4_K (16-byte aligned);
 * otherwise the same result through one launch per matrix. Arguments are those of zc_dmmv, per matrix
 * in arrays of length n. */
int32_t zc_dmmv_multi(zc_ctx* ctx, uint32_t quant_type, uint32_t n,
                      const void* const* A, const uint64_t* a_size, const uint64_t* a_offset,
                      const void* x, uint64_t x_size, uint64_t x_offset,
                      void* const* y, const uint64_t* y_size, const uint64_t* y_offset,
                      const uint32_t* M, uint32_t K, uint32_t acc_mode);

/* out[r] = silu(Wg[r].x) * (Wu[r].x), one pass over both weight streams.
 * Replaces dispatchDmmvFusedGateUpSwiglu and its Q8_0 sibling
 * (src/compute/forward.zig:8237-8313; src/shaders/dmmv_q4k_fused_gate_up_swiglu.comp:195-218).
 * Gate and up must share `type`. The reference has q4_k and q8_0 only; every
 * DMMV type is accepted here. */
int32_t zc_dmmv_fused_gate_up_swiglu(zc_ctx* ctx, uint32_t type,
                                     const void* Wg, uint64_t wg_size, const void* Wu, uint64_t wu_size,
                                     const void* x, uint64_t x_size, void* out, uint64_t out_size,
                                     uint32_t M, uint32_t K,
                                     uint64_t gate_offset, uint64_t up_offset,
                                     uint64_t x_offset, uint64_t out_offset);

/* y[r] += sigmoid(gate[gate_index]) * (W[r].x).  Replaces dispatchDmmvQ8_0SigmoidAcc
 * (src/compute/forward.zig:8321-8359; src/compute/dmmv.zig:101-108;
 * src/shaders/dmmv_q8_0_sigmoid_acc.comp:95-132). `gate_index` counts f32
 * elements. The reference has q8_0 only; every DMMV type is accepted. */
int32_t zc_dmmv_sigmoid_acc(zc_ctx* ctx, uint32_t type,
                            const void* A, uint64_t a_size, const void* x, uint64_t x_size,
                            void* y, uint64_t y_size, const void* gate, uint64_t gate_size,
                            uint32_t M, uint32_t K,
                            uint64_t a_offset, uint64_t x_offset, uint64_t y_offset, uint32_t gate_index);

/* ---- batched prefill -------------------------------------------------------------
 * Y[c][M] = W . X[c][K] for c < num_cols; X is [num_cols][K] f32, Y is
 * [num_cols][M] f32 (src/compute/forward.zig:8141-8146). Replaces
 * recordBatchDispatchPush (src/compute/dmmv.zig:880-926) and the 40-column
 * chunk loop of dispatchProjectionBatched (src/compute/forward.zig:8147-8216):
 * num_cols is unbounded and chunking is internal. The reference supports q4_k
 * and q6_k; every K-quant and 32-block type is accepted. */
int32_t zc_dmmv_batch(zc_ctx* ctx, uint32_t type,
                      const void* A, uint64_t a_size, const void* X, uint64_t x_size,
                      void* Y, uint64_t y_size,
                      uint32_t M, uint32_t K,
                      uint64_t a_offset, uint64_t x_offset, uint64_t y_offset, uint32_t num_cols);

/* Tiled dequant-GEMM on the tensor cores: D[col][row] = sum_k A[row][k] B[col][k].
 * Replaces recordMulMmQ4K (src/compute/dmmv.zig:1045-1094; src/shaders/mul_mm_q4k.comp:74-243)
 * and the Metal tiled GEMMs (src/shaders/metal/gemm_q4k.metal:54-225, gemm_q6k.metal:38-68).
 * B and D are column-major with element strides stride_b / stride_d; b_offset
 * and d_offset count ELEMENTS, a_offset BYTES (src/compute/dmmv.zig:139-145).
 * act_type selects B's element type, ZC_F32 or ZC_BF16; D is f32. bf16 activations with Q4_K, Q6_K or
 * MXFP4 weights (A and B 16-byte aligned, N >= 16, stride_b a multiple of 8; MXFP4: K a multiple of 64)
 * run on the tensor cores: weights dequantised to bf16 tiles (exactly, for MXFP4), f32 accumulation in
 * tensor memory. Every other combination (f32 activations included, which keep f32 precision) runs a
 * CUDA-core kernel.
 * K must be a multiple of 256 for K-quants (InvalidArgument otherwise, as the reference). */
int32_t zc_mul_mm(zc_ctx* ctx, uint32_t type,
                  const void* A, uint64_t a_size, const void* B, uint64_t b_size,
                  void* D, uint64_t d_size,
                  uint32_t M, uint32_t N, uint32_t K,
                  uint32_t stride_b, uint32_t stride_d,
                  uint64_t a_offset, uint64_t b_offset, uint64_t d_offset, uint32_t act_type);

/* ---- MoE expert matvecs ---------------------------------------------------------------
 * For slot s < n_used: e = routing[s]; Y[s][M] = W[e] . X[s*x_expert_stride .. +K].
 * x_expert_stride 0 = all slots share x. routing holds u32 expert ids first
 * (src/shaders/softmax_topk.comp:19-22). Replaces recordMoeDispatch
 * (src/compute/dmmv.zig:709-739) and the per-type MoE shaders
 * (src/shaders/dmmv_q4k_moe_kpar.comp:56-175 and siblings). */
int32_t zc_moe_dmmv(zc_ctx* ctx, uint32_t type,
                    const void* A, uint64_t a_size, const void* x, uint64_t x_size,
                    void* y, uint64_t y_size, const void* routing, uint64_t routing_size,
                    uint32_t M, uint32_t K,
                    uint64_t expert_stride, uint32_t n_used, uint32_t x_expert_stride,
                    uint64_t x_offset, uint64_t y_offset);

/* Gate and up for the same slots in one pass: Yg[s] = Wg[e].x, Yu[s] = Wu[e].x.
 * Replaces the fused gate+up MoE dispatch
 * (src/shaders/dmmv_q4k_fused_gate_up_moe.comp:77-217; src/compute/forward.zig:6206-6222). */
int32_t zc_moe_fused_gate_up(zc_ctx* ctx, uint32_t type,
                             const void* Wg, uint64_t wg_size, const void* Wu, uint64_t wu_size,
                             const void* x, uint64_t x_size,
                             void* y_gate, uint64_t yg_size, void* y_up, uint64_t yu_size,
                             const void* routing, uint64_t routing_size,
                             uint32_t M, uint32_t K,
                             uint64_t expert_stride, uint32_t n_used, uint32_t x_expert_stride,
                             uint64_t x_offset, uint64_t y_offset);

/* The same with the activation applied in the kernel's epilogue: y[s][r] = silu(Wg[e].x) * (Wu[e].x)
 * (oai = 0, src/shaders/swiglu.comp:25-33) or the GPT-OSS form (oai = 1, src/shaders/swiglu_oai.comp:24-34).
 * One launch instead of the reference's fused gate+up dispatch followed by its activation dispatch
 * (src/compute/forward.zig:6206-6240); results are those of zc_moe_fused_gate_up + zc_swiglu(_oai).
 * Measured on B200 the single launch is not faster than the two (the decode benchmark keeps the two). */
int32_t zc_moe_fused_gate_up_act(zc_ctx* ctx, uint32_t type,
                                 const void* Wg, uint64_t wg_size, const void* Wu, uint64_t wu_size,
                                 const void* x, uint64_t x_size, void* y, uint64_t y_size,
                                 const void* routing, uint64_t routing_size,
                                 uint32_t M, uint32_t K,
                                 uint64_t expert_stride, uint32_t n_used, uint32_t x_expert_stride,
                                 uint64_t x_offset, uint64_t y_offset, uint32_t oai);

/* hidden[r] += sum_{s<n_used} w_s * (W[id_s][r] . X[s*x_expert_stride ..]);
 * routing = [n_used ids u32][n_used weights f32 bits]. Replaces the fused
 * down + weighted-accumulate dispatch (src/compute/dmmv.zig:68-76;
 * src/shaders/dmmv_q4k_moe_fused_down_acc.comp:74-177). */
int32_t zc_moe_fused_down_acc(zc_ctx* ctx, uint32_t type,
                              const void* A, uint64_t a_size, const void* x, uint64_t x_size,
                              void* y, uint64_t y_size, const void* routing, uint64_t routing_size,
                              uint32_t M, uint32_t K,
                              uint64_t expert_stride, uint32_t n_used, uint32_t x_expert_stride,
                              uint64_t x_offset, uint64_t y_offset);

/* The O projection fed directly from split-K flash-attention partials: x[head * head_dim + d] =
 * (sum_c w_c * partial[(head * n_i_chunks + c) * head_dim + d]) / L with w_c = exp(M_c - M) for chunks whose sum
 * L_c is positive, M the maximum over the chunks' maxima and the head's sink (sinks[sink_offset + head]; NaN or a
 * NULL sinks pointer: none), L = sum_c w_c L_c (+ exp(sink - M)); the pairs {M_c, L_c} follow the partials at
 * float index n_heads * n_i_chunks * head_dim. Then y = A x (+ y when acc_mode != 0). K = n_heads * head_dim,
 * n_i_chunks <= 16. Replaces the fused merge + O projection dispatch and its push block
 * (src/compute/dmmv.zig:76-93 OprojMergePushConstants; src/compute/forward.zig:8360-8411;
 * src/shaders/dmmv_q4k_o_proj_merge.comp:96-250). One launch for Q4_K matrices of at least 2 MB with at most four
 * chunks and head_dim a multiple of 8 (the vector is merged while the matvec loads it); otherwise a small merge
 * kernel runs first. Any DMMV type. */
int32_t zc_dmmv_o_proj_merge(zc_ctx* ctx, uint32_t type,
                             const void* A, uint64_t a_size,
                             const void* partial, uint64_t partial_size,
                             void* y, uint64_t y_size,
                             const void* sinks, uint64_t sinks_size,
                             uint32_t M, uint32_t K, uint64_t a_offset, uint64_t y_offset, uint32_t acc_mode,
                             uint32_t n_heads, uint32_t n_i_chunks, uint32_t sink_offset, uint32_t head_dim);

/* Routing id that selects the shared expert: a matrix outside the expert stack, passed beside it to the two
 * calls below. It lets the always-on expert of a layer (src/compute/forward.zig:6455-6545 runs it as separate
 * dispatches after the routed ones) ride in the routed launches as one more slot with weight 1. */
#define ZC_SHARED_EXPERT 0xFFFFFFFEu

/* zc_moe_fused_gate_up_act with, all optional (NULL / 0): the shared expert's gate and up matrices [M][K] of the
 * same type, selected by a slot whose id is ZC_SHARED_EXPERT; and per-expert f32 biases [n_experts][M] added to
 * the gate and up rows before the activation (src/compute/forward.zig:6841-6849, ffn_gate_exps_bias /
 * ffn_up_exps_bias), never to the shared slot. x is shared by the slots. One launch replaces the routed
 * gate + up dispatch, the shared expert's gate + up dispatch, the bias adds and the activation. */
int32_t zc_moe_gate_up_act_ex(zc_ctx* ctx, uint32_t type,
                              const void* Wg, uint64_t wg_size, const void* Wu, uint64_t wu_size,
                              const void* shared_gate, uint64_t shared_gate_size,
                              const void* shared_up, uint64_t shared_up_size,
                              const void* gate_bias, uint64_t gate_bias_size,
                              const void* up_bias, uint64_t up_bias_size,
                              const void* x, uint64_t x_size, void* y, uint64_t y_size,
                              const void* routing, uint64_t routing_size,
                              uint32_t M, uint32_t K, uint64_t expert_stride, uint32_t n_used,
                              uint64_t x_offset, uint64_t y_offset, uint32_t oai);

/* zc_moe_fused_down_acc with, both optional: the shared expert's down matrix [M][K] (slot id ZC_SHARED_EXPERT,
 * weighted by the slot's routing weight like any other) and a per-expert f32 bias [n_experts][M] that joins the
 * weighted sum, hidden[r] += sum_s w_s * (W[id_s][r] . x_s + bias[id_s][r])
 * (src/compute/forward.zig:6923-6927, ffn_down_exps_bias), never for the shared slot. */
int32_t zc_moe_down_acc_ex(zc_ctx* ctx, uint32_t type,
                           const void* A, uint64_t a_size,
                           const void* shared_down, uint64_t shared_down_size,
                           const void* down_bias, uint64_t down_bias_size,
                           const void* x, uint64_t x_size, void* y, uint64_t y_size,
                           const void* routing, uint64_t routing_size,
                           uint32_t M, uint32_t K, uint64_t expert_stride, uint32_t n_used,
                           uint32_t x_expert_stride, uint64_t x_offset, uint64_t y_offset);

/* Router and expert selection of one token in one launch: logits = W_router . xn with xn = hidden, or
 * xn = norm_weights * hidden * rsqrt(mean(hidden^2) + eps) when norm_weights is given (then also written to
 * norm_out if non-NULL); then the selection of zc_softmax_topk (same rules, optional bias on the logits) into
 * routing = [k + shared_slot ids][k + shared_slot weights]. With shared_slot = 1 the last slot is
 * {ZC_SHARED_EXPERT, 1.0f}. routing_local (optional, same layout) receives the selection as the expert-parallel
 * rank that owns experts [e_lo, e_hi) sees it: those ids renumbered from 0, the others 0xFFFFFFFF, the shared
 * slot kept if local_shared != 0 and 0xFFFFFFFF otherwise. At most 1024 experts; K a multiple of 4.
 * Replaces the router DMMV / fused norm + router dispatch followed by the softmax_topk dispatch
 * (src/compute/forward.zig:6139-6190; src/shaders/rms_norm_dmmv_f32.comp, softmax_topk.comp), and
 * zc_moe_ep_filter behind them. */
int32_t zc_moe_router_topk(zc_ctx* ctx, const void* hidden, uint64_t hidden_size,
                           const void* norm_weights, uint64_t norm_size,
                           const void* router_weights, uint64_t router_size,
                           const void* bias, uint64_t bias_size,
                           void* norm_out, uint64_t norm_out_size,
                           void* logits, uint64_t logits_size,
                           void* routing, uint64_t routing_size,
                           void* routing_local, uint64_t routing_local_size,
                           uint32_t n_experts, uint32_t K, uint32_t k, uint32_t rule, float eps,
                           uint32_t shared_slot, uint32_t e_lo, uint32_t e_hi, uint32_t local_shared);

/* Cross-token MoE matvec: Y[t][s][M] = W[routing[t*n_experts_used + s]] . X[t][K];
 * routing is the flattened [n_tokens][n_experts_used] id table; strides in
 * elements. K % 256 != 0 returns ZC_ERR_INVALID_ARG for K-quants. Replaces
 * recordMoeBatchedDispatch (src/compute/dmmv.zig:746-792;
 * src/shaders/dmmv_q4k_moe_batched.comp:70-164). Without a workspace every (token, slot) pair is
 * computed on its own in f32, like the reference's kernel. With a workspace (zc_set_workspace) of at
 * least zc_moe_grouped_workspace_bytes(...), n_tokens >= 16, type Q4_K, Q6_K or MXFP4 (K % 64 == 0) and 16-byte aligned
 * A / expert_stride / X, the pairs are grouped by expert (as the reference's Metal path does,
 * src/shaders/metal/moe_route_pack.metal:13-36) and each expert's weights are dequantised once per
 * tile of its tokens on the tensor cores: bf16 operands, f32 accumulation (relative L2 <= 5e-3).
 * Ids >= n_experts are skipped there (their output rows are left untouched). */
int32_t zc_moe_dmmv_batched(zc_ctx* ctx, uint32_t type,
                            const void* A, uint64_t a_size, const void* X, uint64_t x_size,
                            void* Y, uint64_t y_size, const void* routing, uint64_t routing_size,
                            uint32_t M, uint32_t K, uint64_t expert_stride,
                            uint32_t n_experts, uint32_t n_experts_used, uint32_t n_tokens,
                            uint32_t x_token_stride, uint32_t y_token_stride);

/* Gate and up of a prefill batch in one call: Yg = Wg[...] X, Yu = Wu[...] X with the arguments of
 * zc_moe_dmmv_batched. On the grouped path the pairs are grouped and the activations packed once for both
 * matrices; otherwise it is the two single calls. The prefill counterpart of zc_moe_fused_gate_up
 * (src/compute/forward.zig:6206-6222). */
int32_t zc_moe_dmmv_batched_pair(zc_ctx* ctx, uint32_t type,
                                 const void* Wg, uint64_t wg_size, const void* Wu, uint64_t wu_size,
                                 const void* X, uint64_t x_size, void* Yg, uint64_t yg_size, void* Yu, uint64_t yu_size,
                                 const void* routing, uint64_t routing_size,
                                 uint32_t M, uint32_t K, uint64_t expert_stride,
                                 uint32_t n_experts, uint32_t n_experts_used, uint32_t n_tokens,
                                 uint32_t x_token_stride, uint32_t y_token_stride);

/* Caller-owned device scratch for the grouped MoE prefill path; NULL / 0 removes it. The library never
 * allocates on the hot path, so the engine lends the bytes (its prefill scratch arena). 256-byte aligned.
 * The contents are only meaningful during one zc_moe_dmmv_batched call (in stream order). No counterpart
 * in the reference, whose Metal path owns route_ids / route_counts buffers (src/compute/forward_metal.zig). */
int32_t zc_set_workspace(zc_ctx* ctx, void* workspace, uint64_t size);
uint64_t zc_moe_grouped_workspace_bytes(uint32_t n_tokens, uint32_t n_experts_used, uint32_t K, uint32_t n_experts);

/* zc_mul_mm for MXFP4 weights and bf16 activations on the block-scaled tensor-core path
 * (tcgen05.mma kind::mxf8f6f4 with E8M0 block scales): the weights stay as stored (E2M1 nibbles + one E8M0 scale
 * byte per 32 elements are the tensor core's own operand format; src/compute/forward.zig:441-459 gives the
 * element order), the activations are split into two FP8 (E4M3) terms with power-of-two block scales whose sum
 * is the bf16 value exactly, written into `workspace` (zc_mul_mm_workspace_bytes(type, N, K) bytes, 256-byte
 * aligned, caller-owned) by a small kernel before the GEMM. N >= 64 tokens, K >= 128 and a multiple of 32; A and
 * B 16-byte aligned, stride_b a multiple of 8; offsets in elements of B and D as in zc_mul_mm. Results equal
 * zc_mul_mm's to the rounding of the f32 accumulation. As measured it is not yet faster than zc_mul_mm's route
 * (weights dequantised to bf16 tiles), which therefore stays the default. */
uint64_t zc_mul_mm_workspace_bytes(uint32_t type, uint32_t N, uint32_t K);
int32_t zc_mul_mm_block_scaled(zc_ctx* ctx, uint32_t type,
                               const void* A, uint64_t a_size, const void* B, uint64_t b_size,
                               void* D, uint64_t d_size,
                               uint32_t M, uint32_t N, uint32_t K, uint32_t stride_b, uint32_t stride_d,
                               uint64_t a_offset, uint64_t b_offset, uint64_t d_offset,
                               void* workspace, uint64_t workspace_size);

/* ---- routing, combine, activation -----------------------------------------------------------
 * zc_softmax_topk: per token t, out[t*out_stride ..] = [k ids u32][k weights f32 bits].
 * Replaces dispatchSoftmaxTopk (src/compute/forward.zig:4135-4210;
 * src/shaders/softmax_topk.comp:35-103) and the CPU routers
 * (src/compute/forward.zig:496-571). `bias` may be NULL; otherwise bias[e] is
 * added to logit e first (src/compute/forward.zig:6752-6754). n_experts is not
 * limited to 256 and k not to 16. */
int32_t zc_softmax_topk(zc_ctx* ctx, const void* logits, uint64_t logits_size,
                        const void* bias, void* out, uint64_t out_size,
                        uint32_t n_experts, uint32_t k, uint32_t rule,
                        uint32_t n_tokens, uint32_t logits_stride, uint32_t out_stride);

/* a[i] += sum_j w_j * b[j*src_stride + i]; w_j = f32 bits at routing[n_used + j].
 * Replaces dispatchMoeWeightedAcc (src/shaders/moe_weighted_acc.comp:23-33). */
int32_t zc_moe_weighted_acc(zc_ctx* ctx, void* a, uint64_t a_size, const void* b, uint64_t b_size,
                            const void* routing, uint64_t routing_size,
                            uint32_t n, uint32_t n_used, uint32_t src_stride);

/* y = silu(gate) * up (src/shaders/swiglu.comp:25-33) and the GPT-OSS variant
 * (src/shaders/swiglu_oai.comp:24-34; src/compute/forward.zig:607-616). */
int32_t zc_swiglu(zc_ctx* ctx, const void* gate, const void* up, void* y, uint32_t n);
int32_t zc_swiglu_oai(zc_ctx* ctx, const void* gate, const void* up, void* y, uint32_t n);

/* out[i] += bias[src_offset + i] for i < n. Replaces dispatchBiasAddSlice
 * (src/compute/forward.zig:3875-3913; src/shaders/bias_add.comp:19-23), which the reference uses for
 * the per-expert gate / up / down biases of GPT-OSS (forward.zig:6841-6849, 6923-6927). */
int32_t zc_bias_add(zc_ctx* ctx, void* out, uint64_t out_size, const void* bias, uint64_t bias_size,
                    uint32_t n, uint32_t src_offset);
/* The same biases for all selected slots at once, fused with the activation that follows them in the
 * reference's sequence (forward.zig:6841-6860): y[s][i] = act(gate[s][i] + gate_bias[e_s][i],
 * up[s][i] + up_bias[e_s][i]) with e_s = routing[s], biases [n_experts][M] f32 (either may be NULL),
 * act = swiglu (oai = 0) or swiglu_oai (oai = 1). */
int32_t zc_moe_bias_act(zc_ctx* ctx, const void* gate, uint64_t gate_size, const void* up, uint64_t up_size,
                        const void* gate_bias, uint64_t gate_bias_size,
                        const void* up_bias, uint64_t up_bias_size,
                        const void* routing, uint64_t routing_size, void* y, uint64_t y_size,
                        uint32_t M, uint32_t n_used, uint32_t n_experts, uint32_t oai);
/* a[i] += sum_s w_s * bias[e_s][i]: the down projection's per-expert bias (forward.zig:6923-6927) inside
 * the weighted sum of the expert outputs; routing = [ids n_used][weights n_used], bias [n_experts][n]. */
int32_t zc_moe_weighted_bias_acc(zc_ctx* ctx, void* a, uint64_t a_size, const void* bias, uint64_t bias_size,
                                 const void* routing, uint64_t routing_size,
                                 uint32_t n, uint32_t n_used, uint32_t n_experts);

/* Expert parallelism (no counterpart in the single-GPU reference): out = routing with the ids of the experts
 * [expert_lo, expert_hi) renumbered from 0 and every other id replaced by 0xFFFFFFFF ("no expert in this slot on
 * this rank"); the k weights of a row are copied. Every MoE entry point reads no weights for such a slot and
 * contributes zeros for it, so a rank that holds a contiguous range of whole experts runs the same calls on its
 * own stack with the filtered routing, and the ranks' partial hidden vectors are then summed. Rows of
 * routing_stride / out_stride words; with k <= out_stride < 2k only the k ids of a row are written (the flattened
 * id table zc_moe_dmmv_batched takes). zc_moe_route_scatter leaves out the slots marked 0xFFFFFFFF. */
int32_t zc_moe_ep_filter(zc_ctx* ctx, const void* routing, uint64_t routing_size, void* out, uint64_t out_size,
                         uint32_t k, uint32_t n_tokens, uint32_t routing_stride, uint32_t out_stride,
                         uint32_t expert_lo, uint32_t expert_hi);

/* counts[e] = number of cells equal to e in the routing capture buffer of one
 * layer. Replaces recordCountExperts (src/compute/dmmv.zig:981-1028;
 * src/shaders/count_experts.comp:58-83). d_offset_bytes as there. */
int32_t zc_count_experts(zc_ctx* ctx, const void* routing, uint64_t routing_size,
                         void* counts, uint64_t counts_size,
                         uint32_t n_tokens, uint32_t n_layers, uint32_t layer,
                         uint32_t n_experts_used, uint32_t n_experts, uint64_t d_offset_bytes);

/* Grouped-by-expert prefill path (the reference's Metal path):
 * zc_moe_route_pack: per expert the list of route ids (token*k + slot) in
 * token order and their count (src/shaders/metal/moe_route_pack.metal:13-36).
 * zc_moe_route_scatter: dst[t][d] += sum_slot w * src[t*k + slot][d]
 * (src/shaders/metal/moe_route_scatter.metal:20-96). */
int32_t zc_moe_route_pack(zc_ctx* ctx, const void* routing, uint64_t routing_size,
                          void* counts, uint64_t counts_size, void* ids, uint64_t ids_size,
                          uint32_t n_tokens, uint32_t n_experts, uint32_t k,
                          uint32_t routing_stride, uint32_t ids_stride);
int32_t zc_moe_route_scatter(zc_ctx* ctx, const void* routing, uint64_t routing_size,
                             const void* src, uint64_t src_size, void* dst, uint64_t dst_size,
                             uint32_t n_tokens, uint32_t hidden_dim, uint32_t k, uint32_t routing_stride);

/* ---- parity / embedding rows ---------------------------------------------------------------------
 * out[r][0..K) = dequantised row (first_row + r) of A, bit-identical to the
 * reference's CPU dequantRow (src/compute/forward.zig:242-465; Q5_1 from
 * src/compute/forward_metal.zig:6704-6729): products and differences are
 * rounded separately, never fused. Also serves the embedding-row lookup the
 * reference does on the CPU (src/compute/forward.zig:9391-9398). */
int32_t zc_dequant_rows(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size,
                        void* out, uint64_t out_size,
                        uint64_t first_row, uint32_t n_rows, uint32_t K, uint64_t a_offset);

/* ---- tensor-parallel exchange (no counterpart in the reference, which is single-GPU) -------------
 * One process per GPU. zc_comm_init allocates this rank's receive buffer (3 MB) and returns its
 * 64-byte CUDA IPC handle; the host exchanges the handles of all ranks by any means and passes
 * them, rank-major, to zc_comm_connect. zc_allreduce_sum_f32 then sums buf[0..n) over all ranks
 * in place with one kernel on the context's stream (peer stores over NVLink, bounded flag wait
 * -> ZC_ERR_TIMEOUT at the next zc_submit_and_wait); n a multiple of 4, at most 16384; every rank
 * must issue the same sequence of calls. Sums are formed in rank order: all ranks get identical bits. */
int32_t zc_comm_init(zc_ctx* ctx, uint32_t rank, uint32_t world, uint8_t* out_handle64);
int32_t zc_comm_connect(zc_ctx* ctx, const uint8_t* all_handles);
/* For ranks that live in this process (several contexts, one per GPU, with peer access enabled by the
 * caller): lend rank `rank`'s receive buffer by its device pointer instead of an IPC handle. The buffer
 * (zc_comm_buffer_bytes() bytes, 256-byte aligned, zeroed) stays the caller's; zc_comm_connect skips
 * ranks connected this way. */
int32_t zc_comm_connect_local(zc_ctx* ctx, uint32_t rank, void* receive_buffer, uint64_t size);
uint64_t zc_comm_buffer_bytes(void);
int32_t zc_allreduce_sum_f32(zc_ctx* ctx, void* buf, uint64_t buf_size, uint64_t offset, uint32_t n);
/* dst[r*n .. r*n+n) <- rank r's src[0..n) for every rank r (src may be the rank's own slice of dst);
 * n a multiple of 4, world * n <= 262144. Same protocol and ordering rule as the all-reduce. */
int32_t zc_allgather_f32(zc_ctx* ctx, const void* src, uint64_t src_size, uint64_t src_offset,
                         void* dst, uint64_t dst_size, uint64_t dst_offset, uint32_t n);
int32_t zc_comm_destroy(zc_ctx* ctx);
/* The exchange fused into the matvecs: a K-sharded projection whose partial result is summed over the ranks.
 * Arguments as zc_dmmv; instead of writing y, the kernel's epilogue stores every finished row into the
 * row's slot of every rank's receive buffer (plain peer stores over NVLink, value and tag in one 8-byte
 * store: no flag, no fence, no multicast). The sum dst[i] (+)= sum over ranks (acc_mode 1: added to what dst
 * holds, which must be the same on every rank) is formed, in rank order, by the *next* call on this context:
 * zc_dmmv, zc_dmmv_multi, zc_dmmv_fused_gate_up_swiglu and zc_dmmv_push carry it in their own kernel (their
 * threads wait, bounded, for all ranks' rows after the kernel's dependency wait; a call that reads or writes
 * dst completes it first), any other call completes it with a small kernel of its own first. dst is valid
 * once that next call has completed; zc_submit_and_wait and zc_end_record count as such a call. M <= 16384;
 * every rank must issue the same sequence of pushes, an even number of them per recorded sequence. A wait
 * that gives up reports ZC_ERR_TIMEOUT as the collectives above do. */
int32_t zc_dmmv_push(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size,
                     const void* x, uint64_t x_size, void* dst, uint64_t dst_size,
                     uint32_t M, uint32_t K, uint64_t a_offset, uint64_t x_offset, uint64_t dst_offset,
                     uint32_t acc_mode);

/* ---- matvec without a context and without any allocation ----------------------------------------
 * No counterpart in the reference (its dispatch layer always owns descriptor pools and buffers).
 * The streaming Q4_K matvec of zc_dmmv, y (+)= W x, with its split-K scratch in a __device__
 * array that is part of the library image (1048576 bytes: 4096 worker warps x 32 partial sums,
 * each stored with a tag word) instead of scratch a context allocated. For hosts that cannot let
 * the library allocate: all device memory already belongs to the host's own arena, or an
 * allocation would synchronise the device in the middle of its decode loop. Neither this call
 * nor its set-up allocates memory of any kind.
 *
 * Uses the calling thread's current device; `cuda_stream` (NULL = default stream), A, x, y and
 * status_words must belong to it. Arguments as zc_dmmv for type Q4_K. Limits: K a multiple of
 * 256 and at most 12288; at least 16 (16-row tile x 512-column segment) units, i.e. matrices
 * from about 64 x 1024 up; W + a_offset and x + x_offset 16-byte aligned. Anything outside is
 * refused with ZC_ERR_INVALID_ARG and a message in err_buf (may be NULL): use zc_dmmv there.
 * status_words: two u32 words the device can write (device or mapped host memory), zero before
 * the call; a bounded wait that gave up stores {1, site} there, the result is then invalid and
 * the entry point must not be used again on that device.
 *
 * The first call on each device does the set-up (symbol address, SM count; the array is all
 * zero when the library is loaded and every launch leaves it zero): make it before any stream
 * capture starts on that device.
 * The scratch is shared by all calls on a device: calls ordered on one stream are safe; calls
 * whose kernels may overlap (different streams, unordered threads) race and give wrong results. */
int32_t zc_dmmv_q4k_static_scratch(void* cuda_stream,
                                   const void* A, uint64_t a_size,
                                   const void* x, uint64_t x_size,
                                   void* y, uint64_t y_size,
                                   uint32_t M, uint32_t K,
                                   uint64_t a_offset, uint64_t x_offset, uint64_t y_offset,
                                   uint32_t acc_mode, uint32_t* status_words,
                                   char* err_buf, uint64_t err_cap);

#ifdef __cplusplus
}
#endif
#endif /* ZINC_CUDA_H */
