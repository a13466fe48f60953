// Internal launch interface between the C ABI (api.cu) and the kernel files.
// All pointers are device pointers already offset and validated by the caller.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace zc {

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device property of a kernel: opt in once per device
// ordinal (bit d of `done`), with the device that is current at the launch. Safe from several host threads.
template <typename Kern>
inline cudaError_t ensure_dynamic_smem(Kern kern, int bytes, std::atomic<uint64_t>& done) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (dev & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    done.fetch_or(bit, std::memory_order_release);
    return cudaSuccess;
}

// Epilogue / addressing modes of the decode matvec kernel family.
enum DmmvMode : int {
    MODE_PLAIN = 0,          // y (+)= W x
    MODE_GATE_UP_SWIGLU = 1, // out = silu(Wg x) * (Wu x)
    MODE_SIGMOID_ACC = 2,    // y += sigmoid(gate) * (W x)
    MODE_MOE = 3,            // per slot: Y[s] = W[routing[s]] X[s]
    MODE_MOE_GATE_UP = 4,    // per slot: Yg[s], Yu[s]
    MODE_MOE_DOWN_ACC = 5,   // y += sum_s w_s * W[id_s] X[s]
    MODE_BATCH = 6,          // per column c: Y[c] = W X[c]   (n_used = columns, x_expert_stride = K)
    MODE_MOE_BATCHED = 7,    // per (token t, slot s): Y[t][s] = W[routing[t*n_used+s]] X[t]
};

// ---- tensor-parallel exchange fused into the matvecs (peer memory over NVLink, no multicast) -------------
// A K-sharded projection produces a partial output vector on every rank. Its epilogue stores every finished
// row, as {f32 bits, 1}, into the row's slot of *every* rank's receive buffer (plain peer stores; an 8-byte
// store is one transaction, so value and tag arrive together: no flag, no fence). The next matvec on the
// stream carries the other half: its threads wait, bounded, for the tagged values of all ranks in the local
// buffer, add them in rank order (bit-identical sums everywhere), write the reduced vector and clear the tags.
constexpr uint32_t kCommMaxRanks = 8;
constexpr uint32_t kPushMaxFloats = 16384;  // longest vector the fused exchange carries
struct PushArgs {
    uint2* peers[kCommMaxRanks] = {};  // [r]: this rank's slot (current parity) in rank r's receive buffer
    uint32_t world = 0;                // 0: no push, the kernel writes y
};
struct ConsumeArgs {
    uint2* slots = nullptr;   // local receive buffer, current parity: [world][kPushMaxFloats]
    float* dst = nullptr;     // dst[i] (+)= sum over ranks
    uint32_t n = 0;           // 0: nothing to consume
    uint32_t world = 0, acc = 0;
    uint32_t spin_limit = 1u << 24;
    uint32_t* status = nullptr;
};

// Activation built from split-K flash-attention partials while it is loaded (the fused merge + O projection,
// src/shaders/dmmv_q4k_o_proj_merge.comp): x[head * head_dim + d] = sum_c w_c partial[(head * n_chunks + c) *
// head_dim + d] / L, with the chunks' {max, sum} pairs behind the partials. partial == nullptr: plain x.
struct MergeArgs {
    const float* partial = nullptr;
    const float* sinks = nullptr;  // nullptr: none
    uint32_t n_heads = 0, n_chunks = 0, head_dim = 0, sink_offset = 0;
};

struct DmmvArgs {
    const uint8_t* A = nullptr;   // weights (gate weights for the gate/up modes)
    const uint8_t* A2 = nullptr;  // up weights for the gate/up modes
    const float* x = nullptr;
    float* y = nullptr;
    float* y2 = nullptr;          // second output (MoE gate/up)
    const float* gate = nullptr;  // sigmoid gate scalar
    const uint32_t* routing = nullptr;
    uint32_t M = 0, K = 0;
    uint32_t acc_mode = 0;
    uint32_t n_used = 1;
    uint32_t act = 0;             // MoE gate/up: 0 write both, 1 y = silu(gate) * up, 2 the GPT-OSS (swiglu_oai) form
    uint32_t x_expert_stride = 0;
    uint64_t expert_stride = 0;
    uint32_t n_experts_max = 0xFFFFFFFFu;  // expert ids in `routing` must be below this (experts the buffer holds)
    uint32_t n_tokens = 1;        // MODE_MOE_BATCHED
    uint32_t x_token_stride = 0;  // MODE_MOE_BATCHED, elements
    uint32_t y_token_stride = 0;  // MODE_MOE_BATCHED, elements
    // context scratch of the split-K streaming kernels (null: streaming path not used)
    uint2* scratch_partial = nullptr;   // [kStreamMaxWorkers][32] {f32 bits, tag} partial sums handed across CTAs;
                                        // all zero between launches (the reader of a value clears it)
    uint32_t* status = nullptr;
    uint32_t spin_limit = 1u << 26;     // polls after which a device-side wait gives up
    int sm_count = 0;
    PushArgs push;        // MODE_PLAIN: store the result rows into every rank's receive buffer instead of y
    ConsumeArgs consume;  // a pending reduction of pushed vectors that this launch (or a small kernel before it) completes
    // first byte past the buffers that hold A / A2 (kernels that fetch aligned supersets of unaligned rows
    // must not read beyond them)
    const uint8_t* a_end = nullptr;
    const uint8_t* a2_end = nullptr;
    // MoE launches: the matrices a routing slot with the id kSharedExpert selects (null: there is none)
    const uint8_t* A_sh = nullptr;
    const uint8_t* A2_sh = nullptr;
    const uint8_t* a_sh_end = nullptr;   // first byte past their buffers
    const uint8_t* a2_sh_end = nullptr;
    // MoE launches: per-expert f32 biases [n_experts][M]. Gate / up: added to the gate and up rows before the
    // activation. Down + accumulate: sum_s w_s bias[e_s][row] joins the weighted sum. Never applied to the
    // shared expert's slot.
    const float* bias = nullptr;
    const float* bias2 = nullptr;
    // The kernel right before this one in the stream releases its dependents early and may still be producing
    // the routing buffer: read the routing only after the dependency wait, and release this launch's own
    // dependents only after it (so that a successor's prologue may trust everything older).
    bool late = false;
    MergeArgs merge;  // MODE_PLAIN on the Q4_K streaming kernel: x comes from attention partials
};

// Capacity of the split-K scratch a context owns.
// Below this many weight bytes a matvec is latency-bound and the one-warp-per-row kernels (more CTAs) win.
constexpr uint64_t kStreamMinBytes = 2u << 20;
constexpr uint32_t kStreamMaxWorkers = 4096;  // warps that may publish a partial tile
constexpr size_t kStreamPartialBytes = (size_t)kStreamMaxWorkers * 32 * sizeof(uint2);

// Warp-autonomous streaming (cp.async + tensor-core) matvec: eligibility and launch.
bool warp_dmmv_eligible(uint32_t type, int mode, const DmmvArgs& a);
cudaError_t launch_warp_dmmv(uint32_t type, int mode, const DmmvArgs& a, cudaStream_t s, uint64_t* launches);
// Grouped form: n (2 or 3) Q4_K matrices that share x and K, one launch. `common` carries x, K, acc_mode,
// the scratch, the status words and the SM count.
bool warp_dmmv_multi_eligible(uint32_t type, uint32_t n, const uint8_t* const* A, const uint32_t* M, uint32_t K,
                              const DmmvArgs& common);
cudaError_t launch_warp_dmmv_multi(uint32_t n, const uint8_t* const* A, float* const* y, const uint32_t* M,
                                   const DmmvArgs& common, cudaStream_t s, uint64_t* launches);
// MoE fused gate + up through the streaming kernel (Q4_K, x shared by the slots): a.A / a.A2 the stacked
// expert matrices, a.y / a.y2 the [n_used][M] outputs, a.routing the slot -> expert ids.
bool warp_moe_gate_up_eligible(uint32_t type, const DmmvArgs& a);
cudaError_t launch_warp_moe_gate_up(const DmmvArgs& a, cudaStream_t s, uint64_t* launches);
// Streaming MXFP4 matvec (dmmv_mxfp4.cu): plain / accumulate, and the MoE fused gate + up form.
bool mxfp4_dmmv_eligible(uint32_t type, int mode, const DmmvArgs& a);
cudaError_t launch_mxfp4_dmmv(const DmmvArgs& a, cudaStream_t s, uint64_t* launches);
bool mxfp4_moe_gate_up_eligible(uint32_t type, const DmmvArgs& a);
cudaError_t launch_mxfp4_moe_gate_up(const DmmvArgs& a, cudaStream_t s, uint64_t* launches);
// y += sum_s w_s * W[routing[s]] x_s (the fused MoE down projection + weighted accumulate)
bool mxfp4_moe_down_acc_eligible(uint32_t type, const DmmvArgs& a);
cudaError_t launch_mxfp4_moe_down_acc(const DmmvArgs& a, cudaStream_t s, uint64_t* launches);
bool q6k_dmmv_eligible(uint32_t type, int mode, const DmmvArgs& a);
cudaError_t launch_q6k_dmmv(int mode, const DmmvArgs& a, cudaStream_t s, uint64_t* launches);
bool q6k_moe_down_acc_eligible(uint32_t type, const DmmvArgs& a);
cudaError_t launch_q6k_moe_down_acc(const DmmvArgs& a, cudaStream_t s, uint64_t* launches);

// Returns cudaSuccess or the launch error; *launches is incremented per kernel.
cudaError_t launch_dmmv(uint32_t type, int mode, const DmmvArgs& a, cudaStream_t s, uint64_t* launches);

// Y[c][M] = W X[c][K], X/Y f32 row per column.
cudaError_t launch_dmmv_batch(uint32_t type, const uint8_t* A, const float* X, float* Y, uint32_t M, uint32_t K,
                              uint32_t num_cols, cudaStream_t s, uint64_t* launches);

// Cross-token MoE: Y[t][s][M] = W[routing[t*k+s]] X[t].
cudaError_t launch_moe_dmmv_batched(uint32_t type, const uint8_t* A, const float* X, float* Y,
                                    const uint32_t* routing, uint32_t M, uint32_t K, uint64_t expert_stride,
                                    uint32_t n_experts_used, uint32_t n_tokens, uint32_t x_token_stride,
                                    uint32_t y_token_stride, uint32_t n_experts_max, uint32_t* status, cudaStream_t s,
                                    uint64_t* launches);

// Grouped-by-expert tensor-core form of the cross-token MoE matmul (moe_gemm_tc.cu): Q4_K / Q6_K, bf16
// operands, needs a device workspace of moe_grouped_workspace_bytes(n_tokens * n_used, K, n_experts).
uint64_t moe_grouped_workspace_bytes(uint64_t n_pairs, uint32_t K, uint32_t n_experts);
bool moe_grouped_eligible(uint32_t type, const uint8_t* A, uint32_t K, uint64_t expert_stride, uint32_t n_experts,
                          uint64_t n_pairs, const float* X, uint32_t x_token_stride, uint64_t ws_size);
cudaError_t launch_moe_grouped(uint32_t type, const uint8_t* A, uint64_t a_bytes, const float* X, float* Y,
                               const uint32_t* routing, uint32_t M, uint32_t K, uint64_t expert_stride,
                               uint32_t n_experts, uint32_t n_used, uint32_t n_tokens, uint32_t x_token_stride,
                               uint32_t y_token_stride, void* ws, uint32_t* status, cudaStream_t s,
                               uint64_t* launches, const uint8_t* A2 = nullptr, uint64_t a2_bytes = 0,
                               float* Y2 = nullptr);  // A2 / Y2: a second matrix on the same grouping (gate + up)

// Prefill GEMM for the weight layouts without a 16-byte row pitch (MXFP4, Q6_K with K % 2048 != 0): bf16
// activations, raw blocks fetched with cp.async, same tile kernel as the grouped MoE path (moe_gemm_tc.cu).
// MXFP4 weights on the block-scaled tensor-core path (gemm_mx.cu): weights as stored, bf16 activations split into
// two FP8 terms in a caller-lent workspace.
uint64_t mul_mm_mx_workspace_bytes(uint32_t N, uint32_t K);
bool mul_mm_mx_eligible(uint32_t type, const uint8_t* A, const void* B, uint32_t N, uint32_t K, uint32_t stride_b,
                        const void* workspace, uint64_t workspace_size);
cudaError_t launch_mul_mm_mx(const uint8_t* A, uint64_t a_bytes, const void* B, float* D, uint32_t M, uint32_t N,
                             uint32_t K, uint32_t stride_b, uint32_t stride_d, void* workspace, uint32_t* status,
                             int sm_count, cudaStream_t s, uint64_t* launches);
bool mul_mm_cp_async_eligible(uint32_t type, const uint8_t* A, const void* B, uint32_t N, uint32_t K,
                              uint32_t stride_b);
cudaError_t launch_mul_mm_cp_async(uint32_t type, const uint8_t* A, uint64_t a_bytes, const void* B, float* D,
                                   uint32_t M, uint32_t N, uint32_t K, uint32_t stride_b, uint32_t stride_d,
                                   uint32_t* status, cudaStream_t s, uint64_t* launches);

cudaError_t launch_dequant_rows(uint32_t type, const uint8_t* A, float* out, uint64_t first_row, uint32_t n_rows,
                                uint32_t K, cudaStream_t s, uint64_t* launches);

cudaError_t launch_softmax_topk(const float* logits, const float* bias, uint32_t* out, uint32_t n_experts,
                                uint32_t k, uint32_t rule, uint32_t n_tokens, uint32_t logits_stride,
                                uint32_t out_stride, cudaStream_t s, uint64_t* launches);
cudaError_t launch_moe_weighted_acc(float* a, const float* b, const uint32_t* routing, uint32_t n, uint32_t n_used,
                                    uint32_t src_stride, cudaStream_t s, uint64_t* launches);
cudaError_t launch_swiglu(const float* gate, const float* up, float* y, uint32_t n, bool oai, cudaStream_t s,
                          uint64_t* launches);
// out[i] += bias[src_offset + i]
cudaError_t launch_bias_add(float* out, const float* bias, uint32_t n, uint32_t src_offset, cudaStream_t s,
                            uint64_t* launches);
// y[s][i] = act(gate[s][i] + gate_bias[e_s][i], up[s][i] + up_bias[e_s][i]), e_s = routing[s]; biases may be null
cudaError_t launch_moe_bias_act(const float* gate, const float* up, const float* gate_bias, const float* up_bias,
                                const uint32_t* routing, float* y, uint32_t M, uint32_t n_used, uint32_t n_experts,
                                bool oai, uint32_t* status, cudaStream_t s, uint64_t* launches);
// a[i] += sum_s w_s * bias[e_s][i], routing = [ids n_used][weights n_used]
cudaError_t launch_moe_weighted_bias_acc(float* a, const float* bias, const uint32_t* routing, uint32_t n,
                                         uint32_t n_used, uint32_t n_experts, uint32_t* status, cudaStream_t s,
                                         uint64_t* launches);
// y[m] = sum_k W[m][k] * xn[k], xn = norm_w * (x * rsqrt(mean(x^2) + eps)) (also written to norm_out when
// given); norm_w == nullptr: xn = x. One CTA per row: for matrices with few rows (routers). K % 4 == 0.
// With W2 / y2: a second M x K matrix on the same normalised vector in the same launch (y2 = W2 xn).
cudaError_t launch_rms_norm_dmmv_f32(const float* x, const float* norm_w, const float* W, float* norm_out, float* y,
                                     uint32_t M, uint32_t K, float eps, cudaStream_t s, uint64_t* launches,
                                     const float* W2 = nullptr, float* y2 = nullptr);
// Expert parallelism: routing rows [k ids][k weights] -> ids of the experts [lo, hi) renumbered from 0, the others
// replaced by the "no expert" mark (kernels read no weights for such a slot and contribute zeros).
// Router matvec (optionally behind the RMS norm) + expert selection in one launch, for up to 1024 experts
// (cudaErrorNotSupported beyond, or when K is not a multiple of 4). `tagged`: 1024 zeroed uint2 of context scratch
// (zero again when the kernel ends); `status` / `spin_limit`: where and after how many polls a wait gives up.
cudaError_t launch_moe_router_topk(const float* x, const float* norm_w, const float* W, const float* bias,
                                   float* norm_out, float* logits, uint32_t* routing, uint32_t* routing_local,
                                   uint2* tagged, uint32_t* status, uint32_t spin_limit, uint32_t n_experts, uint32_t K, uint32_t k, uint32_t rule,
                                   uint32_t shared, uint32_t e_lo, uint32_t e_hi, uint32_t local_shared, float eps,
                                   cudaStream_t s, uint64_t* launches);
// x[n_heads * head_dim] merged from split-K attention partials (the stand-alone form of MergeArgs).
cudaError_t launch_attn_merge(const MergeArgs& m, float* out, cudaStream_t s, uint64_t* launches);
cudaError_t launch_moe_ep_filter(const uint32_t* in, uint32_t* out, uint32_t k, uint32_t n_tokens, uint32_t stride_in,
                                 uint32_t stride_out, uint32_t lo, uint32_t hi, cudaStream_t s, uint64_t* launches);
cudaError_t launch_count_experts(const uint32_t* a, uint32_t* counts, uint32_t n_experts, uint32_t ne00,
                                 uint32_t ne01, uint32_t nb00, uint32_t nb01, uint32_t a_offset, cudaStream_t s,
                                 uint64_t* launches);
cudaError_t launch_moe_route_pack(const uint32_t* routing, uint32_t* counts, uint32_t* ids, uint32_t n_tokens,
                                  uint32_t n_experts, uint32_t k, uint32_t routing_stride, uint32_t ids_stride,
                                  cudaStream_t s, uint64_t* launches);
cudaError_t launch_moe_route_scatter(const uint32_t* routing, const float* src, float* dst, uint32_t n_tokens,
                                     uint32_t hidden, uint32_t k, uint32_t routing_stride, cudaStream_t s,
                                     uint64_t* launches);

// ---- one-shot all-reduce over peer memory (comm.cu) -------------------------------------------
constexpr size_t kCommSlotBytes = 64 * 1024;  // largest vector: 16384 floats
constexpr size_t kCommGatherBytes = 1024 * 1024;  // largest gathered vector: 262144 floats over all ranks
constexpr size_t kCommGatherOffset = 2 * kCommMaxRanks * kCommSlotBytes;       // [2 parities][kCommGatherBytes]
constexpr size_t kCommFlagOffset = kCommGatherOffset + 2 * kCommGatherBytes;   // reduce flags [2][ranks]
constexpr size_t kCommGatherFlagOffset = kCommFlagOffset + 2 * kCommMaxRanks * sizeof(uint32_t);
constexpr size_t kCommEpochOffset = kCommGatherFlagOffset + 2 * kCommMaxRanks * sizeof(uint32_t);
// words at kCommEpochOffset: [0] reduce epoch, [1] gather epoch, [2] gather arrivals, [3] gather departures
constexpr size_t kCommPushOffset = kCommEpochOffset + 256;  // fused exchange: [2 parities][ranks][kPushMaxFloats] uint2
constexpr size_t kCommPushParityBytes = (size_t)kCommMaxRanks * kPushMaxFloats * sizeof(uint2);
constexpr size_t kCommBufBytes = kCommPushOffset + 2 * kCommPushParityBytes;
// Completes a pending reduction on its own (when the next call on the stream cannot carry it).
cudaError_t launch_consume(const ConsumeArgs& c, cudaStream_t s, uint64_t* launches);
struct CommArgs {
    uint8_t* peers[kCommMaxRanks];  // receive buffer of every rank as mapped in this process; [rank] is local
    uint32_t rank = 0, world = 0;
    uint32_t* status = nullptr;
    uint32_t spin_limit = 1u << 24;  // polls after which a wait for a peer's flag gives up
};
// buf[0..n) <- sum over ranks, in place; n a multiple of 4, n * 4 <= kCommSlotBytes
cudaError_t launch_allreduce_oneshot(const CommArgs& c, float* buf, uint32_t n, cudaStream_t s, uint64_t* launches);
// dst[r*n .. r*n+n) <- rank r's src[0..n) for every r; n a multiple of 4, world * n * 4 <= kCommGatherBytes
cudaError_t launch_allgather_oneshot(const CommArgs& c, const float* src, float* dst, uint32_t n, cudaStream_t s,
                                     uint64_t* launches);

// Tensor-core dequant-GEMM: D[col][row] = sum_k A[row][k] B[col][k].
// act_bf16: B holds bf16 (else f32). Returns cudaErrorNotSupported for types
// without a tile dequantiser. tile_flags: n_tile_flags words of device scratch for the kernel that splits tiles
// over CTA pairs (two per tile of 256 rows x 512 tokens; shapes that need more take the other kernels).
cudaError_t launch_mul_mm(uint32_t type, const uint8_t* A, const void* B, float* D, uint32_t M, uint32_t N,
                          uint32_t K, uint32_t stride_b, uint32_t stride_d, bool act_bf16, uint32_t* status,
                          uint32_t* tile_flags, uint32_t n_tile_flags, cudaStream_t s, uint64_t* launches);

}  // namespace zc
