// Decode dequant-matvec kernel family: one warp per output row (or row pair),
// lanes split K, f32 accumulation, shuffle reduction, fused epilogues.
//
// Stands in for the reference's per-type decode shaders and their fused and
// MoE variants (src/shaders/dmmv_q4k.comp:59-240, dmmv_q5k.comp, dmmv_q6k.comp,
// dmmv_q8_0.comp, dmmv_mxfp4.comp, dmmv_q5_0.comp, dmmv_q5_1.comp, dmmv_f16.comp,
// dmmv_f32.comp, dmmv_q4k_fused_gate_up_swiglu.comp, dmmv_q8_0_sigmoid_acc.comp,
// dmmv_q4k_moe_kpar.comp, dmmv_q4k_fused_gate_up_moe.comp,
// dmmv_q4k_moe_fused_down_acc.comp and their per-type siblings).
#include "kernels.h"
#include "rowdot.cuh"

namespace zc {

namespace {

constexpr int kWarps = 8;

// src/shaders/swiglu.comp:25-33 (act = 1), src/shaders/swiglu_oai.comp:24-34 (act = 2)
__device__ __forceinline__ float gate_up_act_v1(uint32_t act, float gate, float up) {
    if (act == 2) {
        const float g = fminf(gate, 7.0f);
        const float u = fmaxf(-7.0f, fminf(up, 7.0f));
        return (g / (1.0f + expf(1.702f * (-g)))) * (u + 1.0f);
    }
    return (gate / (1.0f + expf(-gate))) * up;
}

template <uint32_t TYPE, int MODE, int NR, bool ALIGNED>
__global__ void __launch_bounds__(kWarps * 32) dmmv_kernel(const DmmvArgs a) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const uint64_t row_bytes = (uint64_t)(a.K / block_size(TYPE)) * bytes_per_block(TYPE);

    if constexpr (MODE == MODE_PLAIN || MODE == MODE_SIGMOID_ACC) {
        const uint32_t row0 = (blockIdx.x * kWarps + warp) * NR;
        if (row0 >= a.M) return;
        const uint8_t* rows[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) rows[r] = a.A + (uint64_t)min(row0 + r, a.M - 1) * row_bytes;
        float acc[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] = 0.f;
        rowdot<TYPE, NR, ALIGNED>(rows, a.x, a.K, lane, acc);
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] = warp_sum(acc[r]);
        if (lane == 0) {
            float g = 1.f;
            if constexpr (MODE == MODE_SIGMOID_ACC) g = 1.0f / (1.0f + expf(-__ldg(a.gate)));
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                if (row0 + r < a.M) {
                    float* yp = a.y + row0 + r;
                    if constexpr (MODE == MODE_SIGMOID_ACC) {
                        *yp += g * acc[r];
                    } else if (a.push.world) {  // fused exchange: the row goes to every rank's receive buffer
                        const uint2 pv = make_uint2(__float_as_uint(acc[r]), 1u);
                        for (uint32_t pr = 0; pr < a.push.world; ++pr) a.push.peers[pr][row0 + r] = pv;
                    } else {
                        *yp = a.acc_mode ? *yp + acc[r] : acc[r];
                    }
                }
            }
        }
    } else if constexpr (MODE == MODE_GATE_UP_SWIGLU) {
        const uint32_t row = blockIdx.x * kWarps + warp;
        if (row >= a.M) return;
        const uint8_t* rows[2] = {a.A + (uint64_t)row * row_bytes, a.A2 + (uint64_t)row * row_bytes};
        float acc[2] = {0.f, 0.f};
        rowdot<TYPE, 2, ALIGNED>(rows, a.x, a.K, lane, acc);
        const float g = warp_sum(acc[0]), u = warp_sum(acc[1]);
        if (lane == 0) a.y[row] = (g / (1.0f + expf(-g))) * u;
    } else if constexpr (MODE == MODE_MOE) {
        const uint32_t slot = blockIdx.y;
        const uint32_t row0 = (blockIdx.x * kWarps + warp) * NR;
        if (row0 >= a.M) return;
        const uint32_t e_raw = __ldg(a.routing + slot);
        if (e_raw == kSkipExpert) {  // no expert in this slot on this rank: zeros
            if (lane == 0)
                for (int r = 0; r < NR; ++r)
                    if (row0 + r < a.M) a.y[(size_t)slot * a.M + row0 + r] = 0.f;
            return;
        }
        const uint8_t* base = a.A + (uint64_t)checked_expert(e_raw, a.n_experts_max, a.status) * a.expert_stride;
        const float* x = a.x + (size_t)slot * a.x_expert_stride;
        const uint8_t* rows[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) rows[r] = base + (uint64_t)min(row0 + r, a.M - 1) * row_bytes;
        float acc[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] = 0.f;
        rowdot<TYPE, NR, ALIGNED>(rows, x, a.K, lane, acc);
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] = warp_sum(acc[r]);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r)
                if (row0 + r < a.M) a.y[(size_t)slot * a.M + row0 + r] = acc[r];
        }
    } else if constexpr (MODE == MODE_MOE_GATE_UP) {
        // NR row pairs (gate row, up row) per warp: independent load chains share the x loads
        const uint32_t slot = blockIdx.y;
        const uint32_t row0 = (blockIdx.x * kWarps + warp) * NR;
        if (row0 >= a.M) return;
        const uint32_t e_raw = __ldg(a.routing + slot);
        if (e_raw == kSkipExpert) {  // no expert in this slot on this rank: zeros
            if (lane == 0)
                for (int r = 0; r < NR; ++r)
                    if (row0 + r < a.M) {
                        a.y[(size_t)slot * a.M + row0 + r] = 0.f;
                        if (!a.act) a.y2[(size_t)slot * a.M + row0 + r] = 0.f;
                    }
            return;
        }
        const uint8_t* mg = expert_matrix(a.A, a.A_sh, e_raw, a.expert_stride, a.n_experts_max, a.status);
        const uint8_t* mu = expert_matrix(a.A2, a.A2_sh, e_raw, a.expert_stride, a.n_experts_max, a.status);
        const float* x = a.x + (size_t)slot * a.x_expert_stride;
        const uint8_t* rows[2 * NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint64_t off = (uint64_t)min(row0 + r, a.M - 1) * row_bytes;
            rows[2 * r] = mg + off;
            rows[2 * r + 1] = mu + off;
        }
        float acc[2 * NR];
#pragma unroll
        for (int r = 0; r < 2 * NR; ++r) acc[r] = 0.f;
        rowdot<TYPE, 2 * NR, ALIGNED>(rows, x, a.K, lane, acc);
#pragma unroll
        for (int r = 0; r < 2 * NR; ++r) acc[r] = warp_sum(acc[r]);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r)
                if (row0 + r < a.M) {
                    float vg = acc[2 * r], vu = acc[2 * r + 1];
                    if (e_raw < a.n_experts_max) {  // per-expert biases (not for the shared expert's slot)
                        if (a.bias) vg += __ldg(a.bias + (size_t)e_raw * a.M + row0 + r);
                        if (a.bias2) vu += __ldg(a.bias2 + (size_t)e_raw * a.M + row0 + r);
                    }
                    if (a.act) {
                        a.y[(size_t)slot * a.M + row0 + r] = gate_up_act_v1(a.act, vg, vu);
                    } else {
                        a.y[(size_t)slot * a.M + row0 + r] = vg;
                        a.y2[(size_t)slot * a.M + row0 + r] = vu;
                    }
                }
        }
    } else if constexpr (MODE == MODE_BATCH) {
        const uint32_t col = blockIdx.y;
        const uint32_t row0 = (blockIdx.x * kWarps + warp) * NR;
        if (row0 >= a.M) return;
        const uint8_t* rows[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) rows[r] = a.A + (uint64_t)min(row0 + r, a.M - 1) * row_bytes;
        float acc[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] = 0.f;
        rowdot<TYPE, NR, ALIGNED>(rows, a.x + (size_t)col * a.x_expert_stride, a.K, lane, acc);
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] = warp_sum(acc[r]);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r)
                if (row0 + r < a.M) a.y[(size_t)col * a.M + row0 + r] = acc[r];
        }
    } else if constexpr (MODE == MODE_MOE_BATCHED) {
        const uint32_t slot = blockIdx.y, tok = blockIdx.z;
        const uint32_t row = blockIdx.x * kWarps + warp;
        if (row >= a.M) return;
        const uint32_t e_raw = __ldg(a.routing + (size_t)tok * a.n_used + slot);
        if (e_raw == kSkipExpert) return;
        const uint32_t e = checked_expert(e_raw, a.n_experts_max, a.status);
        if (e != e_raw) return;  // not an expert: reported, its output row stays untouched (as on the grouped path)
        const uint8_t* rows[1] = {a.A + (uint64_t)e * a.expert_stride + (uint64_t)row * row_bytes};
        float acc[1] = {0.f};
        rowdot<TYPE, 1, ALIGNED>(rows, a.x + (size_t)tok * a.x_token_stride, a.K, lane, acc);
        const float v = warp_sum(acc[0]);
        if (lane == 0) a.y[(size_t)tok * a.y_token_stride + (size_t)slot * a.M + row] = v;
    } else {  // MODE_MOE_DOWN_ACC: NR rows per warp, the slots in sequence
        const uint32_t row0 = (blockIdx.x * kWarps + warp) * NR;
        if (row0 >= a.M) return;
        float total[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) total[r] = 0.f;
        for (uint32_t s = 0; s < a.n_used; ++s) {
            const uint32_t e_raw = __ldg(a.routing + s);
            if (e_raw == kSkipExpert) continue;
            const uint8_t* base = expert_matrix(a.A, a.A_sh, e_raw, a.expert_stride, a.n_experts_max, a.status);
            const uint8_t* rows[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) rows[r] = base + (uint64_t)min(row0 + r, a.M - 1) * row_bytes;
            const float w = __uint_as_float(__ldg(a.routing + a.n_used + s));
            float acc[NR];
#pragma unroll
            for (int r = 0; r < NR; ++r) acc[r] = 0.f;
            rowdot<TYPE, NR, ALIGNED>(rows, a.x + (size_t)s * a.x_expert_stride, a.K, lane, acc);
#pragma unroll
            for (int r = 0; r < NR; ++r) total[r] = fmaf(w, acc[r], total[r]);
            if (a.bias && lane == 0 && e_raw < a.n_experts_max) {  // the expert's bias, weighted like its product
#pragma unroll
                for (int r = 0; r < NR; ++r)
                    total[r] = fmaf(w, __ldg(a.bias + (size_t)e_raw * a.M + min(row0 + r, a.M - 1)), total[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) total[r] = warp_sum(total[r]);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < NR; ++r)
                if (row0 + r < a.M) a.y[row0 + r] += total[r];
        }
    }
}

template <uint32_t TYPE, int MODE, int NR, bool ALIGNED>
cudaError_t launch_one(const DmmvArgs& a, cudaStream_t s) {
    const bool per_slot = MODE == MODE_MOE || MODE == MODE_MOE_GATE_UP || MODE == MODE_BATCH || MODE == MODE_MOE_BATCHED;
    const uint32_t rows_per_cta =
        kWarps * ((MODE == MODE_PLAIN || MODE == MODE_SIGMOID_ACC || MODE == MODE_MOE || MODE == MODE_BATCH ||
                   MODE == MODE_MOE_GATE_UP || MODE == MODE_MOE_DOWN_ACC) ? NR : 1);
    dim3 grid((a.M + rows_per_cta - 1) / rows_per_cta, per_slot ? a.n_used : 1,
              MODE == MODE_MOE_BATCHED ? a.n_tokens : 1);
    dmmv_kernel<TYPE, MODE, NR, ALIGNED><<<grid, kWarps * 32, 0, s>>>(a);
    return cudaGetLastError();
}

template <uint32_t TYPE, bool ALIGNED>
cudaError_t launch_type(int mode, const DmmvArgs& a, cudaStream_t s) {
    // Two rows per warp once there are enough rows to fill the machine.
    const bool two = a.M >= 16384;
    switch (mode) {
        case MODE_PLAIN:
            return two ? launch_one<TYPE, MODE_PLAIN, 2, ALIGNED>(a, s) : launch_one<TYPE, MODE_PLAIN, 1, ALIGNED>(a, s);
        case MODE_GATE_UP_SWIGLU: return launch_one<TYPE, MODE_GATE_UP_SWIGLU, 1, ALIGNED>(a, s);
        case MODE_SIGMOID_ACC: return launch_one<TYPE, MODE_SIGMOID_ACC, 1, ALIGNED>(a, s);
        case MODE_MOE: return launch_one<TYPE, MODE_MOE, 1, ALIGNED>(a, s);
        // two rows (row pairs) per warp when there are rows enough to keep every SM busy regardless
        case MODE_MOE_GATE_UP:
            return (uint64_t)a.M * a.n_used >= 8192 ? launch_one<TYPE, MODE_MOE_GATE_UP, 2, ALIGNED>(a, s)
                                                    : launch_one<TYPE, MODE_MOE_GATE_UP, 1, ALIGNED>(a, s);
        case MODE_MOE_DOWN_ACC:
            return a.M >= 2560 ? launch_one<TYPE, MODE_MOE_DOWN_ACC, 2, ALIGNED>(a, s)
                               : launch_one<TYPE, MODE_MOE_DOWN_ACC, 1, ALIGNED>(a, s);
        case MODE_BATCH: return launch_one<TYPE, MODE_BATCH, 1, ALIGNED>(a, s);
        case MODE_MOE_BATCHED: return launch_one<TYPE, MODE_MOE_BATCHED, 1, ALIGNED>(a, s);
        default: return cudaErrorInvalidValue;
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

cudaError_t launch_dmmv(uint32_t type, int mode, const DmmvArgs& a, cudaStream_t s, uint64_t* launches) {
    if (a.M == 0) return cudaSuccess;
    // Below a couple of megabytes a matvec is latency-bound and one warp per row (more CTAs) wins over the
    // streaming kernels.
    const uint64_t wbytes = (uint64_t)a.M * (a.K / block_size(type)) * bytes_per_block(type) *
                            (mode == MODE_GATE_UP_SWIGLU ? 2 : 1);
    if (wbytes >= kStreamMinBytes) {
        if (warp_dmmv_eligible(type, mode, a)) return launch_warp_dmmv(type, mode, a, s, launches);
        if (q6k_dmmv_eligible(type, mode, a)) return launch_q6k_dmmv(mode, a, s, launches);
    }
    // the kernels below do not carry a pending reduction: complete it first
    if (a.consume.n) {
        const cudaError_t ec = launch_consume(a.consume, s, launches);
        if (ec != cudaSuccess) return ec;
    }
    if (wbytes >= kStreamMinBytes && mxfp4_dmmv_eligible(type, mode, a)) return launch_mxfp4_dmmv(a, s, launches);
    cudaError_t e;
    // 128-bit weight loads need every block start 16-byte aligned: true for the
    // 144/176-byte K-quant blocks when the base, the second base and the expert
    // stride are.
    const bool al = aligned16(a.A) && (a.A2 == nullptr || aligned16(a.A2)) && (a.expert_stride % 16 == 0) &&
                    aligned16(a.A_sh) && aligned16(a.A2_sh);
    switch (type) {
        case T_Q4_K: e = al ? launch_type<T_Q4_K, true>(mode, a, s) : launch_type<T_Q4_K, false>(mode, a, s); break;
        case T_Q5_K: e = al ? launch_type<T_Q5_K, true>(mode, a, s) : launch_type<T_Q5_K, false>(mode, a, s); break;
        case T_Q6_K: e = launch_type<T_Q6_K, false>(mode, a, s); break;
        case T_Q8_0: e = launch_type<T_Q8_0, false>(mode, a, s); break;
        case T_MXFP4: e = launch_type<T_MXFP4, false>(mode, a, s); break;
        case T_Q5_0: e = launch_type<T_Q5_0, false>(mode, a, s); break;
        case T_Q5_1: e = launch_type<T_Q5_1, false>(mode, a, s); break;
        case T_F16: e = launch_type<T_F16, false>(mode, a, s); break;
        case T_F32: e = launch_type<T_F32, false>(mode, a, s); break;
        default: return cudaErrorNotSupported;
    }
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

cudaError_t launch_dmmv_batch(uint32_t type, const uint8_t* A, const float* X, float* Y, uint32_t M, uint32_t K,
                              uint32_t num_cols, cudaStream_t s, uint64_t* launches) {
    // One matvec per column; grid.y is limited to 65535 columns per launch.
    for (uint32_t c0 = 0; c0 < num_cols; c0 += 65535u) {
        DmmvArgs a;
        a.A = A;
        a.x = X + (size_t)c0 * K;
        a.y = Y + (size_t)c0 * M;
        a.M = M;
        a.K = K;
        a.n_used = num_cols - c0 < 65535u ? num_cols - c0 : 65535u;
        a.x_expert_stride = K;
        cudaError_t e = launch_dmmv(type, MODE_BATCH, a, s, launches);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

cudaError_t launch_moe_dmmv_batched(uint32_t type, const uint8_t* A, const float* X, float* Y,
                                    const uint32_t* routing, uint32_t M, uint32_t K, uint64_t expert_stride,
                                    uint32_t n_experts_used, uint32_t n_tokens, uint32_t x_token_stride,
                                    uint32_t y_token_stride, uint32_t n_experts_max, uint32_t* status, cudaStream_t s,
                                    uint64_t* launches) {
    for (uint32_t t0 = 0; t0 < n_tokens; t0 += 65535u) {
        DmmvArgs a;
        a.A = A;
        a.x = X + (size_t)t0 * x_token_stride;
        a.y = Y + (size_t)t0 * y_token_stride;
        a.routing = routing + (size_t)t0 * n_experts_used;
        a.M = M;
        a.K = K;
        a.expert_stride = expert_stride;
        a.n_used = n_experts_used;
        a.n_tokens = n_tokens - t0 < 65535u ? n_tokens - t0 : 65535u;
        a.x_token_stride = x_token_stride;
        a.y_token_stride = y_token_stride;
        a.n_experts_max = n_experts_max;
        a.status = status;
        cudaError_t e = launch_dmmv(type, MODE_MOE_BATCHED, a, s, launches);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace zc
