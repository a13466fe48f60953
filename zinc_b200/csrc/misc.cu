// Routing, activation, combine and parity kernels around the expert matmuls.
#include <float.h>

#include "dequant.cuh"
#include "kernels.h"

namespace zc {

namespace {

// ---- dequant rows -------------------------------------------------------------
template <uint32_t TYPE>
__global__ void dequant_rows_kernel(const uint8_t* __restrict__ A, float* __restrict__ out, uint64_t first_row,
                                    uint32_t K, uint64_t total) {
    const uint64_t row_bytes = (uint64_t)(K / block_size(TYPE)) * bytes_per_block(TYPE);
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t r = idx / K;
        const uint32_t i = (uint32_t)(idx - r * K);
        out[idx] = dequant_elem<TYPE>(A + (first_row + r) * row_bytes, i);
    }
}

// ---- top-k routing ---------------------------------------------------------------
// One CTA per token. Values live in dynamic shared memory; k rounds of a
// block-wide arg-max with ties to the lowest index, as the strict '>' ascending
// scans of the reference do (src/compute/forward.zig:516-529, 544-556;
// src/shaders/softmax_topk.comp:49-81).
struct ValIdx {
    float v;
    uint32_t i;
};
__device__ __forceinline__ ValIdx better(ValIdx a, ValIdx b) {
    return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// Order-preserving map of (non-NaN) floats to unsigned integers and back; -0 and +0 share a key.
__device__ __forceinline__ uint32_t float_key(float v) {
    const uint32_t b = __float_as_uint(v + 0.0f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

constexpr int kTopkThreads = 256;

__global__ void __launch_bounds__(kTopkThreads) softmax_topk_kernel(
    const float* __restrict__ logits, const float* __restrict__ bias, uint32_t* __restrict__ out,
    uint32_t n, uint32_t k, uint32_t rule, uint32_t logits_stride, uint32_t out_stride) {
    extern __shared__ float vals[];  // n values the selection runs on
    __shared__ ValIdx red[kTopkThreads / 32];
    __shared__ float red_f[kTopkThreads / 32];
    __shared__ float bcast;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* lg = logits + (size_t)blockIdx.x * logits_stride;
    uint32_t* o = out + (size_t)blockIdx.x * out_stride;
    const float floor_v = rule == 0u ? -1.0f : -INFINITY;

    float lmax = -INFINITY;
    for (uint32_t i = tid; i < n; i += kTopkThreads) {
        const float v = lg[i] + (bias ? bias[i] : 0.0f);
        vals[i] = v;
        lmax = fmaxf(lmax, v);
    }
    if (rule == 0u) {
        // softmax over all experts first
        for (int o2 = 16; o2 > 0; o2 >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xFFFFFFFFu, lmax, o2));
        if (lane == 0) red_f[warp] = lmax;
        __syncthreads();
        if (tid == 0) {
            float m = red_f[0];
            for (int w = 1; w < kTopkThreads / 32; ++w) m = fmaxf(m, red_f[w]);
            bcast = m;
        }
        __syncthreads();
        const float mx = bcast;
        float lsum = 0.f;
        for (uint32_t i = tid; i < n; i += kTopkThreads) {
            const float p = expf(vals[i] - mx);
            vals[i] = p;
            lsum += p;
        }
        lsum = warp_sum(lsum);
        __syncthreads();
        if (lane == 0) red_f[warp] = lsum;
        __syncthreads();
        if (tid == 0) {
            float s = 0.f;
            for (int w = 0; w < kTopkThreads / 32; ++w) s += red_f[w];
            bcast = s;
        }
        __syncthreads();
        const float sum = bcast;
        if (sum > 0.f)
            for (uint32_t i = tid; i < n; i += kTopkThreads) vals[i] = vals[i] / sum;
    }
    __syncthreads();

    for (uint32_t ki = 0; ki < k; ++ki) {
        ValIdx best{floor_v, 0u};
        for (uint32_t i = tid; i < n; i += kTopkThreads) {
            const float v = vals[i];
            if (v > best.v) best = ValIdx{v, i};
        }
        for (int o2 = 16; o2 > 0; o2 >>= 1) {
            ValIdx other{__shfl_xor_sync(0xFFFFFFFFu, best.v, o2), __shfl_xor_sync(0xFFFFFFFFu, best.i, o2)};
            best = better(best, other);
        }
        if (lane == 0) red[warp] = best;
        __syncthreads();
        if (tid == 0) {
            ValIdx b = red[0];
            for (int w = 1; w < kTopkThreads / 32; ++w) b = better(b, red[w]);
            // nothing above the floor: the reference's scans leave index 0
            if (!(b.v > floor_v)) b = ValIdx{rule == 0u ? floor_v : vals[0], 0u};
            o[ki] = b.i;
            o[k + ki] = __float_as_uint(b.v);
            vals[b.i] = rule == 0u ? -2.0f : -INFINITY;  // never selected again
        }
        __syncthreads();
    }

    if (tid == 0) {
        if (rule == 0u) {
            float ws = 0.f;
            for (uint32_t i = 0; i < k; ++i) ws += __uint_as_float(o[k + i]);
            if (ws > 0.f)
                for (uint32_t i = 0; i < k; ++i) o[k + i] = __float_as_uint(__uint_as_float(o[k + i]) / ws);
        } else {
            float mx = -INFINITY;
            for (uint32_t i = 0; i < k; ++i) mx = fmaxf(mx, __uint_as_float(o[k + i]));
            float sum = 0.f;
            for (uint32_t i = 0; i < k; ++i) {
                const float w = expf(__uint_as_float(o[k + i]) - mx);
                o[k + i] = __float_as_uint(w);
                sum += w;
            }
            if (sum > 0.f)
                for (uint32_t i = 0; i < k; ++i) o[k + i] = __float_as_uint(__uint_as_float(o[k + i]) / sum);
        }
    }
}

// One warp selects for one token: lane l holds experts l, l + 32, ... in registers. Ids go to o[0..k), weights (f32 bits) to o[wofs .. wofs + k): wofs = k is the
// reference's layout, a larger wofs leaves room for slots behind the selected ones. The logits are read past
// L1 (they may have been written by other CTAs of the same launch).
// Where the selection takes its logits from, in two steps so that all of a lane's reads are in flight before any
// of them is waited for: first(i) issues the read, value(i, q) completes it.
struct LogitsPlain {  // logits in global memory, read past L1
    const float* lg;
    __device__ __forceinline__ uint2 first(uint32_t i) const { return make_uint2(__float_as_uint(__ldcg(lg + i)), 1u); }
    __device__ __forceinline__ float value(uint32_t, uint2 q) const { return __uint_as_float(q.x); }
};

template <int VPL, typename Load>
__device__ __forceinline__ void softmax_topk_warp(const Load& load, const float* __restrict__ bias, uint32_t* o,
                                                  uint32_t n, uint32_t k, uint32_t rule, uint32_t wofs, int lane,
                                                  uint32_t* my_id = nullptr, uint32_t* my_w = nullptr) {
    const float floor_v = rule == 0u ? -1.0f : -INFINITY;
    const float gone = rule == 0u ? -2.0f : -INFINITY;  // never selected (again)

    float v[VPL];
    uint2 raw[VPL];
    float lmax = -INFINITY;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const uint32_t i = lane + 32 * j;
        raw[j] = i < n ? load.first(i) : make_uint2(0xFF800000u, 1u);
    }
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const uint32_t i = lane + 32 * j;
        v[j] = i < n ? load.value(i, raw[j]) : -INFINITY;
    }
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
        const uint32_t i = lane + 32 * j;
        if (bias && i < n) v[j] += bias[i];
        lmax = fmaxf(lmax, v[j]);
    }
    if (rule == 0u) {  // softmax over all experts first
        for (int o2 = 16; o2 > 0; o2 >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xFFFFFFFFu, lmax, o2));
        float lsum = 0.f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const uint32_t i = lane + 32 * j;
            v[j] = i < n ? expf(v[j] - lmax) : 0.f;
            lsum += v[j];
        }
        const float sum = warp_sum(lsum);
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const uint32_t i = lane + 32 * j;
            if (sum > 0.f) v[j] = v[j] / sum;
            if (i >= n) v[j] = gone;
        }
    }
    const float v0 = __shfl_sync(0xFFFFFFFFu, v[0], 0);  // expert 0, for the "nothing above the floor" case
    // Up to 32 selections stay in registers (selection ki in lane ki) and reach memory once, at the end: a
    // round trip through global memory per selection and per weight costs more than the whole selection.
    const bool in_regs = k <= 32;
    float sel_v = 0.f;
    uint32_t sel_i = 0u;
    for (uint32_t ki = 0; ki < k; ++ki) {
        ValIdx best{floor_v, 0u};
#pragma unroll
        for (int j = 0; j < VPL; ++j)
            if (v[j] > best.v) best = ValIdx{v[j], (uint32_t)(lane + 32 * j)};
        // arg-max over the warp with two integer reductions: the largest value (as an order-preserving key, -0
        // folded into +0), then the lowest index among the lanes that hold it
        const uint32_t kmax = __reduce_max_sync(0xFFFFFFFFu, float_key(best.v));
        const uint32_t imin = __reduce_min_sync(0xFFFFFFFFu, float_key(best.v) == kmax ? best.i : 0xFFFFFFFFu);
        best = ValIdx{key_float(kmax), imin};
        if (!(best.v > floor_v)) best = ValIdx{rule == 0u ? floor_v : v0, 0u};
        if (in_regs) {
            if ((uint32_t)lane == ki) {
                sel_v = best.v;
                sel_i = best.i;
            }
        } else if (lane == 0) {
            o[ki] = best.i;
            o[wofs + ki] = __float_as_uint(best.v);
        }
#pragma unroll
        for (int j = 0; j < VPL; ++j)
            if (best.i == (uint32_t)(lane + 32 * j)) v[j] = gone;
    }
    if (in_regs) {
        // the sums run over the selections in order, as the sequential loops of the reference do
        float w;
        if (rule == 0u) {
            float ws = 0.f;
            for (uint32_t i = 0; i < k; ++i) ws += __shfl_sync(0xFFFFFFFFu, sel_v, (int)i);
            w = ws > 0.f ? sel_v / ws : sel_v;
        } else {
            float mx = (uint32_t)lane < k ? sel_v : -INFINITY;
            for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o2));
            const float e = expf(sel_v - mx);
            float sum = 0.f;
            for (uint32_t i = 0; i < k; ++i) sum += __shfl_sync(0xFFFFFFFFu, e, (int)i);
            w = sum > 0.f ? e / sum : e;
        }
        if ((uint32_t)lane < k) {
            o[lane] = sel_i;
            o[wofs + lane] = __float_as_uint(w);
        }
        if (my_id) {  // lane ki's selection, for a caller that goes on with it
            *my_id = sel_i;
            *my_w = __float_as_uint(w);
        }
        return;
    }
    if (lane == 0) {
        if (rule == 0u) {
            float ws = 0.f;
            for (uint32_t i = 0; i < k; ++i) ws += __uint_as_float(o[wofs + i]);
            if (ws > 0.f)
                for (uint32_t i = 0; i < k; ++i) o[wofs + i] = __float_as_uint(__uint_as_float(o[wofs + i]) / ws);
        } else {
            float mx = -INFINITY;
            for (uint32_t i = 0; i < k; ++i) mx = fmaxf(mx, __uint_as_float(o[wofs + i]));
            float sum = 0.f;
            for (uint32_t i = 0; i < k; ++i) {
                const float w = expf(__uint_as_float(o[wofs + i]) - mx);
                o[wofs + i] = __float_as_uint(w);
                sum += w;
            }
            if (sum > 0.f)
                for (uint32_t i = 0; i < k; ++i) o[wofs + i] = __float_as_uint(__uint_as_float(o[wofs + i]) / sum);
        }
    }
}

// The same selection for up to 32 * VPL experts with one warp per token and no block-wide barrier: lane l
// holds experts l, l + 32, ... in registers. A router has at most a few hundred experts, and the k rounds
// of block-wide barriers of the kernel above cost more than the arithmetic.
template <int VPL>
__global__ void __launch_bounds__(128) softmax_topk_warp_kernel(
    const float* __restrict__ logits, const float* __restrict__ bias, uint32_t* __restrict__ out,
    uint32_t n, uint32_t k, uint32_t rule, uint32_t n_tokens, uint32_t logits_stride, uint32_t out_stride) {
    const int lane = threadIdx.x & 31;
    const uint32_t tok = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (tok >= n_tokens) return;
    softmax_topk_warp<VPL>(LogitsPlain{logits + (size_t)tok * logits_stride}, bias, out + (size_t)tok * out_stride, n, k,
                           rule, k, lane);
}

// ---- combine / activation ------------------------------------------------------------
// src/shaders/moe_weighted_acc.comp:23-33
__global__ void moe_weighted_acc_kernel(float* __restrict__ a, const float* __restrict__ b,
                                        const uint32_t* __restrict__ routing, uint32_t n, uint32_t n_used,
                                        uint32_t src_stride) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float sum = 0.f;
    for (uint32_t j = 0; j < n_used; ++j)
        sum = fmaf(__uint_as_float(__ldg(routing + n_used + j)), b[(size_t)j * src_stride + i], sum);
    a[i] += sum;
}

// src/shaders/swiglu.comp:25-33, src/shaders/swiglu_oai.comp:24-34
template <bool OAI>
__global__ void swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ y,
                              uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (OAI) {
        const float g = fminf(gate[i], 7.0f);
        const float u = fmaxf(-7.0f, fminf(up[i], 7.0f));
        y[i] = (g / (1.0f + expf(1.702f * (-g)))) * (u + 1.0f);
    } else {
        const float g = gate[i];
        y[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

template <bool OAI>
__device__ __forceinline__ float swiglu_one(float g, float u) {
    if (OAI) {
        g = fminf(g, 7.0f);
        u = fmaxf(-7.0f, fminf(u, 7.0f));
        return (g / (1.0f + expf(1.702f * (-g)))) * (u + 1.0f);
    }
    return (g / (1.0f + expf(-g))) * u;
}

// the same element by element, four per thread
template <bool OAI>
__global__ void swiglu4_kernel(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ y,
                               uint32_t n4) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 g = __ldg(reinterpret_cast<const float4*>(gate) + i);
    const float4 u = __ldg(reinterpret_cast<const float4*>(up) + i);
    reinterpret_cast<float4*>(y)[i] = make_float4(swiglu_one<OAI>(g.x, u.x), swiglu_one<OAI>(g.y, u.y),
                                                  swiglu_one<OAI>(g.z, u.z), swiglu_one<OAI>(g.w, u.w));
}

// ---- per-expert biases (GPT-OSS) ------------------------------------------------------------
// src/shaders/bias_add.comp:19-23: out[i] += bias[src_offset + i]
__global__ void bias_add_kernel(float* __restrict__ out, const float* __restrict__ bias, uint32_t n,
                                uint32_t src_offset) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] += bias[(size_t)src_offset + i];
}

// The reference adds ffn_gate_exps_bias / ffn_up_exps_bias to an expert's gate and up vectors and then applies
// the activation, expert by expert (src/compute/forward.zig:6841-6860). Here for all selected slots at once, the
// expert of a slot read from the routing buffer: y[s][i] = act(gate[s][i] + gb[e_s][i], up[s][i] + ub[e_s][i]).
template <bool OAI>
__global__ void moe_bias_act_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                    const float* __restrict__ gate_bias, const float* __restrict__ up_bias,
                                    const uint32_t* __restrict__ routing, float* __restrict__ y, uint32_t M,
                                    uint32_t n_experts, uint32_t* status) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
    if (i >= M) return;
    const uint32_t e_raw = __ldg(routing + s);
    if (e_raw == kSkipExpert) {  // no expert in this slot on this rank
        y[(size_t)s * M + i] = 0.f;
        return;
    }
    const uint32_t e = checked_expert(e_raw, n_experts, status);
    const size_t o = (size_t)s * M + i, b = (size_t)e * M + i;
    const float g = gate[o] + (gate_bias ? gate_bias[b] : 0.f);
    const float u = up[o] + (up_bias ? up_bias[b] : 0.f);
    y[o] = swiglu_one<OAI>(g, u);
}

// The down projection's bias enters the weighted sum of the experts' outputs
// (src/compute/forward.zig:6923-6927 followed by the scale-accumulate): a[i] += sum_s w_s * bias[e_s][i].
__global__ void moe_weighted_bias_acc_kernel(float* __restrict__ a, const float* __restrict__ bias,
                                             const uint32_t* __restrict__ routing, uint32_t n, uint32_t n_used,
                                             uint32_t n_experts, uint32_t* status) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float sum = 0.f;
    for (uint32_t s = 0; s < n_used; ++s) {
        const uint32_t e_raw = __ldg(routing + s);
        if (e_raw == kSkipExpert) continue;
        const uint32_t e = checked_expert(e_raw, n_experts, status);
        sum = fmaf(__uint_as_float(__ldg(routing + n_used + s)), bias[(size_t)e * n + i], sum);
    }
    a[i] += sum;
}

// ---- expert parallelism: keep the slots whose expert this rank holds ---------------------------------
// out[s] = in[s] - lo when lo <= in[s] < hi, else the "no expert" mark; the k weights are copied. Rows of 2k
// words, one per token.
__global__ void moe_ep_filter_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, uint32_t k,
                                     uint32_t n_tokens, uint32_t stride_in, uint32_t stride_out, uint32_t lo,
                                     uint32_t hi) {
    // rows of out hold the ids and the weights, or (stride_out < 2k) the ids alone: the flattened id table the
    // cross-token calls take
    const uint32_t per = stride_out < 2 * k ? k : 2 * k;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tokens * per) return;
    const uint32_t tok = i / per, j = i - tok * per;
    const uint32_t v = in[(size_t)tok * stride_in + j];
    out[(size_t)tok * stride_out + j] = j >= k ? v : (v >= lo && v < hi) ? v - lo : 0xFFFFFFFFu;
}

// ---- merge of split-K attention partials ----------------------------------------------------
// One thread per output element (src/shaders/dmmv_q4k_o_proj_merge.comp:104-148, without the matvec: the form
// used when the streaming kernel cannot build the vector while loading it).
__global__ void attn_merge_kernel(const MergeArgs m, float* __restrict__ out) {
    const uint32_t k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= m.n_heads * m.head_dim) return;
    const uint32_t head = k / m.head_dim, d = k - head * m.head_dim;
    const float* lse = m.partial + (size_t)m.n_heads * m.n_chunks * m.head_dim + (size_t)head * m.n_chunks * 2;
    float acc = 0.f, inv;
    if (m.n_chunks <= 16) {
        float w[16];
        inv = attn_merge_weights<16>(lse, m.sinks, m.sink_offset + head, m.n_chunks, w);
#pragma unroll
        for (int c = 0; c < 16; ++c)
            if ((uint32_t)c < m.n_chunks)
                acc = fmaf(w[c], __ldg(m.partial + ((size_t)head * m.n_chunks + c) * m.head_dim + d), acc);
    } else {
        inv = 0.f;  // refused on the host
    }
    out[k] = acc * inv;
}

// ---- fused RMS norm + f32 router matvec -------------------------------------------------
// src/shaders/rms_norm_dmmv_f32.comp:68-127: every CTA recomputes rms_inv = rsqrt(mean(x^2) + eps) (same
// reads in the same order everywhere), CTA 0 also writes the normalised vector
// norm_out[i] = w[i] * (x[i] * rms_inv), and each CTA dots one router row with the normalised vector.
// One CTA per row: a router has a few hundred rows at most, so rows are the only parallelism.
// With norm_w == nullptr the kernel is a plain f32 matvec for small M (no normalisation).
constexpr int kRouterThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();  // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kRouterThreads / 32; ++i) t += scratch[i];
    return t;
}

__global__ void __launch_bounds__(kRouterThreads) rms_norm_dmmv_f32_kernel(
    const float* __restrict__ x, const float* __restrict__ norm_w, const float* __restrict__ W,
    float* __restrict__ norm_out, float* __restrict__ y, uint32_t M, uint32_t K, float eps,
    const float* __restrict__ W2, float* __restrict__ y2) {
    __shared__ float scratch[kRouterThreads / 32];
    // CTAs [0, M) take the rows of W, CTAs [M, 2M) those of a second matrix on the same normalised vector
    // (src/shaders/rms_norm_dmmv_q4k_alpha_beta.comp:64-133: the alpha and beta projections of an SSM layer)
    const uint32_t tid = threadIdx.x;
    const bool second = blockIdx.x >= M;
    const uint32_t row = second ? blockIdx.x - M : blockIdx.x;
    if (second) {
        W = W2;
        y = y2;
    }
    const uint32_t K4 = K >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float rms_inv = 1.f;
    if (norm_w) {
        float ss = 0.f;
        for (uint32_t i = tid; i < K4; i += kRouterThreads) {
            const float4 v = __ldg(x4 + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum(ss, scratch);
        rms_inv = rsqrtf(ss / (float)K + eps);
    }
    const float4* w4 = reinterpret_cast<const float4*>(norm_w);
    const float4* r4 = reinterpret_cast<const float4*>(W + (size_t)row * K);
    float sum = 0.f;
    for (uint32_t i = tid; i < K4; i += kRouterThreads) {
        float4 v = __ldg(x4 + i);
        if (norm_w) {
            const float4 w = __ldg(w4 + i);
            v = make_float4(w.x * (v.x * rms_inv), w.y * (v.y * rms_inv), w.z * (v.z * rms_inv), w.w * (v.w * rms_inv));
            if (blockIdx.x == 0 && norm_out) reinterpret_cast<float4*>(norm_out)[i] = v;
        }
        const float4 r = __ldg(r4 + i);
        sum += v.x * r.x + v.y * r.y + v.z * r.z + v.w * r.w;
    }
    sum = block_sum(sum, scratch);
    if (tid == 0) y[row] = sum;
}

// ---- router matvec + expert selection in one launch ----------------------------------------------
// The f32 router of one token (optionally behind the RMS norm, as above) and the selection that follows it
// (src/compute/forward.zig:6139-6190: router DMMV, then softmax_topk): one CTA per router row; every CTA hands
// its logit to CTA 0 as a tagged 64-bit value, and CTA 0's first warp, once its own row is done, collects them
// (bounded polls) and runs the one-warp selection. Behind the k selected slots the routing buffer can carry one more slot for the
// shared expert (id kSharedExpert, weight 1), and a second routing buffer can receive the same selection as an
// expert-parallel rank sees it: ids in [e_lo, e_hi) renumbered from zero, every other slot marked "no expert
// here", the shared slot kept only where `local_shared` says so.
// Launched as a programmatic dependent: the row of router weights is in registers before the wait for the
// previous kernel, and the next kernel of the stream is released at once.
struct RouterArgs {
    const float* x;
    const float* norm_w;
    const float* W;
    const float* bias;
    float* norm_out;
    float* logits;
    uint32_t* routing;
    uint32_t* routing_local;
    uint2* tagged;    // [n_experts] {logit bits, 1}: how the rows' CTAs hand their logits to CTA 0 ({0, 0} between launches)
    uint32_t* status;
    uint32_t spin_limit;
    uint32_t n_experts, K, k, rule, shared, e_lo, e_hi, local_shared;
    float eps;
};
constexpr int kRouterPrefetch = 4;  // float4 per thread held across the dependency wait (K <= 4096)

__global__ void __launch_bounds__(kRouterThreads) moe_router_topk_kernel(const RouterArgs a) {
    __shared__ float scratch[kRouterThreads / 32];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t tid = threadIdx.x, row = blockIdx.x;
    const uint32_t K4 = a.K >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(a.W + (size_t)row * a.K);
    float4 wreg[kRouterPrefetch];
#pragma unroll
    for (int j = 0; j < kRouterPrefetch; ++j) {
        const uint32_t i = tid + j * kRouterThreads;
        wreg[j] = i < K4 ? __ldg(r4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float4* x4 = reinterpret_cast<const float4*>(a.x);
    float rms_inv = 1.f;
    if (a.norm_w) {
        float ss = 0.f;
        for (uint32_t i = tid; i < K4; i += kRouterThreads) {
            const float4 v = __ldg(x4 + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_sum(ss, scratch);
        rms_inv = rsqrtf(ss / (float)a.K + a.eps);
    }
    const float4* w4 = reinterpret_cast<const float4*>(a.norm_w);
    float sum = 0.f;
    auto term = [&](uint32_t i, const float4 r) {
        float4 v = __ldg(x4 + i);
        if (a.norm_w) {
            const float4 w = __ldg(w4 + i);
            v = make_float4(w.x * (v.x * rms_inv), w.y * (v.y * rms_inv), w.z * (v.z * rms_inv), w.w * (v.w * rms_inv));
            if (row == 0 && a.norm_out) reinterpret_cast<float4*>(a.norm_out)[i] = v;
        }
        sum += v.x * r.x + v.y * r.y + v.z * r.z + v.w * r.w;
    };
#pragma unroll
    for (int j = 0; j < kRouterPrefetch; ++j) {
        const uint32_t i = tid + j * kRouterThreads;
        if (i < K4) term(i, wreg[j]);
    }
    for (uint32_t i = tid + kRouterPrefetch * kRouterThreads; i < K4; i += kRouterThreads) term(i, __ldg(r4 + i));
    sum = block_sum(sum, scratch);
    if (tid == 0) {
        a.logits[row] = sum;
        a.tagged[row] = make_uint2(__float_as_uint(sum), 1u);  // value and tag in one 64-bit store: no fence, no flag
    }
    if (row != 0 || tid >= 32) return;
    // ---- CTA 0's first warp collects every row's logit (bounded polls; the tags are cleared for the next launch)
    // and runs the selection ----
    const uint32_t n = a.n_experts, k = a.k, slots = k + a.shared;
    uint32_t* o = a.routing;
    uint32_t id = 0u, wt = 0u;  // lane j's selection (k <= 32)
    struct LogitsTagged {
        const RouterArgs& a;
        __device__ __forceinline__ uint2 first(uint32_t i) const {
            uint2 q;
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(q.x), "=r"(q.y) : "l"(a.tagged + i) : "memory");
            return q;
        }
        __device__ __forceinline__ float value(uint32_t i, uint2 q) const {
            uint2* p = a.tagged + i;
            uint32_t spins = 0;
            while (q.y == 0u) {
                if (++spins > a.spin_limit) {
                    a.status[0] = 1;
                    a.status[1] = 500u;
                    break;
                }
                asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(q.x), "=r"(q.y) : "l"(p) : "memory");
            }
            *p = make_uint2(0u, 0u);
            return __uint_as_float(q.x);
        }
    };
    const LogitsTagged load{a};
    if (n <= 32) softmax_topk_warp<1>(load, a.bias, o, n, k, a.rule, slots, (int)tid, &id, &wt);
    else if (n <= 256) softmax_topk_warp<8>(load, a.bias, o, n, k, a.rule, slots, (int)tid, &id, &wt);
    else softmax_topk_warp<32>(load, a.bias, o, n, k, a.rule, slots, (int)tid, &id, &wt);
    if (tid == 0 && a.shared) {
        o[k] = kSharedExpert;
        o[slots + k] = 0x3F800000u;
    }
    if (a.routing_local) {
        if (k > 32) __syncwarp();  // the selections went through memory, written by lane 0
        for (uint32_t j = tid; j < slots; j += 32) {
            if (k > 32 && j < k) {
                id = o[j];
                wt = o[slots + j];
            }
            uint32_t lid;
            if (j >= k) {
                lid = a.local_shared ? kSharedExpert : kSkipExpert;
                wt = 0x3F800000u;
            } else {
                lid = (id >= a.e_lo && id < a.e_hi) ? id - a.e_lo : kSkipExpert;
            }
            a.routing_local[j] = lid;
            a.routing_local[slots + j] = wt;
        }
    }
}

// src/shaders/count_experts.comp:58-83: one CTA per expert.
__global__ void __launch_bounds__(256) count_experts_kernel(const uint32_t* __restrict__ a,
                                                            uint32_t* __restrict__ counts, uint32_t ne00,
                                                            uint32_t ne01, uint32_t nb00, uint32_t nb01,
                                                            uint32_t a_offset) {
    __shared__ uint32_t red[8];
    const uint32_t e = blockIdx.x;
    const uint32_t total = ne00 * ne01;
    uint32_t c = 0;
    for (uint32_t idx = threadIdx.x; idx < total; idx += 256) {
        const uint32_t i01 = idx / ne00, i00 = idx - i01 * ne00;
        c += __ldg(a + a_offset + (size_t)i01 * nb01 + (size_t)i00 * nb00) == e;
    }
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t s = 0;
        for (int w = 0; w < 8; ++w) s += red[w];
        counts[e] = s;
    }
}

// src/shaders/metal/moe_route_pack.metal:13-36. One warp per expert; the route
// list keeps token order through a ballot prefix.
__global__ void moe_route_pack_kernel(const uint32_t* __restrict__ routing, uint32_t* __restrict__ counts,
                                      uint32_t* __restrict__ ids, uint32_t n_tokens, uint32_t n_experts, uint32_t k,
                                      uint32_t routing_stride, uint32_t ids_stride) {
    const uint32_t e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (e >= n_experts) return;
    const uint32_t total = n_tokens * k;
    uint32_t n = 0;
    for (uint32_t base = 0; base < total; base += 32) {
        const uint32_t idx = base + lane;
        bool hit = false;
        if (idx < total) {
            const uint32_t t = idx / k, s = idx - t * k;
            hit = __ldg(routing + (size_t)t * routing_stride + s) == e;
        }
        const uint32_t mask = __ballot_sync(0xFFFFFFFFu, hit);
        if (hit) ids[(size_t)e * ids_stride + n + __popc(mask & ((1u << lane) - 1u))] = idx;
        n += __popc(mask);
    }
    if (lane == 0) counts[e] = n;
}

// src/shaders/metal/moe_route_scatter.metal:20-96
__global__ void moe_route_scatter_kernel(const uint32_t* __restrict__ routing, const float* __restrict__ src,
                                         float* __restrict__ dst, uint32_t n_tokens, uint32_t hidden, uint32_t k,
                                         uint32_t routing_stride) {
    const uint64_t id = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (uint64_t)n_tokens * hidden) return;
    const uint32_t t = (uint32_t)(id / hidden), d = (uint32_t)(id - (uint64_t)t * hidden);
    const uint32_t* row = routing + (size_t)t * routing_stride;
    float sum = 0.f;
    for (uint32_t s = 0; s < k; ++s) {
        if (__ldg(row + s) == kSkipExpert) continue;  // no expert in this slot on this rank: its src row was never written
        sum = fmaf(__uint_as_float(__ldg(row + k + s)), src[((size_t)t * k + s) * hidden + d], sum);
    }
    dst[id] += sum;
}

}  // namespace

cudaError_t launch_dequant_rows(uint32_t type, const uint8_t* A, float* out, uint64_t first_row, uint32_t n_rows,
                                uint32_t K, cudaStream_t s, uint64_t* launches) {
    const uint64_t total = (uint64_t)n_rows * K;
    if (total == 0) return cudaSuccess;
    const int threads = 256;
    const uint32_t blocks = (uint32_t)((total + threads - 1) / threads < 148u * 64u ? (total + threads - 1) / threads
                                                                                    : 148u * 64u);
#define ZC_DQ(T) \
    case T: dequant_rows_kernel<T><<<blocks, threads, 0, s>>>(A, out, first_row, K, total); break;
    switch (type) {
        ZC_DQ(T_F32) ZC_DQ(T_F16) ZC_DQ(T_Q8_0) ZC_DQ(T_Q4_K) ZC_DQ(T_Q5_K) ZC_DQ(T_Q6_K)
        ZC_DQ(T_Q5_0) ZC_DQ(T_Q5_1) ZC_DQ(T_MXFP4)
        default: return cudaErrorNotSupported;
    }
#undef ZC_DQ
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_softmax_topk(const float* logits, const float* bias, uint32_t* out, uint32_t n_experts,
                                uint32_t k, uint32_t rule, uint32_t n_tokens, uint32_t logits_stride,
                                uint32_t out_stride, cudaStream_t s, uint64_t* launches) {
    if (n_tokens == 0) return cudaSuccess;
    if (n_experts <= 1024) {  // one warp per token, values in registers
        const uint32_t grid = (n_tokens + 3) / 4;
        if (n_experts <= 32)
            softmax_topk_warp_kernel<1><<<grid, 128, 0, s>>>(logits, bias, out, n_experts, k, rule, n_tokens,
                                                             logits_stride, out_stride);
        else if (n_experts <= 256)
            softmax_topk_warp_kernel<8><<<grid, 128, 0, s>>>(logits, bias, out, n_experts, k, rule, n_tokens,
                                                             logits_stride, out_stride);
        else
            softmax_topk_warp_kernel<32><<<grid, 128, 0, s>>>(logits, bias, out, n_experts, k, rule, n_tokens,
                                                              logits_stride, out_stride);
        if (launches) ++*launches;
        return cudaGetLastError();
    }
    const size_t smem = (size_t)n_experts * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(softmax_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
    }
    softmax_topk_kernel<<<n_tokens, kTopkThreads, smem, s>>>(logits, bias, out, n_experts, k, rule, logits_stride,
                                                             out_stride);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_moe_router_topk(const float* x, const float* norm_w, const float* W, const float* bias,
                                   float* norm_out, float* logits, uint32_t* routing, uint32_t* routing_local,
                                   uint2* tagged, uint32_t* status, uint32_t spin_limit, uint32_t n_experts, uint32_t K, uint32_t k, uint32_t rule,
                                   uint32_t shared, uint32_t e_lo, uint32_t e_hi, uint32_t local_shared, float eps,
                                   cudaStream_t s, uint64_t* launches) {
    if (n_experts == 0 || n_experts > 1024 || (K & 3u)) return cudaErrorNotSupported;
    RouterArgs a{x, norm_w, W, bias, norm_out, logits, routing, routing_local, tagged, status, spin_limit,
                 n_experts, K, k, rule, shared, e_lo, e_hi, local_shared, eps};
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_experts, 1, 1);
    cfg.blockDim = dim3(kRouterThreads, 1, 1);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, moe_router_topk_kernel, a);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

cudaError_t launch_moe_weighted_acc(float* a, const float* b, const uint32_t* routing, uint32_t n, uint32_t n_used,
                                    uint32_t src_stride, cudaStream_t s, uint64_t* launches) {
    if (n == 0) return cudaSuccess;
    moe_weighted_acc_kernel<<<(n + 255) / 256, 256, 0, s>>>(a, b, routing, n, n_used, src_stride);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_swiglu(const float* gate, const float* up, float* y, uint32_t n, bool oai, cudaStream_t s,
                          uint64_t* launches) {
    if (n == 0) return cudaSuccess;
    const bool vec = n >= 4096 && (n & 3u) == 0 &&
                     ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) |
                       reinterpret_cast<uintptr_t>(y)) & 15u) == 0;
    if (vec) {  // prefill-sized vectors: 16 bytes per thread and array
        const uint32_t n4 = n / 4;
        if (oai) swiglu4_kernel<true><<<(n4 + 255) / 256, 256, 0, s>>>(gate, up, y, n4);
        else swiglu4_kernel<false><<<(n4 + 255) / 256, 256, 0, s>>>(gate, up, y, n4);
    } else if (oai) swiglu_kernel<true><<<(n + 255) / 256, 256, 0, s>>>(gate, up, y, n);
    else swiglu_kernel<false><<<(n + 255) / 256, 256, 0, s>>>(gate, up, y, n);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_bias_add(float* out, const float* bias, uint32_t n, uint32_t src_offset, cudaStream_t s,
                            uint64_t* launches) {
    if (n == 0) return cudaSuccess;
    bias_add_kernel<<<(n + 255) / 256, 256, 0, s>>>(out, bias, n, src_offset);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_moe_bias_act(const float* gate, const float* up, const float* gate_bias, const float* up_bias,
                                const uint32_t* routing, float* y, uint32_t M, uint32_t n_used, uint32_t n_experts,
                                bool oai, uint32_t* status, cudaStream_t s, uint64_t* launches) {
    const dim3 grid((M + 255) / 256, n_used);
    if (oai) moe_bias_act_kernel<true><<<grid, 256, 0, s>>>(gate, up, gate_bias, up_bias, routing, y, M, n_experts, status);
    else moe_bias_act_kernel<false><<<grid, 256, 0, s>>>(gate, up, gate_bias, up_bias, routing, y, M, n_experts, status);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_moe_weighted_bias_acc(float* a, const float* bias, const uint32_t* routing, uint32_t n,
                                         uint32_t n_used, uint32_t n_experts, uint32_t* status, cudaStream_t s,
                                         uint64_t* launches) {
    moe_weighted_bias_acc_kernel<<<(n + 255) / 256, 256, 0, s>>>(a, bias, routing, n, n_used, n_experts, status);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_attn_merge(const MergeArgs& m, float* out, cudaStream_t s, uint64_t* launches) {
    const uint32_t n = m.n_heads * m.head_dim;
    attn_merge_kernel<<<(n + 255) / 256, 256, 0, s>>>(m, out);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_moe_ep_filter(const uint32_t* in, uint32_t* out, uint32_t k, uint32_t n_tokens, uint32_t stride_in,
                                 uint32_t stride_out, uint32_t lo, uint32_t hi, cudaStream_t s, uint64_t* launches) {
    const uint32_t n = n_tokens * 2 * k;
    moe_ep_filter_kernel<<<(n + 255) / 256, 256, 0, s>>>(in, out, k, n_tokens, stride_in, stride_out, lo, hi);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_count_experts(const uint32_t* a, uint32_t* counts, uint32_t n_experts, uint32_t ne00,
                                 uint32_t ne01, uint32_t nb00, uint32_t nb01, uint32_t a_offset, cudaStream_t s,
                                 uint64_t* launches) {
    count_experts_kernel<<<n_experts, 256, 0, s>>>(a, counts, ne00, ne01, nb00, nb01, a_offset);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_moe_route_pack(const uint32_t* routing, uint32_t* counts, uint32_t* ids, uint32_t n_tokens,
                                  uint32_t n_experts, uint32_t k, uint32_t routing_stride, uint32_t ids_stride,
                                  cudaStream_t s, uint64_t* launches) {
    const int warps = 4;
    moe_route_pack_kernel<<<(n_experts + warps - 1) / warps, warps * 32, 0, s>>>(routing, counts, ids, n_tokens,
                                                                                n_experts, k, routing_stride,
                                                                                ids_stride);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_moe_route_scatter(const uint32_t* routing, const float* src, float* dst, uint32_t n_tokens,
                                     uint32_t hidden, uint32_t k, uint32_t routing_stride, cudaStream_t s,
                                     uint64_t* launches) {
    const uint64_t total = (uint64_t)n_tokens * hidden;
    if (total == 0) return cudaSuccess;
    moe_route_scatter_kernel<<<(uint32_t)((total + 255) / 256), 256, 0, s>>>(routing, src, dst, n_tokens, hidden, k,
                                                                             routing_stride);
    if (launches) ++*launches;
    return cudaGetLastError();
}

cudaError_t launch_rms_norm_dmmv_f32(const float* x, const float* norm_w, const float* W, float* norm_out, float* y,
                                     uint32_t M, uint32_t K, float eps, cudaStream_t s, uint64_t* launches,
                                     const float* W2, float* y2) {
    rms_norm_dmmv_f32_kernel<<<W2 ? 2 * M : M, kRouterThreads, 0, s>>>(x, norm_w, W, norm_out, y, M, K, eps, W2, y2);
    if (launches) ++*launches;
    return cudaGetLastError();
}

}  // namespace zc
