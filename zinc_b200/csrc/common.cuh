// Shared device helpers: GGUF block geometry, unaligned loads, f16 decode,
// 6-bit K-quant scale extraction and warp reductions.
#pragma once

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace zc {

// GGML type ids (src/model/gguf.zig:38-69 in the reference project).
enum : uint32_t {
    T_F32 = 0, T_F16 = 1, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8,
    T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_BF16 = 30, T_MXFP4 = 39,
};

// Elements per block / bytes per block (src/model/gguf.zig:75-122).
__host__ __device__ constexpr uint32_t block_size(uint32_t t) {
    return (t == T_Q4_K || t == T_Q5_K || t == T_Q6_K) ? 256u
         : (t == T_Q5_0 || t == T_Q5_1 || t == T_Q8_0 || t == T_MXFP4) ? 32u
         : 1u;
}
__host__ __device__ constexpr uint32_t bytes_per_block(uint32_t t) {
    return t == T_F32 ? 4u : t == T_F16 ? 2u : t == T_BF16 ? 2u
         : t == T_Q5_0 ? 22u : t == T_Q5_1 ? 24u : t == T_Q8_0 ? 34u
         : t == T_Q4_K ? 144u : t == T_Q5_K ? 176u : t == T_Q6_K ? 210u
         : t == T_MXFP4 ? 17u : 0u;
}

__device__ __forceinline__ float h2f(uint32_t bits16) {
    return __half2float(__ushort_as_half((unsigned short)(bits16 & 0xFFFFu)));
}

// MXFP4 block scale: E8M0 exponent byte -> f32 (e == 0 maps to 2^-127, the
// subnormal 0x00400000). src/compute/forward.zig:451
__device__ __forceinline__ float e8m0_to_f32(uint32_t e) {
    return __uint_as_float(e == 0u ? 0x00400000u : (e << 23));
}

// E2M1 value table. src/compute/forward.zig:445
__device__ __forceinline__ float e2m1_to_f32(uint32_t n) {
    // magnitude from 3 bits {0,.5,1,1.5,2,3,4,6}; bit 3 is the sign
    const uint32_t m = n & 7u;
    // exponent/mantissa: m = (e << 1) | mant; e == 0 is subnormal (mant * 0.5)
    const uint32_t e = m >> 1, mant = m & 1u;
    const float mag = e == 0u ? 0.5f * (float)mant : __uint_as_float(((e + 126u) << 23) | (mant << 22));
    return (n & 8u) ? -mag : mag;
}

// Expert ids come from a routing buffer on the device, so the host cannot range-check them. An id at or
// beyond n_max (the number of experts the weight buffer holds) is recorded in the status words as
// {2, id} (reported by zc_submit_and_wait as an invalid argument) and replaced by expert 0, so that no
// kernel ever forms an address outside the expert stack.
// A routing slot that holds kSkipExpert names no expert: under expert parallelism the slots whose expert lives
// on another rank are rewritten to it (zc_moe_ep_filter). Such a slot reads no weights and contributes zeros.
constexpr uint32_t kSkipExpert = 0xFFFFFFFFu;

// A routing slot that holds kSharedExpert names the shared expert: a matrix outside the expert stack that the
// launch passes beside it (the always-on expert of a Qwen MoE layer, folded into the routed launch as one more
// slot). Without such a matrix the id is reported like any other id past the stack.
constexpr uint32_t kSharedExpert = 0xFFFFFFFEu;

__device__ __forceinline__ uint32_t checked_expert(uint32_t e, uint32_t n_max, uint32_t* status) {
    if (e < n_max) return e;
    if (status) {
        status[0] = 2u;
        status[1] = e;
    }
    return 0u;
}

// Merge weights of one head's split-K attention chunks (src/shaders/dmmv_q4k_o_proj_merge.comp:104-134):
// w[c] = exp(M_c - M_full) for chunks with L_c > 0, and 1 / L_full (0 when nothing contributed).
template <int kMaxChunks>
__device__ __forceinline__ float attn_merge_weights(const float* __restrict__ lse, const float* __restrict__ sinks,
                                                    uint32_t sink_index, uint32_t nc, float (&w)[kMaxChunks]) {
    float Mc[kMaxChunks], Lc[kMaxChunks];
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
        const float2 ml = (uint32_t)c < nc ? __ldg(reinterpret_cast<const float2*>(lse) + c) : make_float2(-INFINITY, 0.f);
        Mc[c] = ml.x;
        Lc[c] = ml.y;
    }
    float Mg = Mc[0];
#pragma unroll
    for (int c = 1; c < kMaxChunks; ++c)
        if ((uint32_t)c < nc) Mg = fmaxf(Mg, Mc[c]);
    const float sink = sinks ? __ldg(sinks + sink_index) : __int_as_float(0x7FC00000);
    const bool has_sink = !isnan(sink);
    const float Mf = has_sink ? fmaxf(Mg, sink) : Mg;
    float Lf = 0.f;
#pragma unroll
    for (int c = 0; c < kMaxChunks; ++c) {
        w[c] = ((uint32_t)c < nc && Lc[c] > 0.f) ? expf(Mc[c] - Mf) : 0.f;
        Lf += w[c] * Lc[c];
    }
    if (has_sink) Lf += expf(sink - Mf);
    return Lf > 0.f ? 1.0f / Lf : 0.f;
}

// Matrix of the expert a (non-skipped) routing slot names.
__device__ __forceinline__ const uint8_t* expert_matrix(const uint8_t* stack, const uint8_t* shared, uint32_t e_raw,
                                                        uint64_t stride, uint32_t n_max, uint32_t* status) {
    if (e_raw == kSharedExpert && shared) return shared;
    return stack + (uint64_t)checked_expert(e_raw, n_max, status) * stride;
}

// ---- loads -----------------------------------------------------------------

__device__ __forceinline__ uint32_t ldg_u32(const void* p) {
    return __ldg(reinterpret_cast<const uint32_t*>(p));
}
__device__ __forceinline__ uint4 ldg_u128(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

// NW consecutive little-endian 32-bit words starting at an arbitrarily aligned
// byte address, read with aligned 32-bit loads and funnel shifts. Touches only
// aligned words that contain at least one requested byte, so it never reads
// outside the 4-byte-aligned envelope of [p, p + 4*NW).
template <int NW>
__device__ __forceinline__ void ld_words(const uint8_t* p, uint32_t (&w)[NW]) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t* base = reinterpret_cast<const uint32_t*>(a & ~uintptr_t(3));
    const uint32_t sh = (uint32_t)(a & 3u) * 8u;
    uint32_t prev = __ldg(base);
    if (sh == 0u) {
        w[0] = prev;
#pragma unroll
        for (int i = 1; i < NW; ++i) w[i] = __ldg(base + i);
    } else {
#pragma unroll
        for (int i = 0; i < NW; ++i) {
            const uint32_t next = __ldg(base + i + 1);
            w[i] = __funnelshift_r(prev, next, sh);
            prev = next;
        }
    }
}

// 16-bit little-endian value at a 2-byte aligned or unaligned address.
__device__ __forceinline__ uint32_t ld_u16(const uint8_t* p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    if ((a & 1u) == 0u) return __ldg(reinterpret_cast<const unsigned short*>(p));
    return (uint32_t)__ldg(p) | ((uint32_t)__ldg(p + 1) << 8);
}

// ---- K-quant 6-bit scale / min extraction ------------------------------------
// s0,s1,s2 are the three little-endian words of the 12 packed scale bytes.
// Follows getScaleMinK4 (src/compute/forward.zig:229-238).
__device__ __forceinline__ uint32_t sbyte(uint32_t s0, uint32_t s1, uint32_t s2, int i) {
    const uint32_t w = i < 4 ? s0 : (i < 8 ? s1 : s2);
    return (w >> (8 * (i & 3))) & 0xFFu;
}
__device__ __forceinline__ void scale_min_k4(int j, uint32_t s0, uint32_t s1, uint32_t s2,
                                             uint32_t& sc, uint32_t& m) {
    if (j < 4) {
        sc = sbyte(s0, s1, s2, j) & 63u;
        m = sbyte(s0, s1, s2, j + 4) & 63u;
    } else {
        sc = (sbyte(s0, s1, s2, j + 4) & 0xFu) | ((sbyte(s0, s1, s2, j - 4) >> 6) << 4);
        m = (sbyte(s0, s1, s2, j + 4) >> 4) | ((sbyte(s0, s1, s2, j) >> 6) << 4);
    }
}

// ---- reductions ------------------------------------------------------------------

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

__device__ __forceinline__ float silu(float g) { return g / (1.0f + __expf(-g)); }
__device__ __forceinline__ float sigmoidf(float g) { return 1.0f / (1.0f + __expf(-g)); }

}  // namespace zc
