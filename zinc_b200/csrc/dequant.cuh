// Element-wise dequantisation with the reference's exact rounding sequence:
// every product, sum and difference is a separately rounded f32 operation
// (__fmul_rn / __fadd_rn / __fsub_rn are never contracted into an FMA), so the
// result is bit-identical to dequantRow of the reference
// (src/compute/forward.zig:242-465; Q5_1: src/compute/forward_metal.zig:6704-6729).
#pragma once

#include "common.cuh"

namespace zc {

// Value of element i (0 <= i < K) of the row that starts at `row`.
template <uint32_t TYPE>
__device__ __forceinline__ float dequant_elem(const uint8_t* __restrict__ row, uint32_t i) {
    if constexpr (TYPE == T_F32) {
        uint32_t w[1];
        ld_words<1>(row + 4 * (size_t)i, w);
        return __uint_as_float(w[0]);
    } else if constexpr (TYPE == T_F16) {
        return h2f(ld_u16(row + 2 * (size_t)i));
    } else if constexpr (TYPE == T_Q8_0) {
        const uint8_t* b = row + (size_t)(i >> 5) * 34;
        const float d = h2f(ld_u16(b));
        return __fmul_rn((float)(int8_t)__ldg(b + 2 + (i & 31)), d);
    } else if constexpr (TYPE == T_Q4_K || TYPE == T_Q5_K) {
        constexpr bool Q5 = TYPE == T_Q5_K;
        const uint8_t* b = row + (size_t)(i >> 8) * (Q5 ? 176 : 144);
        const uint32_t r = i & 255u, g = r >> 6, hi = (r >> 5) & 1u, l = r & 31u;
        const int is = (int)(2 * g + hi);
        uint32_t s[3];
        ld_words<3>(b + 4, s);
        uint32_t sc, m;
        scale_min_k4(is, s[0], s[1], s[2], sc, m);
        const float d = h2f(ld_u16(b)), dmin = h2f(ld_u16(b + 2));
        const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)m);
        const uint32_t qb = __ldg(b + (Q5 ? 48 : 16) + 32 * g + l);
        uint32_t q = hi ? (qb >> 4) : (qb & 0xFu);
        if (Q5) q |= ((__ldg(b + 16 + l) >> is) & 1u) << 4;
        return __fsub_rn(__fmul_rn(d1, (float)q), m1);
    } else if constexpr (TYPE == T_Q6_K) {
        const uint8_t* b = row + (size_t)(i >> 8) * 210;
        const uint32_t r = i & 255u, half = r >> 7, quarter = (r >> 5) & 3u, l = r & 31u, is = l >> 4;
        const uint8_t* ql = b + 64 * half;
        const uint32_t qh = __ldg(b + 128 + 32 * half + l);
        const uint32_t qlb = __ldg(ql + l + ((quarter & 1u) ? 32 : 0));
        const uint32_t nib = (quarter & 2u) ? (qlb >> 4) : (qlb & 0xFu);
        const int q = (int)(nib | (((qh >> (2 * quarter)) & 3u) << 4)) - 32;
        const float sc = (float)(int8_t)__ldg(b + 192 + 8 * half + is + 2 * quarter);
        const float d = h2f(ld_u16(b + 208));
        return __fmul_rn(__fmul_rn(d, sc), (float)q);
    } else if constexpr (TYPE == T_Q5_0 || TYPE == T_Q5_1) {
        constexpr bool Q51 = TYPE == T_Q5_1;
        const uint8_t* b = row + (size_t)(i >> 5) * (Q51 ? 24 : 22);
        const uint32_t r = i & 31u, j = r & 15u, hi = r >> 4;
        uint32_t qh[1];
        ld_words<1>(b + (Q51 ? 4 : 2), qh);
        const uint32_t qb = __ldg(b + (Q51 ? 8 : 6) + j);
        const uint32_t q = (hi ? (qb >> 4) : (qb & 0xFu)) | (((qh[0] >> (j + 16 * hi)) & 1u) << 4);
        const float d = h2f(ld_u16(b));
        if (Q51) return __fadd_rn(__fmul_rn(d, (float)q), h2f(ld_u16(b + 2)));
        return __fmul_rn(d, __fsub_rn((float)q, 16.0f));
    } else {  // T_MXFP4
        const uint8_t* b = row + (size_t)(i >> 5) * 17;
        const uint32_t r = i & 31u, j = r & 15u, hi = r >> 4;
        const uint32_t qb = __ldg(b + 1 + j);
        return __fmul_rn(e8m0_to_f32(__ldg(b)), e2m1_to_f32(hi ? (qb >> 4) : (qb & 0xFu)));
    }
}

}  // namespace zc
