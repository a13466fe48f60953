// Per-lane partial dot products of quantized weight rows against an f32 vector.
//
// rowdot<TYPE, NR>(rows, x, K, lane, acc) adds, for each of NR weight rows, this
// lane's share of sum_k W[row][k] * x[k] to acc[r]; a warp_sum over the 32
// lanes completes it. The NR rows share every load of x. Quants are unpacked
// in registers and accumulated in f32; the block scale is applied once per
// sub-block (d*sc*sum(q*x) - dmin*m*sum(x) for the K-quants with a min).
//
// Block layouts and dequant rules follow dequantRow of the reference
// (src/compute/forward.zig:242-465; Q5_1: src/compute/forward_metal.zig:6704-6729).
#pragma once

#include "common.cuh"

namespace zc {

__device__ __forceinline__ void ld_x4(const float* p, float (&v)[4]) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}

// ---- Q4_K (144 B) and Q5_K (176 B): lane = (block, 16-byte chunk of qs) --------
// A warp covers 4 consecutive super-blocks per step (576 / 704 contiguous bytes).
// Chunk c holds qs[16c..16c+16): low nibbles are elements 64j+16h+i of sub-block
// 2j, high nibbles elements 64j+32+16h+i of sub-block 2j+1 (j = c/2, h = c%2).
template <int NR, bool Q5, bool ALIGNED>
__device__ __forceinline__ void rowdot_q45k(const uint8_t* const (&rows)[NR], const float* __restrict__ x,
                                            uint32_t K, int lane, float (&acc)[NR]) {
    constexpr uint32_t BPB = Q5 ? 176u : 144u;
    constexpr uint32_t QS_OFF = Q5 ? 48u : 16u;
    const uint32_t bpr = K >> 8;
    const int c = lane & 7, j = c >> 1, h = c & 1;
    for (uint32_t blk = lane >> 3; blk < bpr; blk += 4) {
        const float* xp = x + (size_t)blk * 256 + 64 * j + 16 * h;
        float xl[16], xh[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(xp) + i);
            const float4 b = __ldg(reinterpret_cast<const float4*>(xp + 32) + i);
            xl[4 * i] = a.x; xl[4 * i + 1] = a.y; xl[4 * i + 2] = a.z; xl[4 * i + 3] = a.w;
            xh[4 * i] = b.x; xh[4 * i + 1] = b.y; xh[4 * i + 2] = b.z; xh[4 * i + 3] = b.w;
        }
        float sxl = 0.f, sxh = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) { sxl += xl[i]; sxh += xh[i]; }
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint8_t* b = rows[r] + (size_t)blk * BPB;
            uint32_t hd[4], q[4], qh[4] = {0, 0, 0, 0};
            if (ALIGNED) {
                const uint4 t = ldg_u128(b);
                hd[0] = t.x; hd[1] = t.y; hd[2] = t.z; hd[3] = t.w;
                const uint4 u = ldg_u128(b + QS_OFF + 16 * c);
                q[0] = u.x; q[1] = u.y; q[2] = u.z; q[3] = u.w;
                if (Q5) {
                    const uint4 v = ldg_u128(b + 16 + 16 * h);
                    qh[0] = v.x; qh[1] = v.y; qh[2] = v.z; qh[3] = v.w;
                }
            } else {
                ld_words<4>(b, hd);
                ld_words<4>(b + QS_OFF + 16 * c, q);
                if (Q5) ld_words<4>(b + 16 + 16 * h, qh);
            }
            const float d = h2f(hd[0]), dmin = h2f(hd[0] >> 16);
            uint32_t sc0, m0, sc1, m1;
            scale_min_k4(2 * j, hd[1], hd[2], hd[3], sc0, m0);
            scale_min_k4(2 * j + 1, hd[1], hd[2], hd[3], sc1, m1);
            float sl = 0.f, sh = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
#pragma unroll
                for (int bb = 0; bb < 4; ++bb) {
                    uint32_t lo = (q[w] >> (8 * bb)) & 0xFu;
                    uint32_t hi = (q[w] >> (8 * bb + 4)) & 0xFu;
                    if (Q5) {
                        const uint32_t hb = (qh[w] >> (8 * bb)) & 0xFFu;
                        lo |= ((hb >> (2 * j)) & 1u) << 4;
                        hi |= ((hb >> (2 * j + 1)) & 1u) << 4;
                    }
                    sl = fmaf((float)lo, xl[4 * w + bb], sl);
                    sh = fmaf((float)hi, xh[4 * w + bb], sh);
                }
            }
            acc[r] += d * (float)sc0 * sl - dmin * (float)m0 * sxl + d * (float)sc1 * sh - dmin * (float)m1 * sxh;
        }
    }
}

// ---- Q6_K (210 B, 2-byte aligned): 16 lanes per super-block, 2 blocks per step ----
// Lane (half, e0) handles l = e0..e0+3 of one 128-element half: 16 weights from
// ql[l], ql[l+32], qh[l] with the four int8 scales is, is+2, is+4, is+6.
template <int NR>
__device__ __forceinline__ void rowdot_q6k(const uint8_t* const (&rows)[NR], const float* __restrict__ x,
                                           uint32_t K, int lane, float (&acc)[NR]) {
    const uint32_t bpr = K >> 8;
    const int l16 = lane & 15, half = l16 >> 3, e0 = (l16 & 7) * 4, is = e0 >> 4;
    for (uint32_t blk = lane >> 4; blk < bpr; blk += 2) {
        const float* xp = x + (size_t)blk * 256 + 128 * half + e0;
        float x0[4], x1[4], x2[4], x3[4];
        ld_x4(xp, x0); ld_x4(xp + 32, x1); ld_x4(xp + 64, x2); ld_x4(xp + 96, x3);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint8_t* b = rows[r] + (size_t)blk * 210;
            uint32_t ql_lo[1], ql_hi[1], qh[1], sc[2];
            ld_words<1>(b + 64 * half + e0, ql_lo);
            ld_words<1>(b + 64 * half + e0 + 32, ql_hi);
            ld_words<1>(b + 128 + 32 * half + e0, qh);
            ld_words<2>(b + 192 + 8 * half, sc);
            const float d = h2f(ld_u16(b + 208));
            float s1 = 0.f, s2 = 0.f, s3 = 0.f, s4 = 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t lo = ql_lo[0] >> (8 * e), hi = ql_hi[0] >> (8 * e), hh = qh[0] >> (8 * e);
                const int q1 = (int)((lo & 0xFu) | ((hh & 3u) << 4)) - 32;
                const int q2 = (int)((hi & 0xFu) | (((hh >> 2) & 3u) << 4)) - 32;
                const int q3 = (int)(((lo >> 4) & 0xFu) | (((hh >> 4) & 3u) << 4)) - 32;
                const int q4 = (int)(((hi >> 4) & 0xFu) | (((hh >> 6) & 3u) << 4)) - 32;
                s1 = fmaf((float)q1, x0[e], s1);
                s2 = fmaf((float)q2, x1[e], s2);
                s3 = fmaf((float)q3, x2[e], s3);
                s4 = fmaf((float)q4, x3[e], s4);
            }
            // scale bytes is, is+2, is+4, is+6 of the 8 scales of this half
            const float c0 = (float)(int8_t)((is ? sc[0] >> 8 : sc[0]) & 0xFFu);
            const float c2 = (float)(int8_t)((is ? sc[0] >> 24 : sc[0] >> 16) & 0xFFu);
            const float c4 = (float)(int8_t)((is ? sc[1] >> 8 : sc[1]) & 0xFFu);
            const float c6 = (float)(int8_t)((is ? sc[1] >> 24 : sc[1] >> 16) & 0xFFu);
            acc[r] += d * (c0 * s1 + c2 * s2 + c4 * s3 + c6 * s4);
        }
    }
}

// ---- 32-element block types: one lane per block --------------------------------
// Q8_0 (34 B): d f16, 32 int8.
template <int NR>
__device__ __forceinline__ void rowdot_q8_0(const uint8_t* const (&rows)[NR], const float* __restrict__ x,
                                            uint32_t K, int lane, float (&acc)[NR]) {
    const uint32_t bpr = K >> 5;
    for (uint32_t blk = lane; blk < bpr; blk += 32) {
        const float* xp = x + (size_t)blk * 32;
        float xv[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(xp) + i);
            xv[4 * i] = a.x; xv[4 * i + 1] = a.y; xv[4 * i + 2] = a.z; xv[4 * i + 3] = a.w;
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint8_t* b = rows[r] + (size_t)blk * 34;
            uint32_t q[8];
            ld_words<8>(b + 2, q);
            const float d = h2f(ld_u16(b));
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) {
#pragma unroll
                for (int bb = 0; bb < 4; ++bb)
                    s = fmaf((float)(int8_t)((q[w] >> (8 * bb)) & 0xFFu), xv[4 * w + bb], s);
            }
            acc[r] = fmaf(d, s, acc[r]);
        }
    }
}

// MXFP4 (17 B): E8M0 scale byte, 16 bytes of E2M1 nibbles; low nibble j -> element j,
// high nibble -> element j+16.
// The eight E2M1 magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6} as f32 have bit patterns 0x0000, 0x3F00, 0x3F80,
// 0x3FC0, 0x4000, 0x4040, 0x4080, 0x40C0 in their upper halves: two byte tables, looked up four
// nibbles at a time with one byte permute each, then one permute per element assembles the float and
// the nibble's bit 3 is moved to the sign bit. Values are exactly those of the table in
// src/compute/forward.zig:445.
__device__ __forceinline__ void e2m1x4_to_f32(uint32_t nib16, float (&out)[4]) {
    // nib16: four nibbles in bits 0..15; out[i] = value of nibble i
    const uint32_t sel = nib16 & 0x7777u;
    const uint32_t hi = __byte_perm(0x3F3F3F00u, 0x40404040u, sel);  // top bytes
    const uint32_t lo = __byte_perm(0xC0800000u, 0xC0804000u, sel);  // second bytes
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // bytes (LSB first): 0, 0, lo[i], hi[i]; 'lo' is operand a (bytes 0..3), 'hi' operand b (bytes 4..7)
        const uint32_t mag = __byte_perm(lo, hi, 0x0000u | ((4u + i) << 12) | ((uint32_t)i << 8)) & 0xFFFF0000u;
        const uint32_t sign = (nib16 << (28 - 4 * i)) & 0x80000000u;
        out[i] = __uint_as_float(mag | sign);
    }
}

template <int NR>
__device__ __forceinline__ void rowdot_mxfp4(const uint8_t* const (&rows)[NR], const float* __restrict__ x,
                                             uint32_t K, int lane, float (&acc)[NR]) {
    const uint32_t bpr = K >> 5;
    for (uint32_t blk = lane; blk < bpr; blk += 32) {
        const float* xp = x + (size_t)blk * 32;
        float xv[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(xp) + i);
            xv[4 * i] = a.x; xv[4 * i + 1] = a.y; xv[4 * i + 2] = a.z; xv[4 * i + 3] = a.w;
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint8_t* b = rows[r] + (size_t)blk * 17;
            uint32_t q[4];
            ld_words<4>(b + 1, q);
            const float d = e8m0_to_f32(__ldg(b));
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    // 16 bits = bytes 4w+2hf, 4w+2hf+1: nibbles (lo0, hi0, lo1, hi1) = elements j, j+16, j+1, j+17
                    float v[4];
                    e2m1x4_to_f32((q[w] >> (16 * hf)) & 0xFFFFu, v);
                    const int j = 4 * w + 2 * hf;
                    s = fmaf(v[0], xv[j], s);
                    s = fmaf(v[1], xv[j + 16], s);
                    s = fmaf(v[2], xv[j + 1], s);
                    s = fmaf(v[3], xv[j + 17], s);
                }
            }
            acc[r] = fmaf(d, s, acc[r]);
        }
    }
}

// Q5_0 (22 B: d, qh u32, 16 qs) and Q5_1 (24 B: d, m, qh u32, 16 qs).
// Factored form d*sum(q*x) (+ m*sum(x)), as src/shaders/dmmv_q5_1.comp:60-95.
template <int NR, bool Q51>
__device__ __forceinline__ void rowdot_q5_01(const uint8_t* const (&rows)[NR], const float* __restrict__ x,
                                             uint32_t K, int lane, float (&acc)[NR]) {
    constexpr uint32_t BPB = Q51 ? 24u : 22u;
    const uint32_t bpr = K >> 5;
    for (uint32_t blk = lane; blk < bpr; blk += 32) {
        const float* xp = x + (size_t)blk * 32;
        float xv[32];
        float sx = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(xp) + i);
            xv[4 * i] = a.x; xv[4 * i + 1] = a.y; xv[4 * i + 2] = a.z; xv[4 * i + 3] = a.w;
            sx += a.x + a.y + a.z + a.w;
        }
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint8_t* b = rows[r] + (size_t)blk * BPB;
            uint32_t w[5];
            ld_words<5>(b + (Q51 ? 4 : 2), w);  // qh, then 16 bytes of qs
            const float d = h2f(ld_u16(b));
            const float mn = Q51 ? h2f(ld_u16(b + 2)) : 0.f;
            const uint32_t qh = w[0];
            float s = 0.f;
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) {
                const uint32_t byte = (w[1 + (jj >> 2)] >> (8 * (jj & 3))) & 0xFFu;
                const uint32_t q0 = (byte & 0xFu) | (((qh >> jj) & 1u) << 4);
                const uint32_t q1 = (byte >> 4) | (((qh >> (jj + 16)) & 1u) << 4);
                s = fmaf((float)q0, xv[jj], s);
                s = fmaf((float)q1, xv[jj + 16], s);
            }
            if (Q51) acc[r] += d * s + mn * sx;
            else acc[r] += d * (s - 16.0f * sx);
        }
    }
}

// F16 and F32 rows: lanes stride over elements.
template <int NR>
__device__ __forceinline__ void rowdot_f16(const uint8_t* const (&rows)[NR], const float* __restrict__ x,
                                           uint32_t K, int lane, float (&acc)[NR]) {
    for (uint32_t i = lane; i < K; i += 32) {
        const float xv = __ldg(x + i);
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] = fmaf(h2f(ld_u16(rows[r] + 2 * (size_t)i)), xv, acc[r]);
    }
}
template <int NR>
__device__ __forceinline__ void rowdot_f32(const uint8_t* const (&rows)[NR], const float* __restrict__ x,
                                           uint32_t K, int lane, float (&acc)[NR]) {
    for (uint32_t i = lane; i < K; i += 32) {
        const float xv = __ldg(x + i);
#pragma unroll
        for (int r = 0; r < NR; ++r)
            acc[r] = fmaf(__ldg(reinterpret_cast<const float*>(rows[r]) + i), xv, acc[r]);
    }
}

template <uint32_t TYPE, int NR, bool ALIGNED>
__device__ __forceinline__ void rowdot(const uint8_t* const (&rows)[NR], const float* __restrict__ x,
                                       uint32_t K, int lane, float (&acc)[NR]) {
    if constexpr (TYPE == T_Q4_K) rowdot_q45k<NR, false, ALIGNED>(rows, x, K, lane, acc);
    else if constexpr (TYPE == T_Q5_K) rowdot_q45k<NR, true, ALIGNED>(rows, x, K, lane, acc);
    else if constexpr (TYPE == T_Q6_K) rowdot_q6k<NR>(rows, x, K, lane, acc);
    else if constexpr (TYPE == T_Q8_0) rowdot_q8_0<NR>(rows, x, K, lane, acc);
    else if constexpr (TYPE == T_MXFP4) rowdot_mxfp4<NR>(rows, x, K, lane, acc);
    else if constexpr (TYPE == T_Q5_0) rowdot_q5_01<NR, false>(rows, x, K, lane, acc);
    else if constexpr (TYPE == T_Q5_1) rowdot_q5_01<NR, true>(rows, x, K, lane, acc);
    else if constexpr (TYPE == T_F16) rowdot_f16<NR>(rows, x, K, lane, acc);
    else rowdot_f32<NR>(rows, x, K, lane, acc);
}

}  // namespace zc
