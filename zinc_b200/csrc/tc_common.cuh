// Shared pieces of the tcgen05 dequant-GEMM kernels: tile constants, the mbarrier block, TMA / tcgen05
// wrappers, shared-memory and instruction descriptors, the bounded wait, and the Q4_K / Q6_K producers
// that write dequantised bf16 weights in the K-major 128-byte-swizzled layout tcgen05.mma consumes.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "stream_common.cuh"

namespace zc {
namespace {

constexpr int kBM = 128;      // weight rows per tile (= TMEM lanes)
constexpr int kBK = 64;       // columns per stage: 128 bytes of bf16, one swizzle row
constexpr int kAStages = 4;   // one per 64-column group of a 256-column block
// control warps ahead of the 16 dequant warps. One accumulator: MMA issuer, activation loader, raw-weight loader.
// Two: the first accumulator's issuer, one loader for both rings, the second accumulator's issuer.
constexpr int kCtlWarps = 3;
constexpr int kThreads = kCtlWarps * 32 + 4 * 128;
constexpr uint32_t kABytes = kBM * kBK * 2;   // 16 KB

// Raw-block staging per weight type. A box is one 256-column block of 128 rows; Q6_K blocks are 210
// bytes and only 2-byte aligned, so their box is the 240-byte aligned superset that contains them.
template <int TYPE>
struct Raw;
template <>
struct Raw<T_Q4_K> {
    static constexpr uint32_t kBlock = 144, kBox = 144, kSlots = 3;
};
template <>
struct Raw<T_Q6_K> {
    static constexpr uint32_t kBlock = 210, kBox = 240, kSlots = 2;
};

// MXFP4: a "block" here is 8 GGUF blocks of 17 bytes (256 columns, 136 bytes, no alignment at all); the box
// is the 16-byte aligned superset (at most 160 bytes) in a 176-byte slot row.
template <>
struct Raw<T_MXFP4> {
    static constexpr uint32_t kBlock = 136, kBox = 176, kSlots = 2;
};

template <int TYPE, int BN>
struct Tile {
    static constexpr int kBSlots = BN == 256 ? 3 : 6;
    static constexpr int kWSlots = Raw<TYPE>::kSlots;
    static constexpr uint32_t kWBytes = kBM * Raw<TYPE>::kBox;
    static constexpr uint32_t kBBytes = BN * kBK * 2;
    static constexpr uint32_t kWOffset = kAStages * kABytes;
    static constexpr uint32_t kBOffset = kWOffset + kWSlots * kWBytes;
    static constexpr uint32_t kBarOffset = kBOffset + kBSlots * kBBytes;
    static constexpr uint32_t kSmemBytes = kBarOffset + 256 + 1024;  // barriers + alignment slack
};

// Barrier block that follows the rings.
struct Bars {
    uint64_t full_a[kAStages];
    uint64_t empty_a[kAStages];
    uint64_t full_w[3];
    uint64_t empty_w[3];
    uint64_t full_b[6];
    uint64_t empty_b[6];
    uint64_t accum;
    uint32_t tmem_base;
    volatile uint32_t failed;
    uint64_t tmem_free;  // persistent kernel: the epilogue has emptied the accumulators
};
static_assert(sizeof(Bars) <= 256, "the tiles reserve 256 bytes for the barrier block");

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]^T, bf16 x bf16 -> f32, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster share one MMA of M = 256 --------------------------------
// Each CTA holds its own 128 weight rows (A) and half of the activation tile's tokens (B); the even CTA of the
// pair issues the MMAs and owns the "full" barriers, on which the odd CTA's producers and copies arrive through
// the cluster's shared window; a commit arrives on the barrier at the same offset in both CTAs. No copy is
// multicast: every CTA fetches what it holds itself.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address of `p` in the pair's even CTA, in the cluster's shared window
__device__ __forceinline__ uint32_t leader_addr(const void* p) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(r) : "r"(smem_u32(p)));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar), "r"(bytes)
                 : "memory");
}
// TMA tile into this CTA's shared memory, completion counted on a barrier of the pair's even CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(cluster_bar)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "h"((uint16_t)3)
                 : "memory");
}
// Instruction descriptor of the pair's MMA: as instr_desc, M = 256.
template <int BN>
__host__ __device__ constexpr uint32_t instr_desc_pair() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

// 16 bytes global -> shared; bytes past `n` (0..16) are written as zeros and not read.
__device__ __forceinline__ void cp_async16_zfill(void* smem_dst, const void* gmem_src, uint32_t n) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(n)
                 : "memory");
}

// 32 consecutive columns of this thread's tensor-memory lane (issued, not waited for)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    const uint32_t lo = ((saddr >> 4) & 0x3FFFu) | (1u << 16);         // start address, leading offset (unused) = 1
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);         // stride offset, version 1, SWIZZLE_128B
    return ((uint64_t)hi << 32) | lo;
}

// Instruction descriptor: f32 accumulator, bf16 A and B, both K-major, M = 128, N = BN.
template <int BN>
__host__ __device__ constexpr uint32_t instr_desc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

// Bounded wait. kSleep: back off between polls (every role but the tensor-core issuer has slack).
template <bool kSleep = true>
__device__ __forceinline__ bool wait_or_fail(uint64_t* bar, uint32_t parity, Bars* bars, uint32_t* status,
                                             uint32_t site) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (kSleep) __nanosleep(64);
        if ((i & 63u) == 63u && bars->failed) return false;
    }
    bars->failed = 1;
    if (status) {
        status[0] = 1;
        status[1] = site;
    }
    return false;
}

__device__ __forceinline__ uint32_t bf2_bits(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __nv_bfloat162 bits_bf2(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }

// Four weights (the low nibbles of bytes 0..3 of `nib`, already masked to 0x0F0F0F0F) -> two bf16x2
// words. (128 + q) is built by byte permutation (exact in bf16) and 136 subtracted, which leaves
// q - 8 exactly; the weight d*sc*q - dmin*m is then formed as (q - 8) * dsc + c with
// c = 8*d*sc - dmin*m, so that the bf16 rounding of dsc acts on a term of at most 8*dsc.
__device__ __forceinline__ void deq4(uint32_t nib, __nv_bfloat162 dsc, __nv_bfloat162 c, uint32_t& o0,
                                     uint32_t& o1) {
    const __nv_bfloat162 k136 = bits_bf2(0x43084308u);
    const uint32_t p0 = __byte_perm(nib, 0x43434343u, 0x4140);
    const uint32_t p1 = __byte_perm(nib, 0x43434343u, 0x4342);
    o0 = bf2_bits(__hfma2(__hsub2(bits_bf2(p0), k136), dsc, c));
    o1 = bf2_bits(__hfma2(__hsub2(bits_bf2(p1), k136), dsc, c));
}

// One 64-column group of a Q4_K row: 32 bytes of nibbles -> 8 chunks of 8 bf16 written to the
// swizzled row `row` of the stage at `a_stage`.
__device__ __forceinline__ void dequant_group_q4k(const uint4& q0, const uint4& q1, float d_sc_lo, float dm_lo,
                                                  float d_sc_hi, float dm_hi, uint8_t* a_stage, int row) {
    const __nv_bfloat162 s_lo = __float2bfloat162_rn(d_sc_lo), m_lo = __float2bfloat162_rn(8.f * d_sc_lo - dm_lo);
    const __nv_bfloat162 s_hi = __float2bfloat162_rn(d_sc_hi), m_hi = __float2bfloat162_rn(8.f * d_sc_hi - dm_hi);
    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    uint8_t* rowp = a_stage + row * 128;
    const int sw = row & 7;
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // chunk c: bytes 8c..8c+7 -> low nibbles = columns 8c.., high = 32+8c..
        uint4 lo, hi;
        deq4(w[2 * c] & 0x0F0F0F0Fu, s_lo, m_lo, lo.x, lo.y);
        deq4(w[2 * c + 1] & 0x0F0F0F0Fu, s_lo, m_lo, lo.z, lo.w);
        deq4((w[2 * c] >> 4) & 0x0F0F0F0Fu, s_hi, m_hi, hi.x, hi.y);
        deq4((w[2 * c + 1] >> 4) & 0x0F0F0F0Fu, s_hi, m_hi, hi.z, hi.w);
        *reinterpret_cast<uint4*>(rowp + ((c ^ sw) << 4)) = lo;
        *reinterpret_cast<uint4*>(rowp + (((c + 4) ^ sw) << 4)) = hi;
    }
}

// N consecutive 32-bit words starting `sh` bits (0 or 16) into the aligned word at p.
template <int N>
__device__ __forceinline__ void lds_shifted(const uint32_t* p, uint32_t sh, uint32_t (&w)[N]) {
    uint32_t prev = p[0];
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const uint32_t next = p[i + 1];
        w[i] = __funnelshift_r(prev, next, sh);
        prev = next;
    }
}

// Four 6-bit weights (one per byte of q4, values 0..63) -> two bf16x2 words: (128 + q) - 160 = q - 32
// exactly, times d*scale.
__device__ __forceinline__ void deq4_q6(uint32_t q4, __nv_bfloat162 dsc, uint32_t& o0, uint32_t& o1) {
    const __nv_bfloat162 k160 = bits_bf2(0x43204320u);
    const uint32_t p0 = __byte_perm(q4, 0x43434343u, 0x4140);
    const uint32_t p1 = __byte_perm(q4, 0x43434343u, 0x4342);
    o0 = bf2_bits(__hmul2(__hsub2(bits_bf2(p0), k160), dsc));
    o1 = bf2_bits(__hmul2(__hsub2(bits_bf2(p1), k160), dsc));
}

// One 64-column group g of a Q6_K block (layout: ql[128] qh[64] scales[16] d, src/model/gguf.zig:38-123;
// element order as dequantRow, src/compute/forward.zig:335-383): half n = g / 2 of the block, low
// (g even) or high (g odd) nibbles of ql[64n .. 64n+64), bit pairs 4*(g&1) and 4*(g&1)+2 of
// qh[32n .. 32n+32), scales[8n + 4*(g&1) .. +4) each covering 16 columns. `blk` points at the aligned
// word that contains the block's first byte, `sh` = 0 or 16.
__device__ __forceinline__ void dequant_group_q6k(const uint32_t* blk, uint32_t sh, int g, uint8_t* a_stage,
                                                  int row) {
    const int n = g >> 1, hi = g & 1;
    uint32_t ql[16], qh[8], scw[1], dw[1];
    lds_shifted<16>(blk + 16 * n, sh, ql);
    lds_shifted<8>(blk + 32 + 8 * n, sh, qh);
    lds_shifted<1>(blk + 48 + 2 * n + hi, sh, scw);
    lds_shifted<1>(blk + 52, sh, dw);
    const float d = __half2float(__ushort_as_half((unsigned short)(dw[0] & 0xFFFFu)));
    uint8_t* rowp = a_stage + row * 128;
    const int sw = row & 7;
#pragma unroll
    for (int c = 0; c < 8; ++c) {  // chunk c = columns 8c .. 8c+7 of the group; scale index c / 2
        const float sc = (float)(int)(int8_t)((scw[0] >> (8 * (c >> 1))) & 0xFFu);
        const __nv_bfloat162 dsc = __float2bfloat162_rn(d * sc);
        uint4 o;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            // columns 8c+4e .. +3: ql byte index (c < 4 ? 0 : 32) + 8*(c&3) + 4e, qh byte index 8*(c&3) + 4e
            const uint32_t lw = ql[(c >> 2) * 8 + (c & 3) * 2 + e];
            const uint32_t hw = qh[(c & 3) * 2 + e];
            const uint32_t nib = (lw >> (4 * hi)) & 0x0F0F0F0Fu;
            const uint32_t top = ((hw >> (4 * hi + 2 * (c >> 2))) & 0x03030303u) << 4;
            uint32_t a, b;
            deq4_q6(nib | top, dsc, a, b);
            if (e == 0) {
                o.x = a;
                o.y = b;
            } else {
                o.z = a;
                o.w = b;
            }
        }
        *reinterpret_cast<uint4*>(rowp + ((c ^ sw) << 4)) = o;
    }
}

// Byte permute with the full selector semantics (bit 3 of a selector nibble replicates the sign bit of
// the selected byte); the __byte_perm intrinsic masks that bit off.
__device__ __forceinline__ uint32_t prmt_full(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Four E2M1 weights in 16 bits (two bytes of a block: nibbles lo0, hi0, lo1, hi1 = columns j, j+16, j+1,
// j+17) -> bf16x2 words for columns (j, j+1) and (j+16, j+17), times the block scale. The magnitudes
// {0, .5, 1, 1.5, 2, 3, 4, 6} are the bf16 patterns 0x0000 3F00 3F80 3FC0 4000 4040 4080 40C0: two byte
// tables looked up with one permute each; the sign bits come from a sign-replicating permute. The
// product with the power-of-two scale is exact (src/compute/forward.zig:441-459).
__device__ __forceinline__ void deq_mx16(uint32_t x16, __nv_bfloat162 scale, uint32_t& lo_pair, uint32_t& hi_pair) {
    const uint32_t sel = x16 & 0x7777u;
    const uint32_t hi4 = __byte_perm(0x3F3F3F00u, 0x40404040u, sel);
    const uint32_t lo4 = __byte_perm(0xC0800000u, 0xC0804000u, sel);
    const uint32_t a = __byte_perm(lo4, hi4, 0x6240) | (prmt_full(x16 << 4, 0u, 0x9988u) & 0x80008000u);
    const uint32_t b = __byte_perm(lo4, hi4, 0x7351) | (prmt_full(x16, 0u, 0x9988u) & 0x80008000u);
    lo_pair = bf2_bits(__hmul2(bits_bf2(a), scale));
    hi_pair = bf2_bits(__hmul2(bits_bf2(b), scale));
}

// One 64-column group (two 17-byte blocks, 34 bytes) of an MXFP4 row -> the swizzled row `row` of the
// stage at `a_stage`. `p` points at the aligned word that holds the group's first byte, `sh` = 8 * (its
// byte position in that word).
__device__ __forceinline__ void dequant_group_mxfp4(const uint32_t* p, uint32_t sh, uint8_t* a_stage, int row) {
    uint32_t w[9];
    lds_shifted<9>(p, sh, w);  // bytes 0..35 of the group: e0, 16 nibble bytes, e1, 16 nibble bytes
    uint8_t* rowp = a_stage + row * 128;
    const int sw = row & 7;
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
        const uint32_t e = blk == 0 ? (w[0] & 0xFFu) : ((w[4] >> 8) & 0xFFu);
        const uint32_t sb = e ? (e << 7) : 0x40u;  // 2^(e-127) as bf16; e = 0 -> 2^-127 as in the reference
        const __nv_bfloat162 scale = bits_bf2(sb | (sb << 16));
        uint32_t q[4];  // the 16 nibble bytes
#pragma unroll
        for (int i = 0; i < 4; ++i)
            q[i] = blk == 0 ? __funnelshift_r(w[i], w[i + 1], 8) : __funnelshift_r(w[4 + i], w[5 + i], 16);
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // bytes 8h .. 8h+7: low nibbles = columns 8h.., high = 16 + 8h..
            uint4 lo, hi;
            deq_mx16(q[2 * h] & 0xFFFFu, scale, lo.x, hi.x);
            deq_mx16(q[2 * h] >> 16, scale, lo.y, hi.y);
            deq_mx16(q[2 * h + 1] & 0xFFFFu, scale, lo.z, hi.z);
            deq_mx16(q[2 * h + 1] >> 16, scale, lo.w, hi.w);
            *reinterpret_cast<uint4*>(rowp + (((4 * blk + h) ^ sw) << 4)) = lo;
            *reinterpret_cast<uint4*>(rowp + (((4 * blk + 2 + h) ^ sw) << 4)) = hi;
        }
    }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

}  // namespace
}  // namespace zc
