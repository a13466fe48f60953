// Warp-autonomous streaming decode matvec for B200 (Q4_K), integer tensor-core dot engine.
//
// Every warp is an independent worker: it owns a contiguous range of work units (16 rows x
// kCB 256-weight super-blocks), prefetches them with coalesced 16-byte asynchronous copies
// (cp.async into the warp's own ring of padded row segments, depth kDepth; bulk TMA copies were
// measured at ~14 cycles of issue each per SM, too slow for 288-byte row segments), masks the 4-bit
// quants into int8 lanes (one logic op per four weights) and feeds them to the int8 tensor cores as a
// 16-row dot-product engine with exact s32 accumulation. There is no block-wide synchronisation after
// the activation vector has been converted. K is split across workers so that all SMs stream the same
// number of bytes; a tile that spans several workers is finished by the worker that owns its first
// unit, which adds the partial sums the later workers have published (shared memory inside a CTA,
// global memory across CTAs) in worker order, so results do not depend on timing.
//
// Stands in for the reference's K-parallel decode shaders and their fused epilogues
// (src/shaders/dmmv_q4k.comp:59-240, dmmv_q4k_wide.comp, dmmv_q4k_fused_gate_up_swiglu.comp:195-218,
// dmmv_q8_0_sigmoid_acc.comp:95-132) for the Q4_K layout of src/compute/forward.zig:370-409.
//
// Arithmetic per super-block of a row, sub-blocks s = 0..7 of 32 weights:
//   y += 2^-f * ( d * sum_s sc_s * P_s  -  dmin * sum_s m_s * SX_s ),   P_s = sum_i q_i * X_i
// X_i = round(x_i * 2^f) is the block of x in 21-bit fixed point (f chosen per 256-element block
// from its largest magnitude), split into three digits X = b0*2^14 + b1*2^7 + b2 that fit int8
// (b0 signed, b1 and b2 in 0..127). The tensor core computes D_j,s = sum_i q_i * b_j,i exactly in s32
// for each digit j; the 6-bit scales are applied in integer arithmetic too (sum_s sc_s * D_j,s < 2^31),
// so one conversion and one f32 multiply-add per row, digit and super-block remain. SX_s = sum_i X_i
// is exact. Weights are never rounded; the only rounding before the f32 scaling is that of x to 21 bits.
//
// Tensor-core mapping (mma.sync m16n8k32, u8 x s8 -> s32): the 16 A rows are 16 weight rows. One 128-bit
// shared-memory read gives lane (g = lane/4, t = lane%4) bytes 16(t%2) .. +15 of the 32-byte qs group
// 2p + t/2 of row g (p = 0, 1), i.e. sixteen low nibbles (sub-block 4p + 2(t/2)) and sixteen high nibbles
// (sub-block 4p + 2(t/2) + 1; kept in place as 16 q, the factor is folded into the scale). An MMA thus
// carries two sub-blocks, k slots of lanes t < 2 one, of lanes t >= 2 the other; B is block-diagonal
// to match: column 2j + u holds digit j of x for the k slots of sub-block half u and zeros elsewhere, so
// D column 2j + u is digit j's dot product with sub-block u alone. Lane t < 3 therefore ends up with
// digit t of both sub-blocks for rows g and g+8 and applies their scales; eight MMAs per 16 x 256 tile.
#include "kernels.h"
#include "stream_skel.cuh"

namespace zc {

namespace {

constexpr int kDepth = 2;                  // units in flight per warp
constexpr int kCB = 2;                     // super-blocks per row segment
constexpr int kRowSeg = kCB * 144 + 32;    // 320: rows land 64 B apart mod 128 B -> conflict-free 128-bit reads
constexpr int kSlotBytes = 16 * kRowSeg;
constexpr int kWarpRing = kDepth * kSlotBytes;
constexpr size_t kTwoPerSm = 113 * 1024;   // shared memory per CTA that still lets two CTAs share an SM
constexpr int kZeroBytes = 256;            // zeros: B operand of the lanes whose column is dead for their k slots
constexpr int kFracBits = 20;              // |X| <= 2^20
constexpr int kPiecesPerRow = kCB * 9;     // 16-byte pieces of one row segment
constexpr int kPiecesPerLane = (16 * kPiecesPerRow + 31) / 32;

struct Smem {
    uint8_t* dig;    // three digit planes of K bytes each, elements in natural order
    uint8_t* zeros;  // kZeroBytes of zeros, 128-byte aligned
    float* sx;       // per 32-element sub-block sum of X
    float* xs;       // per super-block 2^-f
    uint8_t* ring;   // [kWarps][kDepth] stages of 16 padded row segments
    float* spartial; // [kWarps][32] partial sums published inside the CTA
    volatile uint32_t* sflags;  // [kWarps]
};

__host__ __device__ inline size_t smem_bytes(uint32_t K, int kWarps) {
    size_t n = (size_t)K * 3 + (size_t)kZeroBytes;
    n += (size_t)(K / 32) * 4 + (size_t)(K / 256) * 4;
    n = (n + 127) & ~size_t(127);
    n += (size_t)kWarps * kWarpRing;
    n += (size_t)kWarps * 32 * 4 + (size_t)kWarps * 4 + 16;
    return n + 128;
}

__device__ inline Smem carve(uint8_t* base, uint32_t K, int kWarps) {
    Smem s;
    uintptr_t p = (reinterpret_cast<uintptr_t>(base) + 127) & ~uintptr_t(127);
    s.zeros = reinterpret_cast<uint8_t*>(p);
    p += (size_t)kZeroBytes;
    s.dig = reinterpret_cast<uint8_t*>(p);   // K is a multiple of 256: every plane starts 128-byte aligned
    p += (size_t)K * 3;
    s.sx = reinterpret_cast<float*>(p);
    p += (size_t)(K / 32) * 4;
    s.xs = reinterpret_cast<float*>(p);
    p += (size_t)(K / 256) * 4;
    p = (p + 127) & ~uintptr_t(127);
    s.ring = reinterpret_cast<uint8_t*>(p);
    p += (size_t)kWarps * kWarpRing;
    s.spartial = reinterpret_cast<float*>(p);
    p += (size_t)kWarps * 32 * 4;
    s.sflags = reinterpret_cast<volatile uint32_t*>(p);
    return s;
}


// Convert x into int8 digit planes. One warp per super-block; lane l handles the 8 consecutive elements
// 8l .. 8l+7 (a 32-byte coalesced read), so sub-block s is lanes 4s .. 4s+3.
//
// The loads are issued before the weight prefetch (so they are not queued behind it) and
// converted afterwards: kPrepBlocks super-blocks per warp cover K <= kPrepBlocks * kWarps * 256.
constexpr int kPrepBlocks = 6;  // x super-blocks per warp: K <= kPrepBlocks * kWarps * 256
struct XRegs {
    float4 lo[kPrepBlocks], hi[kPrepBlocks];
};
template <int kWarps>
__device__ __forceinline__ void load_x(XRegs& r, const float* __restrict__ x, uint32_t K, int warp, int lane) {
#pragma unroll
    for (int i = 0; i < kPrepBlocks; ++i) {
        const uint32_t blk = warp + i * kWarps;
        if (blk < (K >> 8)) {
            const float* xp = x + (size_t)blk * 256 + 8 * lane;
            r.lo[i] = __ldg(reinterpret_cast<const float4*>(xp));
            r.hi[i] = __ldg(reinterpret_cast<const float4*>(xp) + 1);
        }
    }
}

// The same eight elements per lane, merged from split-K attention partials (up to four chunks; head_dim a
// multiple of 8, so a lane's elements share a head).
constexpr int kMergeChunks = 4;
template <int kWarps>
__device__ __forceinline__ void load_x_merge(XRegs& r, const MergeArgs& m, uint32_t K, int warp, int lane) {
#pragma unroll
    for (int i = 0; i < kPrepBlocks; ++i) {
        const uint32_t blk = warp + i * kWarps;
        if (blk < (K >> 8)) {
            const uint32_t k0 = blk * 256 + 8 * lane, head = k0 / m.head_dim, d = k0 - head * m.head_dim;
            float4 pl[kMergeChunks], ph[kMergeChunks];
#pragma unroll
            for (int c = 0; c < kMergeChunks; ++c) {
                if ((uint32_t)c < m.n_chunks) {
                    const float4* p = reinterpret_cast<const float4*>(
                        m.partial + ((size_t)head * m.n_chunks + c) * m.head_dim + d);
                    pl[c] = __ldg(p);
                    ph[c] = __ldg(p + 1);
                } else {
                    pl[c] = ph[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            float w[kMergeChunks];
            const float inv = attn_merge_weights<kMergeChunks>(
                m.partial + (size_t)m.n_heads * m.n_chunks * m.head_dim + (size_t)head * m.n_chunks * 2, m.sinks,
                m.sink_offset + head, m.n_chunks, w);
            float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
#pragma unroll
            for (int c = 0; c < kMergeChunks; ++c) {
                lo = make_float4(fmaf(w[c], pl[c].x, lo.x), fmaf(w[c], pl[c].y, lo.y), fmaf(w[c], pl[c].z, lo.z),
                                 fmaf(w[c], pl[c].w, lo.w));
                hi = make_float4(fmaf(w[c], ph[c].x, hi.x), fmaf(w[c], ph[c].y, hi.y), fmaf(w[c], ph[c].z, hi.z),
                                 fmaf(w[c], ph[c].w, hi.w));
            }
            r.lo[i] = make_float4(lo.x * inv, lo.y * inv, lo.z * inv, lo.w * inv);
            r.hi[i] = make_float4(hi.x * inv, hi.y * inv, hi.z * inv, hi.w * inv);
        }
    }
}

// Four values' low bytes as one word.
__device__ __forceinline__ uint32_t pack4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

template <int kWarps>
__device__ __forceinline__ void prep_x(const Smem& s, const XRegs& r, uint32_t K, int warp, int lane) {
#pragma unroll
    for (int bi = 0; bi < kPrepBlocks; ++bi) {
        const uint32_t blk = warp + bi * kWarps;
        if (blk >= (K >> 8)) break;
        const float4 lo = r.lo[bi], hi = r.hi[bi];
        const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float mx = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(v[i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        // |x| < 2^(E-126)  ->  |x * 2^f| < 2^20 with f = 146 - E (E = biased exponent of the block maximum)
        uint32_t E = (__float_as_uint(mx) >> 23) & 0xFFu;
        E = E < 32u ? 32u : E;
        const float scale = __uint_as_float((127u + 126u + kFracBits - E) << 23);
        int X[8];
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            X[i] = __float2int_rn(v[i] * scale);
            sum += X[i];
        }
        uint2 d0, d1, d2;
        d0.x = pack4(X[0] >> 14, X[1] >> 14, X[2] >> 14, X[3] >> 14);
        d0.y = pack4(X[4] >> 14, X[5] >> 14, X[6] >> 14, X[7] >> 14);
        d1.x = pack4(X[0] >> 7, X[1] >> 7, X[2] >> 7, X[3] >> 7) & 0x7F7F7F7Fu;
        d1.y = pack4(X[4] >> 7, X[5] >> 7, X[6] >> 7, X[7] >> 7) & 0x7F7F7F7Fu;
        d2.x = pack4(X[0], X[1], X[2], X[3]) & 0x7F7F7F7Fu;
        d2.y = pack4(X[4], X[5], X[6], X[7]) & 0x7F7F7F7Fu;
        uint8_t* dst = s.dig + (size_t)blk * 256 + 8 * lane;
        *reinterpret_cast<uint2*>(dst) = d0;
        *reinterpret_cast<uint2*>(dst + K) = d1;
        *reinterpret_cast<uint2*>(dst + 2 * (size_t)K) = d2;
        // sub-block sums: four lanes per sub-block
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        if ((lane & 3) == 0) s.sx[blk * 8 + (lane >> 2)] = (float)sum;
        if (lane == 0) s.xs[blk] = __uint_as_float((E + 1u - kFracBits) << 23);  // 2^-f = 2^(E-146)
    }
}

// Segment of a grouped launch that holds tile T.
__device__ __forceinline__ int seg_of(const WarpArgs& a, uint32_t T) {
    return (T >= a.seg_end[0] ? 1 : 0) + (T >= a.seg_end[1] ? 1 : 0);
}

// kSeg: 0 one matrix (pair), 1 grouped matrices (host-side segment table), 2 MoE slots (device-side routing)
// kMerge: the activation is merged from split-K attention partials while it is loaded (a kernel of its own, so
// that the plain matvec carries neither the code nor the arguments)
template <int NS, int EPI, int kWarps, int kSeg, bool kMerge>
__device__ __forceinline__ void dmmv_q4k_body(const WarpArgs& a, const MergeArgs& merge) {
    extern __shared__ uint8_t smem_raw[];
    pdl_begin(a);
    const Smem s = carve(smem_raw, a.K, kWarps);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t bpr = a.K >> 8;
    const uint64_t row_bytes = (uint64_t)bpr * 144;
    const uint32_t upt = (bpr + kCB - 1) / kCB;  // row segments (units) per row
    const uint32_t upt_all = upt * NS;            // units per 16-row tile
    const uint32_t tiles = kSeg == 1 ? a.seg_end[a.nseg - 1] : kSeg == 2 ? a.nseg * a.tiles_per_expert : (a.M + 15) / 16;
    const uint32_t U = tiles * upt_all, G = gridDim.x * kWarps;  // units, workers (G <= U)
    const uint32_t me = blockIdx.x * kWarps + warp;
    const uint32_t u0 = (uint32_t)part_begin(me, U, G), u1 = (uint32_t)part_begin(me + 1, U, G);
    const uint32_t n = u1 - u0;
    uint8_t* ring = s.ring + (size_t)warp * kWarpRing;

    // ---- prefetch: coalesced 16-byte asynchronous copies into padded row segments ----
    // piece p = i*32 + lane of a unit covers row p / kPiecesPerRow, 16-byte column p % kPiecesPerRow,
    // so one warp instruction reads 512 contiguous bytes of one or two rows.
    uint32_t piece[kPiecesPerLane];  // row | column << 8
#pragma unroll
    for (int i = 0; i < kPiecesPerLane; ++i) {
        const uint32_t p = i * 32 + lane;
        const uint32_t r = p / kPiecesPerRow;
        piece[i] = r | ((p - r * kPiecesPerRow) << 8);
    }
    uint32_t p_tile = u0 / upt_all, p_strm = (u0 % upt_all) / upt, p_kc = (u0 % upt_all) % upt;
    // per-lane source / destination offsets of its pieces (rows inside the matrix)
    uint32_t src_off[kPiecesPerLane], dst_off[kPiecesPerLane];
#pragma unroll
    for (int i = 0; i < kPiecesPerLane; ++i) {
        const uint32_t r = piece[i] & 0xFFu, c = piece[i] >> 8;
        src_off[i] = r * (uint32_t)row_bytes + c * 16;
        dst_off[i] = r * kRowSeg + c * 16;
    }
    auto request = [&](uint32_t slot) {
        const uint32_t cols = min((uint32_t)kCB, bpr - p_kc * kCB) * 9;  // 16-byte columns in this segment
        const uint32_t row0 = p_tile * 16;
        const uint8_t* base;
        uint32_t Mb;  // row bound in the indexing of `base`
        if constexpr (kSeg == 1) {
            const int sg = seg_of(a, p_tile);
            base = a.segA[sg];
            Mb = a.segM[sg];
        } else if constexpr (kSeg == 2) {
            const uint32_t slot = p_tile / a.tiles_per_expert, t0 = slot * a.tiles_per_expert * 16;
            const uint32_t e_raw = __ldg(a.routing + slot);
            if (e_raw == kSkipExpert) {  // no expert in this slot on this rank: nothing to fetch
                if (++p_kc == upt) {
                    p_kc = 0;
                    if (++p_strm == NS) { p_strm = 0; ++p_tile; }
                }
                return;
            }
            base = expert_matrix(a.A[p_strm], a.A_sh[p_strm], e_raw, a.expert_stride, a.n_experts_max, a.status) -
                   (uint64_t)t0 * row_bytes;
            Mb = t0 + a.M;
        } else {
            base = a.A[p_strm];
            Mb = a.M;
        }
        const uint8_t* src = base + (uint64_t)row0 * row_bytes + (uint64_t)p_kc * (kCB * 144);
        uint8_t* dst = ring + slot * kSlotBytes;
        if (row0 + 16 <= Mb && cols == kPiecesPerRow) {
#pragma unroll
            for (int i = 0; i < kPiecesPerLane; ++i) cp_async16(dst + dst_off[i], src + src_off[i]);
        } else {
            // last tile / last segment: rows past M repeat the last row (never written), short segment
#pragma unroll
            for (int i = 0; i < kPiecesPerLane; ++i) {
                const uint32_t r = piece[i] & 0xFFu, c = piece[i] >> 8;
                if (c < cols) {
                    const uint32_t row = min(row0 + r, Mb - 1);
                    cp_async16(dst + dst_off[i], src + (uint64_t)(row - row0) * row_bytes + c * 16);
                }
            }
        }
        if (++p_kc == upt) {
            p_kc = 0;
            if (++p_strm == NS) { p_strm = 0; ++p_tile; }
        }
    };
    // weights never depend on the previous kernel: fill the whole ring, then wait for that kernel, then
    // fetch x. (Behind a kernel that may still be writing the routing buffer the wait comes first, and x is
    // requested before the routing is read, so that the two round trips overlap.)
    pdl_late(a);
    XRegs xr;
    auto fetch_x = [&]() {
        if constexpr (kMerge) load_x_merge<kWarps>(xr, merge, a.K, warp, lane);
        else load_x<kWarps>(xr, a.x, a.K, warp, lane);
    };
    if (a.late) fetch_x();
#pragma unroll
    for (int i = 0; i < kDepth; ++i) {
        if ((uint32_t)i < n) request(i);
        cp_async_commit();
    }
    pdl_wait();
    if (!a.late) fetch_x();
    if (a.consume.n) consume_pushed(a.consume, blockIdx.x, gridDim.x, tid, kWarps * 32);

    // ---- activation vector -> digit planes (all warps), zero region, flags ----
    if (tid < kZeroBytes / 16) reinterpret_cast<uint4*>(s.zeros)[tid] = make_uint4(0u, 0u, 0u, 0u);
    if (tid < kWarps) s.sflags[tid] = 0u;
    prep_x<kWarps>(s, xr, a.K, warp, lane);
    __syncthreads();

    // ---- consume ----
    uint32_t tile = u0 / upt_all, strm = (u0 % upt_all) / upt, kc = (u0 % upt_all) % upt;
    // per stream, rows g and g+8: digit t's share of d * sum_s sc_s P_s (to be scaled by 2^(10 - 7t)) and this
    // lane's share of dmin * sum_s m_s SX_s
    float accM0[2] = {0.f, 0.f}, accM1[2] = {0.f, 0.f}, accm0[2] = {0.f, 0.f}, accm1[2] = {0.f, 0.f};
    // B operand: lane (g, t) feeds column g for its k slots (elements 64(t/2) + 16(t%2) .. +15 of a 128-element
    // pair of qs groups, +32 for the high nibbles). Column g = 2j + u is live for the lanes with t/2 == u and
    // reads digit plane j; the other lanes read zeros, at a bank offset the live lanes of their quarter-warp
    // do not touch (live: 32h + {0..31, 64..95} mod 128 for nibble half h; zeros at 32 + 32h).
    const bool b_live = g < 6 && (g & 1) == (t >> 1);
    const uint32_t xb_base = b_live ? smem_u32(s.dig) + (uint32_t)(g >> 1) * a.K + 64u * (t >> 1) + 16u * (t & 1)
                                    : smem_u32(s.zeros) + 32u;
    const uint32_t xb_step = b_live ? 256u : 0u;
    const uint32_t ring_s = smem_u32(ring), xs_s = smem_u32(s.xs), sx_s = smem_u32(s.sx) + 8u * t;
    const uint32_t msel = (2u * t) | ((2u * t + 1u) << 4) | 0x7700u;  // bytes 2t, 2t+1 of {mins 0..3, mins 4..7}
    // digit t's sum carries 2^(14 - 7t) and the 1/16 of the in-place high nibbles; lane t = 3 holds zeros
    const float dscale = __uint_as_float((127u + 10u - 7u * t) << 23);
    constexpr uint32_t kLo = 0x0F0F0F0Fu, kHi = 0xF0F0F0F0u;

    for (uint32_t it = 0; it < n; ++it) {
        const uint32_t slot = it % kDepth;
        cp_async_wait<kDepth - 1>();  // this lane's copies of unit `it` have landed
        __syncwarp();                 // ... and so have the other lanes'
        uint32_t nblk = min((uint32_t)kCB, bpr - kc * kCB);
        if constexpr (kSeg == 2) {  // a slot without an expert contributes zeros
            if (__ldg(a.routing + tile / a.tiles_per_expert) == kSkipExpert) nblk = 0;
        }
#pragma unroll
        for (uint32_t bi = 0; bi < (uint32_t)kCB; ++bi) {
            if (bi >= nblk) break;
            const uint32_t blk = kc * kCB + bi;
            const uint32_t sb = ring_s + slot * kSlotBytes + bi * 144;
            const uint32_t rA = sb + g * kRowSeg;
            const uint32_t rB = sb + (g + 8) * kRowSeg;
            const uint4 hA = lds_v4(rA), hB = lds_v4(rB);
            const uint32_t xb = xb_base + blk * xb_step;
            // 6-bit scales of sub-blocks 0..3 and 4..7, one per byte (getScaleMinK4, src/compute/forward.zig:229-238)
            const uint32_t scA[2] = {hA.y & 0x3F3F3F3Fu, (hA.w & 0x0F0F0F0Fu) | ((hA.y >> 2) & 0x30303030u)};
            const uint32_t scB[2] = {hB.y & 0x3F3F3F3Fu, (hB.w & 0x0F0F0F0Fu) | ((hB.y >> 2) & 0x30303030u)};
            int IloA = 0, IhiA = 0, IloB = 0, IhiB = 0;
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const uint4 qa = lds_v4(rA + 16 + 64 * p + 16 * t), qb = lds_v4(rB + 16 + 64 * p + 16 * t);
                const uint4 bl = lds_v4(xb + 128 * p), bh = lds_v4(xb + 128 * p + 32);
                int lo[4] = {0, 0, 0, 0}, hi[4] = {0, 0, 0, 0};
                mma_u8s8(lo, qa.x & kLo, qb.x & kLo, qa.y & kLo, qb.y & kLo, bl.x, bl.y);
                mma_u8s8(lo, qa.z & kLo, qb.z & kLo, qa.w & kLo, qb.w & kLo, bl.z, bl.w);
                mma_u8s8(hi, qa.x & kHi, qb.x & kHi, qa.y & kHi, qb.y & kHi, bh.x, bh.y);
                mma_u8s8(hi, qa.z & kHi, qb.z & kHi, qa.w & kHi, qb.w & kHi, bh.z, bh.w);
                // D columns 2t, 2t+1 = digit t of sub-blocks 4p (+1 for the high nibbles) and 4p + 2 (+1)
                const uint32_t sa = scA[p], sb2 = scB[p];
                IloA += lo[0] * (int)(sa & 0xFFu) + lo[1] * (int)((sa >> 16) & 0xFFu);
                IhiA += hi[0] * (int)((sa >> 8) & 0xFFu) + hi[1] * (int)(sa >> 24);
                IloB += lo[2] * (int)(sb2 & 0xFFu) + lo[3] * (int)((sb2 >> 16) & 0xFFu);
                IhiB += hi[2] * (int)((sb2 >> 8) & 0xFFu) + hi[3] * (int)(sb2 >> 24);
            }
            // the high nibbles were multiplied as 16 q: sum = (16 * lo + hi) / 16, the 1/16 sits in dscale
            const float PA = (float)(IloA * 16 + IhiA), PB = (float)(IloB * 16 + IhiB);
            // mins of sub-blocks 2t, 2t+1
            const uint32_t mnA = __byte_perm(hA.z & 0x3F3F3F3Fu, ((hA.w >> 4) & 0x0F0F0F0Fu) | ((hA.z >> 2) & 0x30303030u), msel);
            const uint32_t mnB = __byte_perm(hB.z & 0x3F3F3F3Fu, ((hB.w >> 4) & 0x0F0F0F0Fu) | ((hB.z >> 2) & 0x30303030u), msel);
            const float xs = lds_f1(xs_s + blk * 4);
            const float2 sxv = lds_f2(sx_s + blk * 32);
            const float dA = h2f(hA.x) * xs, dmA = h2f(hA.x >> 16) * xs;
            const float dB = h2f(hB.x) * xs, dmB = h2f(hB.x >> 16) * xs;
            const float mA = (float)(mnA & 0xFFu) * sxv.x + (float)((mnA >> 8) & 0xFFu) * sxv.y;
            const float mB = (float)(mnB & 0xFFu) * sxv.x + (float)((mnB >> 8) & 0xFFu) * sxv.y;
            if (NS == 1 || strm == 0) {
                accM0[0] = fmaf(dA, PA, accM0[0]);
                accM0[1] = fmaf(dB, PB, accM0[1]);
                accm0[0] = fmaf(dmA, mA, accm0[0]);
                accm0[1] = fmaf(dmB, mB, accm0[1]);
            } else {
                accM1[0] = fmaf(dA, PA, accM1[0]);
                accM1[1] = fmaf(dB, PB, accM1[1]);
                accm1[0] = fmaf(dmA, mA, accm1[0]);
                accm1[1] = fmaf(dmB, mB, accm1[1]);
            }
        }
        // every lane has consumed the stage: request the unit kDepth ahead into it
        __syncwarp();
        if (it + kDepth < n) request(slot);
        cp_async_commit();
        // advance; a tile ends with its last unit or with this worker's range
        const uint32_t T = tile;
        bool tile_done = false;
        if (++kc == upt) {
            kc = 0;
            if (++strm == NS) { strm = 0; ++tile; tile_done = true; }
        }
        if (tile_done || it + 1 == n) {
            float v[NS][2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float w = fmaf(accM0[r], dscale, -accm0[r]);
                w += __shfl_xor_sync(0xFFFFFFFFu, w, 1);
                w += __shfl_xor_sync(0xFFFFFFFFu, w, 2);
                v[0][r] = w;
                accM0[r] = accm0[r] = 0.f;
                if (NS == 2) {
                    float w1 = fmaf(accM1[r], dscale, -accm1[r]);
                    w1 += __shfl_xor_sync(0xFFFFFFFFu, w1, 1);
                    w1 += __shfl_xor_sync(0xFFFFFFFFu, w1, 2);
                    v[NS - 1][r] = w1;
                    accM1[r] = accm1[r] = 0.f;
                }
            }
            if constexpr (kSeg == 2) {
                const uint32_t slot = T / a.tiles_per_expert, t0 = slot * a.tiles_per_expert * 16;
                RowOut o{a.y + (size_t)slot * a.M - t0, a.y2 + (size_t)slot * a.M - t0, t0 + a.M, nullptr, nullptr};
                if (a.bias[0]) {  // the slot's expert's rows of the bias tables (none for a shared or absent expert)
                    const uint32_t e = __ldg(a.routing + slot);
                    if (e < a.n_experts_max) {
                        o.b0 = a.bias[0] + (size_t)e * a.M - t0;
                        o.b1 = a.bias[1] ? a.bias[1] + (size_t)e * a.M - t0 : nullptr;
                    }
                }
                finish_tile<NS, EPI, kWarps>(a, o, s.spartial, s.sflags, v, T, upt_all, u0, u1, U, G, me, warp, lane);
            } else if constexpr (kSeg == 1) {
                const int sg = seg_of(a, T);
                const RowOut o{sg == 0 ? a.segY[0] : sg == 1 ? a.segY[1] : a.segY[2], nullptr,
                               sg == 0 ? a.segM[0] : sg == 1 ? a.segM[1] : a.segM[2], nullptr, nullptr};
                finish_tile<NS, EPI, kWarps>(a, o, s.spartial, s.sflags, v, T, upt_all, u0, u1, U, G, me, warp, lane);
            } else {
                finish_tile<NS, EPI, kWarps>(a, row_out(a), s.spartial, s.sflags, v, T, upt_all, u0, u1, U, G, me, warp, lane);
            }
        }
    }
}

template <int NS, int EPI, int kWarps, int kSeg = 0>
__global__ void __launch_bounds__(kWarps * 32, 16 / kWarps) dmmv_q4k_warp_kernel(const WarpArgs a) {
    dmmv_q4k_body<NS, EPI, kWarps, kSeg, false>(a, MergeArgs());
}
template <int kWarps>
__global__ void __launch_bounds__(kWarps * 32, 16 / kWarps) dmmv_q4k_merge_kernel(const WarpArgs a, const MergeArgs m) {
    dmmv_q4k_body<1, EPI_PLAIN, kWarps, 0, true>(a, m);
}

template <int NS, int EPI, int kWarps, int kSeg = 0>
cudaError_t launch_w(const WarpArgs& a, cudaStream_t st, int sm_count, size_t smem) {
    auto kern = dmmv_q4k_warp_kernel<NS, EPI, kWarps, kSeg>;
    static std::atomic<uint64_t> attr_done{0};  // per device ordinal
    if (cudaError_t ea = ensure_dynamic_smem(kern, kWarps == 8 ? (int)kTwoPerSm : 227 * 1024, attr_done); ea != cudaSuccess) return ea;
    const uint64_t tiles = kSeg == 1 ? a.seg_end[a.nseg - 1] : kSeg == 2 ? (uint64_t)a.nseg * a.tiles_per_expert : (a.M + 15) / 16;
    const uint64_t U = tiles * (((a.K >> 8) + kCB - 1) / kCB) * NS;
    uint64_t grid = (uint64_t)sm_count * (16 / kWarps);  // 16 worker warps per SM
    if (grid * kWarps > U) grid = U / kWarps;
    if (grid * kWarps > kStreamMaxWorkers) grid = kStreamMaxWorkers / kWarps;
    if (grid == 0) return cudaErrorInvalidConfiguration;
    return launch_pdl(kern, (uint32_t)grid, kWarps * 32, smem, st, a);
}

template <int kWarps>
cudaError_t launch_w_merge(const WarpArgs& a, const MergeArgs& m, cudaStream_t st, int sm_count, size_t smem) {
    auto kern = dmmv_q4k_merge_kernel<kWarps>;
    static std::atomic<uint64_t> attr_done{0};  // per device ordinal
    if (cudaError_t ea = ensure_dynamic_smem(kern, kWarps == 8 ? (int)kTwoPerSm : 227 * 1024, attr_done); ea != cudaSuccess) return ea;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * (((a.K >> 8) + kCB - 1) / kCB);
    uint64_t grid = (uint64_t)sm_count * (16 / kWarps);
    if (grid * kWarps > U) grid = U / kWarps;
    if (grid * kWarps > kStreamMaxWorkers) grid = kStreamMaxWorkers / kWarps;
    if (grid == 0) return cudaErrorInvalidConfiguration;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((uint32_t)grid, 1, 1);
    cfg.blockDim = dim3(kWarps * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, a, m);
}

template <int NS, int EPI>
cudaError_t launch_cfg(const WarpArgs& a, cudaStream_t st, int sm_count) {
    const size_t s8 = smem_bytes(a.K, 8);
    if (s8 <= kTwoPerSm) return launch_w<NS, EPI, 8>(a, st, sm_count, s8);  // two CTAs per SM
    return launch_w<NS, EPI, 16>(a, st, sm_count, smem_bytes(a.K, 16));
}

}  // namespace

bool warp_dmmv_eligible(uint32_t type, int mode, const DmmvArgs& a) {
    if (type != T_Q4_K) return false;
    if (a.merge.partial && (mode != MODE_PLAIN || a.merge.n_chunks > (uint32_t)kMergeChunks || (a.merge.head_dim & 7u) ||
                            (reinterpret_cast<uintptr_t>(a.merge.partial) & 15u)))
        return false;
    if (mode != MODE_PLAIN && mode != MODE_GATE_UP_SWIGLU && mode != MODE_SIGMOID_ACC) return false;
    if (!a.scratch_partial || !a.status) return false;
    if ((reinterpret_cast<uintptr_t>(a.A) & 15u) || (a.A2 && (reinterpret_cast<uintptr_t>(a.A2) & 15u))) return false;
    if (smem_bytes(a.K, 16) > 227 * 1024 || (a.K >> 8) > (uint32_t)(kPrepBlocks * 8)) return false;
    const int ns = mode == MODE_GATE_UP_SWIGLU ? 2 : 1;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * (((a.K >> 8) + kCB - 1) / kCB) * ns;
    if (U < 16 || U > 0xFFFFFFFFull) return false;
    return true;
}

cudaError_t launch_warp_dmmv(uint32_t type, int mode, const DmmvArgs& a, cudaStream_t st, uint64_t* launches) {
    (void)type;
    WarpArgs wa;
    wa.A[0] = a.A;
    wa.A[1] = a.A2 ? a.A2 : a.A;
    wa.x = a.x;
    wa.y = a.y;
    wa.gate = a.gate;
    wa.M = a.M;
    wa.K = a.K;
    wa.acc_mode = a.acc_mode;
    wa.gpartial = a.scratch_partial;
    wa.status = a.status;
    wa.spin_limit = a.spin_limit;
    wa.nseg = 0;
    wa.push = a.push;
    wa.consume = a.consume;
    wa.late = a.late;
    cudaError_t e;
    switch (mode) {
        case MODE_PLAIN:
            if (a.merge.partial) {
                const size_t s8 = smem_bytes(a.K, 8);
                e = s8 <= kTwoPerSm ? launch_w_merge<8>(wa, a.merge, st, a.sm_count, s8)
                                    : launch_w_merge<16>(wa, a.merge, st, a.sm_count, smem_bytes(a.K, 16));
            } else {
                e = launch_cfg<1, EPI_PLAIN>(wa, st, a.sm_count);
            }
            break;
        case MODE_GATE_UP_SWIGLU: e = launch_cfg<2, EPI_GATE_UP>(wa, st, a.sm_count); break;
        case MODE_SIGMOID_ACC: e = launch_cfg<1, EPI_SIGMOID_ACC>(wa, st, a.sm_count); break;
        default: return cudaErrorInvalidValue;
    }
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

// Grouped launch: n <= 3 Q4_K matrices with the same K and the same x, y_i = W_i x, in one kernel.
bool warp_dmmv_multi_eligible(uint32_t type, uint32_t n, const uint8_t* const* A, const uint32_t* M, uint32_t K,
                              const DmmvArgs& common) {
    if (type != T_Q4_K || n < 2 || n > 3) return false;
    if (!common.scratch_partial || !common.status) return false;
    if (smem_bytes(K, 16) > 227 * 1024 || (K >> 8) > (uint32_t)(kPrepBlocks * 8) || (K & 255u)) return false;
    uint64_t tiles = 0;
    for (uint32_t i = 0; i < n; ++i) {
        if (reinterpret_cast<uintptr_t>(A[i]) & 15u) return false;
        if (M[i] == 0) return false;
        tiles += (M[i] + 15) / 16;
    }
    const uint64_t U = tiles * (((K >> 8) + kCB - 1) / kCB);
    return U >= 16 && U <= 0xFFFFFFFFull;
}

cudaError_t launch_warp_dmmv_multi(uint32_t n, const uint8_t* const* A, float* const* y, const uint32_t* M,
                                   const DmmvArgs& common, cudaStream_t st, uint64_t* launches) {
    WarpArgs wa;
    wa.A[0] = wa.A[1] = A[0];
    wa.x = common.x;
    wa.y = y[0];
    wa.gate = nullptr;
    wa.M = M[0];
    wa.K = common.K;
    wa.acc_mode = common.acc_mode;
    wa.gpartial = common.scratch_partial;
    wa.status = common.status;
    wa.spin_limit = common.spin_limit;
    wa.consume = common.consume;
    wa.late = common.late;
    wa.nseg = n;
    const uint64_t row_bytes = (uint64_t)(common.K >> 8) * 144;
    uint32_t t0 = 0;
    for (uint32_t i = 0; i < 3; ++i) {
        if (i < n) {
            // shift by the segment's first tile: the kernel indexes with global tile / row numbers
            wa.segA[i] = A[i] - (uint64_t)t0 * 16 * row_bytes;
            wa.segY[i] = y[i] - (uint64_t)t0 * 16;
            wa.segM[i] = t0 * 16 + M[i];
            t0 += (M[i] + 15) / 16;
            wa.seg_end[i] = t0;
        } else {
            wa.segA[i] = nullptr;
            wa.segY[i] = nullptr;
            wa.segM[i] = 0;
            wa.seg_end[i] = 0xFFFFFFFFu;
        }
    }
    if (n == 2) wa.seg_end[1] = t0;
    const size_t s8 = smem_bytes(common.K, 8);
    cudaError_t e = s8 <= kTwoPerSm ? launch_w<1, EPI_PLAIN, 8, 1>(wa, st, common.sm_count, s8)
                                    : launch_w<1, EPI_PLAIN, 16, 1>(wa, st, common.sm_count,
                                                                        smem_bytes(common.K, 16));
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

// MoE fused gate + up: y_gate[s][M], y_up[s][M] = Wg[routing[s]] x, Wu[routing[s]] x for the n_used slots, x shared.
bool warp_moe_gate_up_eligible(uint32_t type, const DmmvArgs& a) {
    if (type != T_Q4_K || a.x_expert_stride != 0 || !a.routing || !a.A2 || (!a.y2 && !a.act)) return false;
    if (!a.scratch_partial || !a.status) return false;
    if ((reinterpret_cast<uintptr_t>(a.A) & 15u) || (reinterpret_cast<uintptr_t>(a.A2) & 15u) || (a.expert_stride & 15u))
        return false;
    if ((reinterpret_cast<uintptr_t>(a.A_sh) & 15u) || (reinterpret_cast<uintptr_t>(a.A2_sh) & 15u)) return false;
    if ((a.K & 255u) || smem_bytes(a.K, 16) > 227 * 1024 || (a.K >> 8) > (uint32_t)(kPrepBlocks * 8)) return false;
    const uint64_t U = (uint64_t)a.n_used * ((a.M + 15) / 16) * (((a.K >> 8) + kCB - 1) / kCB) * 2;
    return a.n_used >= 1 && U >= 16 && U <= 0xFFFFFFFFull;
}

cudaError_t launch_warp_moe_gate_up(const DmmvArgs& a, cudaStream_t st, uint64_t* launches) {
    WarpArgs wa;
    wa.A[0] = a.A;
    wa.A[1] = a.A2;
    wa.x = a.x;
    wa.y = a.y;
    wa.y2 = a.y2;
    wa.act = a.act;
    wa.gate = nullptr;
    wa.M = a.M;
    wa.K = a.K;
    wa.acc_mode = 0;
    wa.gpartial = a.scratch_partial;
    wa.status = a.status;
    wa.spin_limit = a.spin_limit;
    wa.nseg = a.n_used;
    wa.routing = a.routing;
    wa.n_experts_max = a.n_experts_max;
    wa.expert_stride = a.expert_stride;
    wa.tiles_per_expert = (a.M + 15) / 16;
    wa.A_sh[0] = a.A_sh;
    wa.A_sh[1] = a.A2_sh;
    wa.bias[0] = a.bias;
    wa.bias[1] = a.bias2;
    wa.late = a.late;
    const size_t s8 = smem_bytes(a.K, 8);
    cudaError_t e = s8 <= kTwoPerSm ? launch_w<2, EPI_PAIR, 8, 2>(wa, st, a.sm_count, s8)
                                    : launch_w<2, EPI_PAIR, 16, 2>(wa, st, a.sm_count, smem_bytes(a.K, 16));
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
