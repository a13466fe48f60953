// Warp-autonomous streaming decode matvec for B200 (Q4_K), integer tensor-core dot engine.
//
// Every warp is an independent worker: it owns a contiguous range of work units (16 rows x
// kCB 256-weight super-blocks), prefetches them with coalesced 16-byte asynchronous copies
// (cp.async into the warp's own ring of padded row segments, depth kDepth; bulk TMA copies were
// measured at ~14 cycles of issue each per SM, too slow for 288-byte row segments), masks the 4-bit
// quants into int8 lanes (one logic op per four weights) and feeds them to the int8 tensor cores as a 16-row dot-product engine with exact
// s32 accumulation. There is no block-wide synchronisation after the activation vector has
// been converted. K is split across workers so that all SMs stream the same number of bytes;
// a tile that spans several workers is finished by the worker that owns its first unit, which
// adds the partial sums the later workers have published (shared memory inside a CTA, global
// memory across CTAs) in worker order, so results do not depend on timing.
//
// Stands in for the reference's K-parallel decode shaders and their fused epilogues
// (src/shaders/dmmv_q4k.comp:59-240, dmmv_q4k_wide.comp, dmmv_q4k_fused_gate_up_swiglu.comp:195-218,
// dmmv_q8_0_sigmoid_acc.comp:95-132) for the Q4_K layout of src/compute/forward.zig:370-409.
//
// Arithmetic per super-block of a row, sub-blocks s = 0..7 of 32 weights:
//   y += 2^-f * ( d * sum_s sc_s * P_s  -  dmin * sum_s m_s * SX_s ),   P_s = sum_i q_i * X_i
// X_i = round(x_i * 2^f) is the block of x in 21-bit fixed point (f chosen per 256-element block
// from its largest magnitude), split into three 7-bit digits X = b0*2^14 + b1*2^7 + b2 that fit
// int8. The tensor core computes sum_i q_i * b_j,i exactly in s32 for each digit; P_s is
// reassembled in integer arithmetic, SX_s = sum_i X_i is exact too. Weights are never rounded;
// the only rounding before the final f32 scaling is that of x to 21 bits.
//
// Tensor-core mapping (mma.sync m16n8k32, s8 in, s32 out): the 16 A rows are 16 weight rows;
// lane (g = lane/4, t = lane%4) owns the 32-byte qs group t of rows g and g+8, i.e. sub-blocks
// 2t (low nibbles) and 2t+1 (high nibbles). B is block-diagonal: columns 2t and 2t+1 are
// non-zero only in lane t's k slots, so those D columns hold dot products of group t alone and
// land in lane t's own accumulator registers. Scales are applied per lane afterwards.
#include "kernels.h"
#include "stream_skel.cuh"

namespace zc {

namespace {

constexpr int kDepth = 2;                  // units in flight per warp
constexpr int kCB = 2;                     // super-blocks per row segment
constexpr int kRowSeg = kCB * 144 + 16;    // 304: rows land 16 B apart mod 32 B -> conflict-free 128-bit reads
constexpr int kSlotBytes = 16 * kRowSeg;
constexpr int kWarpRing = kDepth * kSlotBytes;
constexpr size_t kTwoPerSm = 113 * 1024;   // shared memory per CTA that still lets two CTAs share an SM
constexpr int kZeroUnits = 72;             // zeros: B operand of the lanes whose columns are dead
constexpr int kFracBits = 20;              // |X| <= 2^20
constexpr int kPiecesPerRow = kCB * 9;     // 16-byte pieces of one row segment
constexpr int kPiecesPerLane = (16 * kPiecesPerRow + 31) / 32;

struct Smem {
    uint4* xf;       // x digits in B-operand order: unit ((blk*8 + s*4 + j)*2 + p)*4 + t
    uint4* zeros;    // kZeroUnits zero units
    float* sx;       // per 32-element sub-block sum of X
    float* xs;       // per super-block 2^-f
    uint8_t* ring;   // [kWarps][kDepth] stages of 16 padded row segments
    float* spartial; // [kWarps][32] partial sums published inside the CTA
    volatile uint32_t* sflags;  // [kWarps]
};

__host__ __device__ inline size_t smem_bytes(uint32_t K, int kWarps) {
    size_t n = (size_t)K * 4 + (size_t)kZeroUnits * 16;
    n += (size_t)(K / 32) * 4 + (size_t)(K / 256) * 4;
    n = (n + 127) & ~size_t(127);
    n += (size_t)kWarps * kWarpRing;
    n += (size_t)kWarps * 32 * 4 + (size_t)kWarps * 4 + 16;
    return n + 128;
}

__device__ inline Smem carve(uint8_t* base, uint32_t K, int kWarps) {
    Smem s;
    uintptr_t p = (reinterpret_cast<uintptr_t>(base) + 127) & ~uintptr_t(127);
    s.xf = reinterpret_cast<uint4*>(p);
    p += (size_t)K * 4;
    s.zeros = reinterpret_cast<uint4*>(p);
    p += (size_t)kZeroUnits * 16;
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


// Convert x into int8 digits in tensor-core operand order. One warp per super-block;
// lane = j*8 + s*4 + t handles the 8 consecutive elements 64t + 32s + 8j .. +7 (bytes 8j..8j+7
// of qs group t; s = 0 low nibbles, 1 high nibbles). Unit p = 0 holds (digit 0 | digit 2) of
// those 8 elements, unit p = 1 (digit 1 | zeros): the two B register pairs of the lanes that
// feed columns 2t and 2t+1.
//
// The loads are issued before the weight prefetch (so they are not queued behind it) and
// converted afterwards: kPrepBlocks super-blocks per warp cover K <= kPrepBlocks * kWarps * 256.
constexpr int kPrepBlocks = 6;  // x super-blocks per warp: K <= kPrepBlocks * kWarps * 256
struct XRegs {
    float4 lo[kPrepBlocks], hi[kPrepBlocks];
};
template <int kWarps>
__device__ __forceinline__ void load_x(XRegs& r, const float* __restrict__ x, uint32_t K, int warp, int lane) {
    const int j = lane >> 3, sh = (lane >> 2) & 1, t = lane & 3;
#pragma unroll
    for (int i = 0; i < kPrepBlocks; ++i) {
        const uint32_t blk = warp + i * kWarps;
        if (blk < (K >> 8)) {
            const float* xp = x + (size_t)blk * 256 + 64 * t + 32 * sh + 8 * j;
            r.lo[i] = __ldg(reinterpret_cast<const float4*>(xp));
            r.hi[i] = __ldg(reinterpret_cast<const float4*>(xp) + 1);
        }
    }
}
template <int kWarps>
__device__ __forceinline__ void prep_x(const Smem& s, const XRegs& r, uint32_t K, int warp, int lane) {
    const int j = lane >> 3, sh = (lane >> 2) & 1, t = lane & 3;
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
        uint32_t d0[2] = {0, 0}, d1[2] = {0, 0}, d2[2] = {0, 0};
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int X = __float2int_rn(v[i] * scale);
            sum += X;
            d0[i >> 2] |= (uint32_t)((X >> 14) & 0xFF) << (8 * (i & 3));
            d1[i >> 2] |= (uint32_t)((X >> 7) & 0x7F) << (8 * (i & 3));
            d2[i >> 2] |= (uint32_t)(X & 0x7F) << (8 * (i & 3));
        }
        const uint32_t u = (blk * 8 + sh * 4 + j) * 2;
        s.xf[(u + 0) * 4 + t] = make_uint4(d0[0], d0[1], d2[0], d2[1]);
        s.xf[(u + 1) * 4 + t] = make_uint4(d1[0], d1[1], 0u, 0u);
        // sub-block sums: reduce over j (lane bits 3 and 4)
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 8);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 16);
        if (j == 0) s.sx[blk * 8 + 2 * t + sh] = (float)sum;
        if (lane == 0) s.xs[blk] = __uint_as_float((E + 1u - kFracBits) << 23);  // 2^-f = 2^(E-146)
    }
}

// Two 6-bit scales and two 6-bit mins of sub-blocks 2t and 2t+1, each pair packed in the low
// 16 bits (getScaleMinK4, src/compute/forward.zig:229-238, evaluated for two indices at once).
__device__ __forceinline__ void scales_mins_pair(uint32_t s0, uint32_t s1, uint32_t s2, int t, uint32_t& sc,
                                                 uint32_t& mn) {
    const uint32_t sh = 16u * (t & 1);
    const uint32_t p0 = s0 >> sh, p1 = s1 >> sh, p2 = s2 >> sh;
    const uint32_t lo_sc = p0 & 0x3F3Fu, lo_mn = p1 & 0x3F3Fu;
    const uint32_t hi_sc = (p2 & 0x0F0Fu) | ((p0 >> 2) & 0x3030u);
    const uint32_t hi_mn = ((p2 >> 4) & 0x0F0Fu) | ((p1 >> 2) & 0x3030u);
    sc = t < 2 ? lo_sc : hi_sc;
    mn = t < 2 ? lo_mn : hi_mn;
}


// Segment of a grouped launch that holds tile T.
__device__ __forceinline__ int seg_of(const WarpArgs& a, uint32_t T) {
    return (T >= a.seg_end[0] ? 1 : 0) + (T >= a.seg_end[1] ? 1 : 0);
}

// kSeg: 0 one matrix (pair), 1 grouped matrices (host-side segment table), 2 MoE slots (device-side routing)
template <int NS, int EPI, int kWarps, int kSeg = 0>
__global__ void __launch_bounds__(kWarps * 32, 16 / kWarps) dmmv_q4k_warp_kernel(const WarpArgs a) {
    extern __shared__ uint8_t smem_raw[];
    pdl_launch_dependents();
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
            base = a.A[p_strm] + (uint64_t)checked_expert(__ldg(a.routing + slot), a.n_experts_max, a.status) * a.expert_stride -
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
    // weights never depend on the previous kernel: start streaming them, then wait for it, then
    // fetch x (ahead of the rest of the prefetch in the memory queues)
    if (n) request(0);
    cp_async_commit();
    pdl_wait();
    XRegs xr;
    load_x<kWarps>(xr, a.x, a.K, warp, lane);
#pragma unroll
    for (int i = 1; i < kDepth; ++i) {
        if ((uint32_t)i < n) request(i);
        cp_async_commit();
    }

    // ---- activation vector -> B operand layout (all warps), zero region, flags ----
    if (tid < kZeroUnits) s.zeros[tid] = make_uint4(0u, 0u, 0u, 0u);
    if (tid < kWarps) s.sflags[tid] = 0u;
    prep_x<kWarps>(s, xr, a.K, warp, lane);
    __syncthreads();

    // ---- consume ----
    uint32_t tile = u0 / upt_all, strm = (u0 % upt_all) / upt, kc = (u0 % upt_all) % upt;
    float acc0[2] = {0.f, 0.f}, acc1[2] = {0.f, 0.f};  // stream 0 / stream 1, rows g and g+8
    const bool b_live = (g >> 1) == t;  // lane (g, t) feeds B column g, live only for g in {2t, 2t+1}
    const uint32_t xu_live = smem_u32(s.xf + (g & 1) * 4 + t);
    const uint32_t xu_dead = smem_u32(s.zeros + (g >> 1) + 1);  // a bank group no live lane of the same quarter-warp uses
    const uint32_t ring_s = smem_u32(ring), xs_s = smem_u32(s.xs), sx_s = smem_u32(s.sx);

    for (uint32_t it = 0; it < n; ++it) {
        const uint32_t slot = it % kDepth;
        cp_async_wait<kDepth - 1>();  // this lane's copies of unit `it` have landed
        __syncwarp();                 // ... and so have the other lanes'
        const uint32_t nblk = min((uint32_t)kCB, bpr - kc * kCB);
#pragma unroll
        for (uint32_t bi = 0; bi < (uint32_t)kCB; ++bi) {
            if (bi >= nblk) break;
            const uint32_t blk = kc * kCB + bi;
            const uint32_t sb = ring_s + slot * kSlotBytes + bi * 144;
            const uint32_t rA = sb + g * kRowSeg;
            const uint32_t rB = sb + (g + 8) * kRowSeg;
            const uint4 hA = lds_v4(rA), hB = lds_v4(rB);
            const uint4 qa0 = lds_v4(rA + 16 + 32 * t), qa1 = lds_v4(rA + 32 + 32 * t);
            const uint4 qb0 = lds_v4(rB + 16 + 32 * t), qb1 = lds_v4(rB + 32 + 32 * t);
            const uint32_t qa[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
            const uint32_t qb[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
            const uint32_t xu = b_live ? xu_live + blk * 1024u : xu_dead;  // 64 units of 16 bytes per super-block
            // D01: digits 0 and 1 in this lane's columns 2t, 2t+1; D2: digit 2 in column 2t
            int lo01[4] = {0, 0, 0, 0}, lo2[4] = {0, 0, 0, 0}, hi01[4] = {0, 0, 0, 0}, hi2[4] = {0, 0, 0, 0};
            constexpr uint32_t kNib = 0x0F0F0F0Fu;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 bl = lds_v4(xu + j * 128), bh = lds_v4(xu + (4 + j) * 128);
                const uint32_t a0 = qa[2 * j], a1 = qb[2 * j], a2 = qa[2 * j + 1], a3 = qb[2 * j + 1];
                const uint32_t l0 = a0 & kNib, l1 = a1 & kNib, l2 = a2 & kNib, l3 = a3 & kNib;
                mma_s8(lo01, l0, l1, l2, l3, bl.x, bl.y);
                mma_s8(lo2, l0, l1, l2, l3, bl.z, bl.w);
                const uint32_t h0 = (a0 >> 4) & kNib, h1 = (a1 >> 4) & kNib, h2 = (a2 >> 4) & kNib,
                               h3 = (a3 >> 4) & kNib;
                mma_s8(hi01, h0, h1, h2, h3, bh.x, bh.y);
                mma_s8(hi2, h0, h1, h2, h3, bh.z, bh.w);
            }
            // P = D0 * 2^14 + D1 * 2^7 + D2, exact in s32 (|P| < 2^31 for 5-bit quants and below)
            const float PloA = (float)(lo01[0] * 16384 + lo01[1] * 128 + lo2[0]);
            const float PloB = (float)(lo01[2] * 16384 + lo01[3] * 128 + lo2[2]);
            const float PhiA = (float)(hi01[0] * 16384 + hi01[1] * 128 + hi2[0]);
            const float PhiB = (float)(hi01[2] * 16384 + hi01[3] * 128 + hi2[2]);
            uint32_t scA, mnA, scB, mnB;
            scales_mins_pair(hA.y, hA.z, hA.w, t, scA, mnA);
            scales_mins_pair(hB.y, hB.z, hB.w, t, scB, mnB);
            const float xs = lds_f1(xs_s + blk * 4);
            const float2 sxv = lds_f2(sx_s + (blk * 8 + 2 * t) * 4);
            const float dA = h2f(hA.x) * xs, dmA = h2f(hA.x >> 16) * xs;
            const float dB = h2f(hB.x) * xs, dmB = h2f(hB.x >> 16) * xs;
            const float vA = dA * ((float)(scA & 0xFFu) * PloA + (float)(scA >> 8) * PhiA) -
                             dmA * ((float)(mnA & 0xFFu) * sxv.x + (float)(mnA >> 8) * sxv.y);
            const float vB = dB * ((float)(scB & 0xFFu) * PloB + (float)(scB >> 8) * PhiB) -
                             dmB * ((float)(mnB & 0xFFu) * sxv.x + (float)(mnB >> 8) * sxv.y);
            if (NS == 1 || strm == 0) { acc0[0] += vA; acc0[1] += vB; }
            else { acc1[0] += vA; acc1[1] += vB; }
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
                float w = acc0[r];
                w += __shfl_xor_sync(0xFFFFFFFFu, w, 1);
                w += __shfl_xor_sync(0xFFFFFFFFu, w, 2);
                v[0][r] = w;
                acc0[r] = 0.f;
                if (NS == 2) {
                    float w1 = acc1[r];
                    w1 += __shfl_xor_sync(0xFFFFFFFFu, w1, 1);
                    w1 += __shfl_xor_sync(0xFFFFFFFFu, w1, 2);
                    v[NS - 1][r] = w1;
                    acc1[r] = 0.f;
                }
            }
            if constexpr (kSeg == 2) {
                WarpArgs am = a;
                const uint32_t slot = T / a.tiles_per_expert, t0 = slot * a.tiles_per_expert * 16;
                am.y = a.y + (size_t)slot * a.M - t0;
                am.y2 = a.y2 + (size_t)slot * a.M - t0;
                am.M = t0 + a.M;
                finish_tile<NS, EPI, kWarps>(am, s.spartial, s.sflags, v, T, upt_all, u0, u1, U, G, me, warp, lane);
            } else if constexpr (kSeg == 1) {
                WarpArgs am = a;
                const int sg = seg_of(a, T);
                am.y = a.segY[sg];
                am.M = a.segM[sg];
                finish_tile<NS, EPI, kWarps>(am, s.spartial, s.sflags, v, T, upt_all, u0, u1, U, G, me, warp, lane);
            } else {
                finish_tile<NS, EPI, kWarps>(a, s.spartial, s.sflags, v, T, upt_all, u0, u1, U, G, me, warp, lane);
            }
        }
    }
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

template <int NS, int EPI>
cudaError_t launch_cfg(const WarpArgs& a, cudaStream_t st, int sm_count) {
    const size_t s8 = smem_bytes(a.K, 8);
    if (s8 <= kTwoPerSm) return launch_w<NS, EPI, 8>(a, st, sm_count, s8);  // two CTAs per SM
    return launch_w<NS, EPI, 16>(a, st, sm_count, smem_bytes(a.K, 16));
}

}  // namespace

bool warp_dmmv_eligible(uint32_t type, int mode, const DmmvArgs& a) {
    if (type != T_Q4_K) return false;
    if (mode != MODE_PLAIN && mode != MODE_GATE_UP_SWIGLU && mode != MODE_SIGMOID_ACC) return false;
    if (!a.scratch_partial || !a.scratch_flags || !a.status) return false;
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
    wa.gflags = a.scratch_flags;
    wa.status = a.status;
    wa.spin_limit = a.spin_limit;
    wa.nseg = 0;
    cudaError_t e;
    switch (mode) {
        case MODE_PLAIN: e = launch_cfg<1, EPI_PLAIN>(wa, st, a.sm_count); break;
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
    if (!common.scratch_partial || !common.scratch_flags || !common.status) return false;
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
    wa.gflags = common.scratch_flags;
    wa.status = common.status;
    wa.spin_limit = common.spin_limit;
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
    if (type != T_Q4_K || a.x_expert_stride != 0 || !a.routing || !a.A2 || !a.y2) return false;
    if (!a.scratch_partial || !a.scratch_flags || !a.status) return false;
    if ((reinterpret_cast<uintptr_t>(a.A) & 15u) || (reinterpret_cast<uintptr_t>(a.A2) & 15u) || (a.expert_stride & 15u))
        return false;
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
    wa.gflags = a.scratch_flags;
    wa.status = a.status;
    wa.spin_limit = a.spin_limit;
    wa.nseg = a.n_used;
    wa.routing = a.routing;
    wa.n_experts_max = a.n_experts_max;
    wa.expert_stride = a.expert_stride;
    wa.tiles_per_expert = (a.M + 15) / 16;
    const size_t s8 = smem_bytes(a.K, 8);
    cudaError_t e = s8 <= kTwoPerSm ? launch_w<2, EPI_PAIR, 8, 2>(wa, st, a.sm_count, s8)
                                    : launch_w<2, EPI_PAIR, 16, 2>(wa, st, a.sm_count, smem_bytes(a.K, 16));
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
