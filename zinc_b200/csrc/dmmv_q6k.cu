// Warp-autonomous streaming decode matvec for B200 (Q6_K), integer tensor-core dot engine.
// Same skeleton as the Q4_K kernel (stream_skel.cuh): every warp owns a contiguous range of
// (16 rows x one 256-weight super-block) units, prefetches them with coalesced 16-byte
// asynchronous copies and finishes split tiles in worker order.
//
// Stands in for src/shaders/dmmv_q6k.comp:58-156 (and its use for the down projection and the LM
// head, src/compute/forward.zig:7420, 7714) for the Q6_K layout of src/compute/forward.zig:276-325:
// 210-byte blocks ql[128] qh[64] scales[16] (int8) d (f16), 16-weight sub-blocks.
//
// Arithmetic per super-block of a row:  y += 2^-f * d * sum_s sc_s * P_s,
//   P_s = sum_{i in s} (v_i - 32) * X_i = sum_j 2^(14-7j) (D_j,s - 32 * SB_j,s),   D_j,s = sum_i v_i * b_j,i
// v_i = 6-bit quant 0..63 fed to the tensor core as u8, X_i = round(x_i * 2^f) the block of x in 21-bit fixed
// point, b_j,i its three digits (s8), SB_j,s = sum_i b_j,i. The MMA accumulators start at -32 * SB_j,s, the
// int8 scales are applied in integer arithmetic (sum_s sc_s * (..) < 2^31), so one conversion and one f32
// multiply-add per row, digit and super-block remain; the only rounding before that is x to 21 bits.
//
// Blocks are only 2-byte aligned (210 = 13*16 + 2), so a unit is copied as the 16-byte aligned superset of
// each row's block into a 240-byte row slot and read back with 32-bit loads: lane (g = lane/4, t = lane%4)
// reads word t of every 16-byte group of rows g and g+8 (bank = 4 * (15 g mod 8) + t + const: conflict-free),
// one load when the block starts on a word boundary inside its slot, two and a funnel shift otherwise.
// That is the native A fragment of mma.sync m16n8k32 (bytes 4t .. 4t+3 and 16 + 4t .. of a 32-byte group):
// an MMA covers the 32 elements 128h + 32j .. of half h, quarter j, i.e. sub-blocks 8h + 2j (k slots 0..15)
// and 8h + 2j + 1 (k slots 16..31). B is block-diagonal to match: column 2d + u holds digit d of x in the k
// slots of sub-block half u and zeros in the other half, so D column 2d + u is digit d's dot product with
// sub-block u alone; lane t < 3 ends up with digit t of both sub-blocks for rows g and g+8.
#include "kernels.h"
#include "stream_skel.cuh"

namespace zc {

namespace {

constexpr int kDepth = 2;
constexpr int kRow6 = 240;                  // bytes per row slot: 224-byte superset + pad (15 x 16: odd)
constexpr int kSlot6 = 16 * kRow6;
constexpr int kRing6 = kDepth * kSlot6;
constexpr int kPieces6 = 14;                // 16-byte pieces per row superset
constexpr int kPiecesLane6 = (16 * kPieces6 + 31) / 32;  // 7
constexpr int kZeroBytes6 = 128;
constexpr int kFracBits = 20;
constexpr int kPrepBlocks = 6;
constexpr int kBBytes = 1536;               // B operand table per super-block: [h 2][j pair 2][column 6][t 4][16 bytes]
constexpr int kNsxBytes = 256;              // accumulator start values per super-block: [h 2][digit 4][j 4][u 2] s32
constexpr size_t kTwoPerSm = 113 * 1024;

struct Smem6 {
    uint8_t* zeros;  // kZeroBytes6 of zeros (B operand of the dead columns 6 and 7)
    uint8_t* bq;     // per super-block kBBytes: {b0, b1} register pairs in B-operand order
    int* nsx;        // per super-block kNsxBytes / 4: -32 * sum of digit d over sub-block (h, j, u)
    float* xs;       // per super-block 2^-f
    uint8_t* ring;   // [kWarps][kDepth] stages of 16 row slots
    float* spartial; // [kWarps][32] partial sums published inside the CTA
    volatile uint32_t* sflags;  // [kWarps]
};

__host__ __device__ inline size_t smem_bytes6(uint32_t K, int kWarps) {
    size_t n = (size_t)kZeroBytes6 + (size_t)(K / 256) * (kBBytes + kNsxBytes + 4);
    n = (n + 127) & ~size_t(127);
    n += (size_t)kWarps * kRing6;
    n += (size_t)kWarps * 32 * 4 + (size_t)kWarps * 4 + 16;
    return n + 128;
}

__device__ inline Smem6 carve6(uint8_t* base, uint32_t K, int kWarps) {
    Smem6 s;
    uintptr_t p = (reinterpret_cast<uintptr_t>(base) + 127) & ~uintptr_t(127);
    s.zeros = reinterpret_cast<uint8_t*>(p);
    p += kZeroBytes6;
    s.bq = reinterpret_cast<uint8_t*>(p);
    p += (size_t)(K / 256) * kBBytes;
    s.nsx = reinterpret_cast<int*>(p);
    p += (size_t)(K / 256) * kNsxBytes;
    s.xs = reinterpret_cast<float*>(p);
    p += (size_t)(K / 256) * 4;
    p = (p + 127) & ~uintptr_t(127);
    s.ring = reinterpret_cast<uint8_t*>(p);
    p += (size_t)kWarps * kRing6;
    s.spartial = reinterpret_cast<float*>(p);
    p += (size_t)kWarps * 32 * 4;
    s.sflags = reinterpret_cast<volatile uint32_t*>(p);
    return s;
}

struct XRegs6 {
    float4 lo[kPrepBlocks], hi[kPrepBlocks];
};
// One warp per super-block; lane l handles the 8 consecutive elements 8l .. 8l+7.
// K: length of the (concatenated) activation. bpe > 0 (MoE down projection): the activation is n_slots
// vectors of bpe * 256 elements, x + s * x_stride, each scaled by the slot's routing weight wts[s].
// Only the n_need super-blocks from b_first on (wrapping at the end of the row) are converted: a CTA whose
// units cover less than a row does not need the rest.
__device__ __forceinline__ uint32_t prep_block(uint32_t i, uint32_t b_first, uint32_t nblk) {
    const uint32_t b = b_first + i;
    return b >= nblk ? b - nblk : b;
}
template <int kWarps>
__device__ __forceinline__ void load_x6(XRegs6& r, const float* __restrict__ x, uint32_t K, uint32_t bpe,
                                        uint32_t x_stride, const uint32_t* __restrict__ wts, int warp, int lane,
                                        uint32_t b_first, uint32_t n_need) {
#pragma unroll
    for (int b = 0; b < kPrepBlocks; ++b) {
        const uint32_t bi = warp + b * kWarps;
        if (bi < n_need) {
            const uint32_t blk = prep_block(bi, b_first, K >> 8);
            const uint32_t slot = bpe ? blk / bpe : 0u, lb = bpe ? blk - slot * bpe : blk;
            const float* xp = x + (size_t)slot * x_stride + (size_t)lb * 256 + 8 * lane;
            float4 lo = __ldg(reinterpret_cast<const float4*>(xp)), hi = __ldg(reinterpret_cast<const float4*>(xp) + 1);
            if (wts) {
                const float w = __uint_as_float(__ldg(wts + slot));
                lo = make_float4(lo.x * w, lo.y * w, lo.z * w, lo.w * w);
                hi = make_float4(hi.x * w, hi.y * w, hi.z * w, hi.w * w);
            }
            r.lo[b] = lo;
            r.hi[b] = hi;
        }
    }
}

__device__ __forceinline__ uint32_t pack4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// Lane l's elements 8l .. 8l+7 lie in half h = l/16, quarter j = (l/4)%4, sub-block half u = (l/2)%2, and are
// the k-slot groups t = 2(l%2) and t+1 of that sub-block half.
template <int kWarps>
__device__ __forceinline__ void prep_x6(const Smem6& s, const XRegs6& r, uint32_t K, int warp, int lane,
                                        uint32_t b_first, uint32_t n_need) {
    const uint32_t h = lane >> 4, j = (lane >> 2) & 3, u = (lane >> 1) & 1, t0 = 2 * (lane & 1);
#pragma unroll
    for (int b = 0; b < kPrepBlocks; ++b) {
        const uint32_t bi = warp + b * kWarps;
        if (bi >= n_need) break;
        const uint32_t blk = prep_block(bi, b_first, K >> 8);
        const float4 lo = r.lo[b], hi = r.hi[b];
        const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        float mx = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) mx = fmaxf(mx, fabsf(v[e]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        uint32_t E = (__float_as_uint(mx) >> 23) & 0xFFu;
        E = E < 32u ? 32u : E;
        const float scale = __uint_as_float((127u + 126u + kFracBits - E) << 23);
        int X[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) X[e] = __float2int_rn(v[e] * scale);
        uint32_t dw[3][2];
        int ds[3];
        dw[0][0] = pack4(X[0] >> 14, X[1] >> 14, X[2] >> 14, X[3] >> 14);
        dw[0][1] = pack4(X[4] >> 14, X[5] >> 14, X[6] >> 14, X[7] >> 14);
        dw[1][0] = pack4(X[0] >> 7, X[1] >> 7, X[2] >> 7, X[3] >> 7) & 0x7F7F7F7Fu;
        dw[1][1] = pack4(X[4] >> 7, X[5] >> 7, X[6] >> 7, X[7] >> 7) & 0x7F7F7F7Fu;
        dw[2][0] = pack4(X[0], X[1], X[2], X[3]) & 0x7F7F7F7Fu;
        dw[2][1] = pack4(X[4], X[5], X[6], X[7]) & 0x7F7F7F7Fu;
        ds[0] = ds[1] = ds[2] = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            ds[0] += X[e] >> 14;
            ds[1] += (X[e] >> 7) & 0x7F;
            ds[2] += X[e] & 0x7F;
        }
        uint8_t* bq = s.bq + (size_t)blk * kBBytes + h * 768 + (j >> 1) * 384 + (j & 1) * 8;
#pragma unroll
        for (int d = 0; d < 3; ++d) {
            uint8_t* dst = bq + (2 * d + u) * 64 + t0 * 16;
            // {b0, b1}: the digit word sits in the register that feeds the k slots of sub-block half u
            *reinterpret_cast<uint2*>(dst) = u ? make_uint2(0u, dw[d][0]) : make_uint2(dw[d][0], 0u);
            *reinterpret_cast<uint2*>(dst + 16) = u ? make_uint2(0u, dw[d][1]) : make_uint2(dw[d][1], 0u);
            const int sum = ds[d] + __shfl_xor_sync(0xFFFFFFFFu, ds[d], 1);
            if ((lane & 1) == 0) s.nsx[blk * 64 + h * 32 + d * 8 + j * 2 + u] = -32 * sum;
        }
        if ((lane & 1) == 0) s.nsx[blk * 64 + h * 32 + 24 + j * 2 + u] = 0;  // digit 3 does not exist: lane t = 3
        if (lane == 0) s.xs[blk] = __uint_as_float((E + 1u - kFracBits) << 23);
    }
}

__device__ __forceinline__ uint32_t lds_u32s(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16s(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}

// The 32-bit word at byte address saddr (2-byte aligned): one load when kFunnel is false (saddr is a multiple
// of 4), else the two words around it and a funnel shift by sh = 8 * (saddr % 4).
template <bool kFunnel>
__device__ __forceinline__ uint32_t lds_word(uint32_t saddr, uint32_t sh) {
    if constexpr (kFunnel) {
        const uint32_t base = saddr & ~3u;
        return __funnelshift_r(lds_u32s(base), lds_u32s(base + 4), sh);
    } else {
        return lds_u32s(saddr);
    }
}

// sign-extended byte n of w
template <int n>
__device__ __forceinline__ int sbyte(uint32_t w) {
    int r;  // prmt: selector nibble n takes byte n, 8 | n replicates that byte's sign bit
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "n"(n | ((8 | n) << 4) | ((8 | n) << 8) | ((8 | n) << 12)));
    return r;
}

// One super-block of rows g (at slot address rA) and g+8 (rB) against the B table at xb / accumulator start
// values at nb; returns sum_s sc_s * (D_t,s - 32 SB_t,s) for digit t = lane % 4 and both rows.
template <bool kFunnel>
__device__ __forceinline__ void block6(uint32_t rA, uint32_t rB, uint32_t shA, uint32_t shB, uint32_t xb, uint32_t xh,
                                       uint32_t nb, int t, int& IA, int& IB) {
    constexpr uint32_t kNib = 0x0F0F0F0Fu, kTop = 0x30303030u;
    IA = IB = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t vA[4][2], vB[4][2];  // [quarter j][sub-block half m]
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            const uint32_t o = 16 * m + 4 * t;
            const uint32_t la0 = lds_word<kFunnel>(rA + 64 * h + o, shA), la1 = lds_word<kFunnel>(rA + 64 * h + 32 + o, shA);
            const uint32_t ha = lds_word<kFunnel>(rA + 128 + 32 * h + o, shA);
            const uint32_t lb0 = lds_word<kFunnel>(rB + 64 * h + o, shB), lb1 = lds_word<kFunnel>(rB + 64 * h + 32 + o, shB);
            const uint32_t hb = lds_word<kFunnel>(rB + 128 + 32 * h + o, shB);
            vA[0][m] = (la0 & kNib) | ((ha << 4) & kTop);
            vA[1][m] = (la1 & kNib) | ((ha << 2) & kTop);
            vA[2][m] = ((la0 >> 4) & kNib) | (ha & kTop);
            vA[3][m] = ((la1 >> 4) & kNib) | ((ha >> 2) & kTop);
            vB[0][m] = (lb0 & kNib) | ((hb << 4) & kTop);
            vB[1][m] = (lb1 & kNib) | ((hb << 2) & kTop);
            vB[2][m] = ((lb0 >> 4) & kNib) | (hb & kTop);
            vB[3][m] = ((lb1 >> 4) & kNib) | ((hb >> 2) & kTop);
        }
        // int8 scales of the half's eight sub-blocks, rows g and g+8
        const uint32_t sA0 = lds_word<kFunnel>(rA + 192 + 8 * h, shA), sA1 = lds_word<kFunnel>(rA + 196 + 8 * h, shA);
        const uint32_t sB0 = lds_word<kFunnel>(rB + 192 + 8 * h, shB), sB1 = lds_word<kFunnel>(rB + 196 + 8 * h, shB);
        // {b0, b1} of quarters 0, 1 / 2, 3 (xh: 0 for the lanes of the dead columns, which read zeros at xb)
        const uint4 b01 = lds_v4(xb + (768 * h & xh)), b23 = lds_v4(xb + ((768 * h + 384) & xh));
        const uint4 n01 = lds_v4(nb + 128 * h), n23 = lds_v4(nb + 128 * h + 16);  // start values: (j, u) pairs
        int c0[4] = {(int)n01.x, (int)n01.y, (int)n01.x, (int)n01.y};
        int c1[4] = {(int)n01.z, (int)n01.w, (int)n01.z, (int)n01.w};
        int c2[4] = {(int)n23.x, (int)n23.y, (int)n23.x, (int)n23.y};
        int c3[4] = {(int)n23.z, (int)n23.w, (int)n23.z, (int)n23.w};
        mma_u8s8(c0, vA[0][0], vB[0][0], vA[0][1], vB[0][1], b01.x, b01.y);
        mma_u8s8(c1, vA[1][0], vB[1][0], vA[1][1], vB[1][1], b01.z, b01.w);
        mma_u8s8(c2, vA[2][0], vB[2][0], vA[2][1], vB[2][1], b23.x, b23.y);
        mma_u8s8(c3, vA[3][0], vB[3][0], vA[3][1], vB[3][1], b23.z, b23.w);
        // D columns 2t, 2t+1 = digit t of sub-blocks 8h + 2j, 8h + 2j + 1: scale bytes 2j, 2j+1 of the half
        IA += c0[0] * sbyte<0>(sA0) + c0[1] * sbyte<1>(sA0) + c1[0] * sbyte<2>(sA0) + c1[1] * sbyte<3>(sA0) +
              c2[0] * sbyte<0>(sA1) + c2[1] * sbyte<1>(sA1) + c3[0] * sbyte<2>(sA1) + c3[1] * sbyte<3>(sA1);
        IB += c0[2] * sbyte<0>(sB0) + c0[3] * sbyte<1>(sB0) + c1[2] * sbyte<2>(sB0) + c1[3] * sbyte<3>(sB0) +
              c2[2] * sbyte<0>(sB1) + c2[3] * sbyte<1>(sB1) + c3[2] * sbyte<2>(sB1) + c3[3] * sbyte<3>(sB1);
    }
}

// kMoe: MoE down projection, y += sum_s w_s W[routing[s]] x_s: the n_used selected matrices side by side along
// K, each with its own activation (scaled by w_s while it is converted to fixed point).
// kRowsAligned: every row starts on a 16-byte boundary (K a multiple of 2048), so all rows of a unit share
// one offset inside their aligned supersets; otherwise each row has its own (rows are 2-byte aligned).
template <int EPI, int kWarps, bool kRowsAligned, bool kMoe = false>
__global__ void __launch_bounds__(kWarps * 32, 16 / kWarps) dmmv_q6k_warp_kernel(const WarpArgs a,
                                                                                 const uint8_t* a_end) {
    extern __shared__ uint8_t smem_raw[];
    pdl_begin(a);
    const uint32_t bpe = a.K >> 8;                        // blocks per row of one matrix
    const uint32_t bpr = kMoe ? bpe * a.nseg : bpe;       // blocks per (concatenated) row = units per tile
    const Smem6 s = carve6(smem_raw, bpr * 256, kWarps);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint64_t row_bytes = (uint64_t)bpe * 210;
    // matrix that holds block `b` of the concatenated row, and the block's index inside it
    auto matrix_of = [&](uint32_t b, uint32_t& lb) -> const uint8_t* {
        if constexpr (kMoe) {
            const uint32_t slot = b / bpe;
            lb = b - slot * bpe;
            const uint32_t e_raw = __ldg(a.routing + slot);
            if (e_raw == kSkipExpert) return nullptr;  // no expert in this slot on this rank
            return expert_matrix(a.A[0], a.A_sh[0], e_raw, a.expert_stride, a.n_experts_max, a.status);
        } else {
            lb = b;
            return a.A[0];
        }
    };
    const uint32_t tiles = (a.M + 15) / 16;
    const uint32_t U = tiles * bpr, G = gridDim.x * kWarps;
    const uint32_t me = blockIdx.x * kWarps + warp;
    const uint32_t u0 = (uint32_t)part_begin(me, U, G), u1 = (uint32_t)part_begin(me + 1, U, G);
    const uint32_t n = u1 - u0;
    uint8_t* ring = s.ring + (size_t)warp * kRing6;

    uint32_t piece[kPiecesLane6];  // row | column << 8
#pragma unroll
    for (int i = 0; i < kPiecesLane6; ++i) {
        const uint32_t p = i * 32 + lane;
        const uint32_t r = p / kPieces6;
        piece[i] = r | ((p - r * kPieces6) << 8);
    }
    uint32_t p_tile = u0 / bpr, p_blk = u0 % bpr;
    // Rows aligned and a whole number of tiles: a piece's place in the slot and its offset from the tile's first
    // row are fixed per lane
    const bool whole_tiles = kRowsAligned && (a.M & 15u) == 0;
    uint32_t pdst[kPiecesLane6], psrc[kPiecesLane6];
    if constexpr (kRowsAligned) {
#pragma unroll
        for (int i = 0; i < kPiecesLane6; ++i) {
            const uint32_t r = piece[i] & 0xFFu, col = piece[i] >> 8;
            pdst[i] = r * kRow6 + col * 16;
            psrc[i] = r * (uint32_t)row_bytes + col * 16;
        }
    }
    const uint32_t ring_addr = smem_u32(ring);
    auto request = [&](uint32_t slot) {
        uint8_t* dst = ring + slot * kSlot6;
        const uint32_t row0 = p_tile * 16;
        if constexpr (kRowsAligned) {
            const uint32_t al = (p_blk * 210u) & ~15u;  // aligned start of the block's superset within the row
            if (whole_tiles) {
                const uint8_t* base = a.A[0] + (uint64_t)row0 * row_bytes + al;
                const uint32_t room = (uint32_t)row_bytes - al, ds = ring_addr + slot * kSlot6;
#pragma unroll
                for (int i = 0; i < kPiecesLane6; ++i)
                    if ((piece[i] >> 8) * 16 < room)  // rows are 16-byte aligned: a piece never crosses the row end
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ds + pdst[i]), "l"(base + psrc[i])
                                     : "memory");
            } else {
#pragma unroll
                for (int i = 0; i < kPiecesLane6; ++i) {
                    const uint32_t r = piece[i] & 0xFFu, col = piece[i] >> 8;
                    if (al + col * 16 < (uint32_t)row_bytes) {
                        const uint32_t row = min(row0 + r, a.M - 1);
                        cp_async16(dst + r * kRow6 + col * 16, a.A[0] + (uint64_t)row * row_bytes + al + col * 16);
                    }
                }
            }
        } else {
            uint32_t lb;
            const uint8_t* mat = matrix_of(p_blk, lb);
            // first byte past the buffer that holds `mat` (the shared expert lives in a buffer of its own)
            const uint8_t* m_end = kMoe && mat == a.A_sh[0] ? a.A_sh_end[0] : a_end;
#pragma unroll
            for (int i = 0; i < kPiecesLane6; ++i) {
                if (kMoe && mat == nullptr) break;  // nothing to fetch
                const uint32_t r = piece[i] & 0xFFu, col = piece[i] >> 8;
                const uint32_t row = min(row0 + r, a.M - 1);
                const uint8_t* start = mat + (uint64_t)row * row_bytes + lb * 210u;
                const uint32_t o = (uint32_t)(reinterpret_cast<uintptr_t>(start) & 15u);
                if (col * 16 < o + 210u) {  // the piece holds bytes of the block
                    const uint8_t* src = start - o + col * 16;
                    uint8_t* d = dst + r * kRow6 + col * 16;
                    if (src + 16 <= m_end) {
                        cp_async16(d, src);
                    } else {  // the very end of the tensor: copy only the bytes that exist
                        for (const uint8_t* q = src; q < m_end; ++q) d[q - src] = __ldg(q);
                    }
                }
            }
        }
        if (++p_blk == bpr) { p_blk = 0; ++p_tile; }
    };
    // super-blocks of the activation this CTA's units touch
    const uint32_t cu0 = (uint32_t)part_begin((uint64_t)blockIdx.x * kWarps, U, G);
    const uint32_t cu1 = (uint32_t)part_begin((uint64_t)(blockIdx.x + 1) * kWarps, U, G);
    const uint32_t x_first = cu1 - cu0 >= bpr ? 0u : cu0 % bpr, x_need = min(bpr, cu1 - cu0);
    pdl_late(a);
    XRegs6 xr;
    if (a.late)
        load_x6<kWarps>(xr, a.x, bpr * 256, kMoe ? bpe : 0u, kMoe ? a.x_slot_stride : 0u,
                        kMoe ? a.routing + a.nseg : nullptr, warp, lane, x_first, x_need);
#pragma unroll
    for (int i = 0; i < kDepth; ++i) {
        if ((uint32_t)i < n) request(i);
        cp_async_commit();
    }
    pdl_wait();
    if (!a.late)
        load_x6<kWarps>(xr, a.x, bpr * 256, kMoe ? bpe : 0u, kMoe ? a.x_slot_stride : 0u,
                        kMoe ? a.routing + a.nseg : nullptr, warp, lane, x_first, x_need);
    if (a.consume.n) consume_pushed(a.consume, blockIdx.x, gridDim.x, tid, kWarps * 32);

    if (tid < kZeroBytes6 / 16) reinterpret_cast<uint4*>(s.zeros)[tid] = make_uint4(0u, 0u, 0u, 0u);
    if (tid < kWarps) s.sflags[tid] = 0u;
    prep_x6<kWarps>(s, xr, bpr * 256, warp, lane, x_first, x_need);
    __syncthreads();

    uint32_t tile = u0 / bpr, blk = u0 % bpr;
    float acc[2] = {0.f, 0.f};
    // B operand: lane (g, t) feeds column g; columns 6 and 7 are dead (zeros, one address for the quarter-warp)
    const bool b_live = g < 6;
    const uint32_t xb_base = b_live ? smem_u32(s.bq) + (uint32_t)g * 64u + (uint32_t)t * 16u : smem_u32(s.zeros);
    const uint32_t xb_step = b_live ? (uint32_t)kBBytes : 0u;
    const uint32_t xh = b_live ? 0xFFFFFFFFu : 0u;
    const uint32_t nsx_s = smem_u32(s.nsx) + 32u * t, xs_s = smem_u32(s.xs), ring_s = smem_u32(ring);
    const float dscale = __uint_as_float((127u + 14u - 7u * t) << 23);  // digit t carries 2^(14 - 7t)

    for (uint32_t it = 0; it < n; ++it) {
        const uint32_t slot = it % kDepth;
        cp_async_wait<kDepth - 1>();
        __syncwarp();
        // byte offset of the block inside each row's aligned superset
        uint32_t oA, oB;
        bool skip = false;  // MoE: the block belongs to a slot without an expert on this rank
        if constexpr (kRowsAligned) {
            oA = oB = (blk * 210u) & 15u;
        } else {
            const uint32_t rowA = min(tile * 16 + g, a.M - 1), rowB = min(tile * 16 + g + 8, a.M - 1);
            uint32_t lb;
            const uint8_t* mat = matrix_of(blk, lb);
            skip = kMoe && mat == nullptr;
            oA = (uint32_t)(reinterpret_cast<uintptr_t>(mat + (uint64_t)rowA * row_bytes + lb * 210u) & 15u);
            oB = (uint32_t)(reinterpret_cast<uintptr_t>(mat + (uint64_t)rowB * row_bytes + lb * 210u) & 15u);
        }
        const uint32_t sb = ring_s + slot * kSlot6;
        const uint32_t rA = sb + g * kRow6 + oA, rB = sb + (g + 8) * kRow6 + oB;
        const uint32_t xb = xb_base + blk * xb_step, nb = nsx_s + blk * (uint32_t)kNsxBytes;
        int IA = 0, IB = 0;
        uint32_t dA = 0, dB = 0;
        if (skip) {
        } else if (kRowsAligned && (oA & 2u) == 0) {  // the same for the whole warp
            block6<false>(rA, rB, 0u, 0u, xb, xh, nb, t, IA, IB);
        } else {
            block6<true>(rA, rB, (oA & 3u) * 8u, (oB & 3u) * 8u, xb, xh, nb, t, IA, IB);
        }
        if (!skip) {
            dA = lds_u16s(rA + 208);
            dB = lds_u16s(rB + 208);
        }
        // every lane has read the stage: refill it
        __syncwarp();
        if (it + kDepth < n) request(slot);
        cp_async_commit();
        const float xs = lds_f1(xs_s + blk * 4);
        acc[0] = fmaf(h2f(dA) * xs, (float)IA, acc[0]);
        acc[1] = fmaf(h2f(dB) * xs, (float)IB, acc[1]);

        const uint32_t T = tile;
        bool tile_done = false;
        if (++blk == bpr) { blk = 0; ++tile; tile_done = true; }
        if (tile_done || it + 1 == n) {
            float v[1][2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float w = acc[r] * dscale;
                w += __shfl_xor_sync(0xFFFFFFFFu, w, 1);
                w += __shfl_xor_sync(0xFFFFFFFFu, w, 2);
                v[0][r] = w;
                acc[r] = 0.f;
            }
            finish_tile<1, EPI, kWarps>(a, row_out(a), s.spartial, s.sflags, v, T, bpr, u0, u1, U, G, me, warp, lane);
        }
    }
}

template <int EPI, int kWarps, bool kRowsAligned, bool kMoe = false>
cudaError_t launch_w6(const WarpArgs& a, const uint8_t* a_end, cudaStream_t st, int sm_count, size_t smem) {
    auto kern = dmmv_q6k_warp_kernel<EPI, kWarps, kRowsAligned, kMoe>;
    static std::atomic<uint64_t> attr_done{0};  // per device ordinal
    if (cudaError_t ea = ensure_dynamic_smem(kern, kWarps == 8 ? (int)kTwoPerSm : 227 * 1024, attr_done); ea != cudaSuccess) return ea;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * (a.K >> 8) * (kMoe ? a.nseg : 1u);
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
    return cudaLaunchKernelEx(&cfg, kern, a, a_end);
}

template <int EPI>
cudaError_t launch_cfg6(const WarpArgs& a, const uint8_t* a_end, cudaStream_t st, int sm_count) {
    const size_t s8 = smem_bytes6(a.K, 8);
    const bool al = ((a.K >> 8) % 8u) == 0;  // 210 * K/256 bytes per row: a multiple of 16 for K % 2048 == 0
    if (s8 <= kTwoPerSm)
        return al ? launch_w6<EPI, 8, true>(a, a_end, st, sm_count, s8) : launch_w6<EPI, 8, false>(a, a_end, st, sm_count, s8);
    const size_t s16 = smem_bytes6(a.K, 16);
    return al ? launch_w6<EPI, 16, true>(a, a_end, st, sm_count, s16) : launch_w6<EPI, 16, false>(a, a_end, st, sm_count, s16);
}

}  // namespace

bool q6k_dmmv_eligible(uint32_t type, int mode, const DmmvArgs& a) {
    if (type != T_Q6_K) return false;
    if (mode != MODE_PLAIN && mode != MODE_SIGMOID_ACC) return false;
    if (!a.scratch_partial || !a.status) return false;
    const uint32_t bpr = a.K >> 8;
    if (reinterpret_cast<uintptr_t>(a.A) & 15u) return false;  // supersets are fetched in 16-byte pieces from the base
    if ((bpr % 8u) != 0 && !a.a_end) return false;          // unaligned rows: the end of the buffer must be known
    if (smem_bytes6(a.K, 16) > 227 * 1024 || bpr > (uint32_t)(kPrepBlocks * 8)) return false;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * bpr;
    if (U < 16 || U > 0xFFFFFFFFull) return false;
    return true;
}

// MoE down projection + weighted accumulate (y += sum_s w_s W[routing[s]] x_s) through the streaming kernel.
bool q6k_moe_down_acc_eligible(uint32_t type, const DmmvArgs& a) {
    if (type != T_Q6_K || !a.routing || a.n_used == 0 || !a.a_end) return false;
    if (!a.scratch_partial || !a.status) return false;
    if ((reinterpret_cast<uintptr_t>(a.A) & 15u) || (a.expert_stride & 15u) || (a.K & 255u)) return false;
    if ((a.x_expert_stride & 3u) || (reinterpret_cast<uintptr_t>(a.x) & 15u)) return false;
    if (a.A_sh && ((reinterpret_cast<uintptr_t>(a.A_sh) & 15u) || !a.a_sh_end)) return false;
    const uint32_t bpr = (a.K >> 8) * a.n_used;
    if (smem_bytes6(bpr * 256, 16) > 227 * 1024 || bpr > (uint32_t)(kPrepBlocks * 8)) return false;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * bpr;
    if ((uint64_t)a.M * bpr * 210u < kStreamMinBytes) return false;  // small expert sets: latency-bound either way
    return U >= 16 && U <= 0xFFFFFFFFull;
}

cudaError_t launch_q6k_moe_down_acc(const DmmvArgs& a, cudaStream_t st, uint64_t* launches) {
    WarpArgs wa;
    wa.A[0] = wa.A[1] = a.A;
    wa.x = a.x;
    wa.y = a.y;
    wa.gate = nullptr;
    wa.M = a.M;
    wa.K = a.K;
    wa.acc_mode = 1;
    wa.gpartial = a.scratch_partial;
    wa.status = a.status;
    wa.spin_limit = a.spin_limit;
    wa.nseg = a.n_used;
    wa.routing = a.routing;
    wa.n_experts_max = a.n_experts_max;
    wa.expert_stride = a.expert_stride;
    wa.x_slot_stride = a.x_expert_stride;
    wa.A_sh[0] = wa.A_sh[1] = a.A_sh;
    wa.A_sh_end[0] = wa.A_sh_end[1] = a.a_sh_end;
    wa.bias[0] = a.bias;
    wa.late = a.late;
    const uint32_t Kt = a.K * a.n_used;
    const size_t s8 = smem_bytes6(Kt, 8);
    const cudaError_t e = s8 <= kTwoPerSm ? launch_w6<EPI_ACC, 8, false, true>(wa, a.a_end, st, a.sm_count, s8)
                                          : launch_w6<EPI_ACC, 16, false, true>(wa, a.a_end, st, a.sm_count,
                                                                                 smem_bytes6(Kt, 16));
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

cudaError_t launch_q6k_dmmv(int mode, const DmmvArgs& a, cudaStream_t st, uint64_t* launches) {
    WarpArgs wa;
    wa.A[0] = a.A;
    wa.A[1] = a.A;
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
    cudaError_t e = mode == MODE_PLAIN ? launch_cfg6<EPI_PLAIN>(wa, a.a_end, st, a.sm_count)
                                       : launch_cfg6<EPI_SIGMOID_ACC>(wa, a.a_end, st, a.sm_count);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
