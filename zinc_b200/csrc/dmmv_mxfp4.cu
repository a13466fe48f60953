// Warp-autonomous streaming decode matvec for MXFP4 weights (17-byte blocks: E8M0 scale + 32 E2M1
// nibbles), same structure as the Q4_K kernel: contiguous unit ranges per warp, coalesced 16-byte
// cp.async prefetch into per-warp rings, activations in 21-bit fixed point split into three 7-bit
// digits, int8 tensor-core dot products with exact s32 accumulation, split-K hand-off between
// workers. What differs:
//   * rows are only 2-byte aligned (17 * K/32 bytes), so a unit's row segment (16 blocks = 272 bytes)
//     is fetched as the 16-byte-aligned superset that contains it (18 pieces) and read back from
//     shared memory at the row's own byte offset with funnel shifts;
//   * a weight is 2 * E2M1 as a signed byte {0, +-1, +-2, +-3, +-4, +-6, +-8, +-12}: two 8-entry byte
//     tables (positive / negative) looked up four nibbles at a time with byte permutes and selected
//     by a sign mask that a sign-replicating permute builds; exact, the 0.5 is folded into the scale;
//   * lane (g, t) owns block 4q + t of each group of four blocks for rows g and g + 8; its k slots
//     carry that block's elements (block-diagonal B operand), one MMA pair per eight elements;
//   * the block scale 2^(e - 127) is applied per lane after the four MMA steps of a block.
//
// Stands in for the reference's dmmv_mxfp4.comp and its MoE forms (src/shaders/dmmv_mxfp4.comp,
// dmmv_mxfp4_moe*.comp) for the block layout of src/compute/forward.zig:431-465.
#include "kernels.h"
#include "stream_skel.cuh"

namespace zc {

namespace {

constexpr int kDepthX = 2;                   // units in flight per warp
constexpr int kUnitBlocks = 16;              // blocks per row segment: 272 bytes, 512 weights
constexpr int kSegBytes = kUnitBlocks * 17;  // 272
constexpr int kRowSlot = 304;                // 288-byte aligned superset + 16: rows 16 B apart mod 32 B
constexpr int kSlotBytesX = 16 * kRowSlot;
constexpr int kRingX = kDepthX * kSlotBytesX;
constexpr int kPiecesRow = 18;
constexpr int kPiecesLane = 16 * kPiecesRow / 32;  // 9
constexpr size_t kTwoPerSmX = 113 * 1024;
constexpr int kZeroUnitsX = 72;
constexpr int kFracBitsX = 20;
constexpr int kPrepX = 6;                    // 256-element chunks of x per warp: K <= 6 * kWarps * 256

struct SmemX {
    uint4* xf;       // x digits in B-operand order: unit ((q*4 + j)*2 + p)*4 + t, q = group of four blocks
    uint4* zeros;
    float* xs;       // per 256 elements: 2^-f * 0.5
    uint8_t* ring;
    float* spartial;
    volatile uint32_t* sflags;
};

__host__ __device__ inline uint32_t k_padded(uint32_t K) { return (K + 255u) & ~255u; }

__host__ __device__ inline size_t smem_bytes_x(uint32_t Kp, int kWarps) {  // Kp: padded length of the activation
    size_t n = (size_t)Kp * 4 + (size_t)kZeroUnitsX * 16 + (size_t)(Kp / 256) * 4;
    n = (n + 127) & ~size_t(127);
    n += (size_t)kWarps * kRingX + 64;  // ring (+ slack: the last row's reads may run a few bytes past its slot)
    n += (size_t)kWarps * 32 * 4 + (size_t)kWarps * 4 + 16;
    return n + 128;
}

__device__ inline SmemX carve_x(uint8_t* base, uint32_t Kp, int kWarps) {
    SmemX s;
    uintptr_t p = (reinterpret_cast<uintptr_t>(base) + 127) & ~uintptr_t(127);
    s.xf = reinterpret_cast<uint4*>(p);
    p += (size_t)Kp * 4;
    s.zeros = reinterpret_cast<uint4*>(p);
    p += (size_t)kZeroUnitsX * 16;
    s.xs = reinterpret_cast<float*>(p);
    p += (size_t)(Kp / 256) * 4;
    p = (p + 127) & ~uintptr_t(127);
    s.ring = reinterpret_cast<uint8_t*>(p);
    p += (size_t)kWarps * kRingX + 64;
    s.spartial = reinterpret_cast<float*>(p);
    p += (size_t)kWarps * 32 * 4;
    s.sflags = reinterpret_cast<volatile uint32_t*>(p);
    return s;
}

// x -> digits. One warp per 256 elements (two groups of four blocks); lane = qq*16 + t*4 + j handles, for
// block (2*chunk + qq)*4 + t, the eight elements of MMA step j: e[4j..4j+3] and e[16+4j..16+4j+3].
// Byte order inside the B registers follows the weight conversion: b0 = (e[4j], e[16+4j], e[4j+1],
// e[17+4j]), b1 = (e[4j+2], e[18+4j], e[4j+3], e[19+4j]). Elements at or beyond K read as zero.
struct XRegsX {
    float4 lo[kPrepX], hi[kPrepX];
};
// n_slots > 1 (MoE down projection): the activation is the concatenation of n_slots vectors of K
// elements, x + s * x_stride, each padded to whole 256-element chunks and scaled by the slot's routing
// weight wts[s] (f32 bits), so that sum_s w_s * W_s x_s becomes one long dot product.
template <int kWarps>
__device__ __forceinline__ void load_x_x(XRegsX& r, const float* __restrict__ x, uint32_t K, uint32_t n_slots,
                                         uint32_t x_stride, const uint32_t* __restrict__ wts, int warp, int lane) {
    const int qq = lane >> 4, t = (lane >> 2) & 3, j = lane & 3;
    const uint32_t cps = k_padded(K) / 256;  // chunks per slot
#pragma unroll
    for (int i = 0; i < kPrepX; ++i) {
        const uint32_t chunk = warp + i * kWarps;
        const uint32_t slot = chunk / cps, lc = chunk - slot * cps;
        const uint32_t e0 = lc * 256 + (qq * 4 + t) * 32 + 4 * j;
        float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
        if (slot < n_slots) {
            const float* xs = x + (size_t)slot * x_stride;
            const float w = wts ? __uint_as_float(__ldg(wts + slot)) : 1.0f;
            if (e0 + 4 <= K) {
                lo = __ldg(reinterpret_cast<const float4*>(xs + e0));
                lo = make_float4(lo.x * w, lo.y * w, lo.z * w, lo.w * w);
            }
            if (e0 + 20 <= K) {
                hi = __ldg(reinterpret_cast<const float4*>(xs + e0 + 16));
                hi = make_float4(hi.x * w, hi.y * w, hi.z * w, hi.w * w);
            }
        }
        r.lo[i] = lo;
        r.hi[i] = hi;
    }
}
template <int kWarps>
__device__ __forceinline__ void prep_x_x(const SmemX& s, const XRegsX& r, uint32_t Kp_total, int warp, int lane) {
    const int qq = lane >> 4, t = (lane >> 2) & 3, j = lane & 3;
#pragma unroll
    for (int i = 0; i < kPrepX; ++i) {
        const uint32_t chunk = warp + i * kWarps;
        if (chunk * 256 >= Kp_total) break;
        const float4 lo = r.lo[i], hi = r.hi[i];
        // order of the eight bytes: b0 = (lo.x, hi.x, lo.y, hi.y), b1 = (lo.z, hi.z, lo.w, hi.w)
        const float v[8] = {lo.x, hi.x, lo.y, hi.y, lo.z, hi.z, lo.w, hi.w};
        float mx = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) mx = fmaxf(mx, fabsf(v[e]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        uint32_t E = (__float_as_uint(mx) >> 23) & 0xFFu;
        E = E < 32u ? 32u : E;
        const float scale = __uint_as_float((127u + 126u + kFracBitsX - E) << 23);
        uint32_t d0[2] = {0, 0}, d1[2] = {0, 0}, d2[2] = {0, 0};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int X = __float2int_rn(v[e] * scale);
            d0[e >> 2] |= (uint32_t)((X >> 14) & 0xFF) << (8 * (e & 3));
            d1[e >> 2] |= (uint32_t)((X >> 7) & 0x7F) << (8 * (e & 3));
            d2[e >> 2] |= (uint32_t)(X & 0x7F) << (8 * (e & 3));
        }
        const uint32_t q = chunk * 2 + qq;
        const uint32_t u = (q * 4 + j) * 2;
        s.xf[(u + 0) * 4 + t] = make_uint4(d0[0], d0[1], d2[0], d2[1]);
        s.xf[(u + 1) * 4 + t] = make_uint4(d1[0], d1[1], 0u, 0u);
        // 2^-f, times the 0.5 of "weights are stored as 2 * E2M1"
        if (lane == 0) s.xs[chunk] = __uint_as_float((E - kFracBitsX) << 23);
    }
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ uint4 lds_u128(uint32_t saddr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
    return v;
}

// Eight nibbles of q -> signed bytes 2 * E2M1: lo from nibbles 0..3, hi from nibbles 4..7 (eleven operations for
// eight weights; the selector of a byte permute is its low 16 bits, so the low half needs no extraction).
__device__ __forceinline__ void e2m1x8_to_s8(uint32_t q, uint32_t& lo, uint32_t& hi) {
    const uint32_t sel = q & 0x77777777u, sel_hi = sel >> 16;
    const uint32_t pos_lo = __byte_perm(0x03020100u, 0x0C080604u, sel);
    const uint32_t neg_lo = __byte_perm(0xFDFEFF00u, 0xF4F8FAFCu, sel);
    const uint32_t pos_hi = __byte_perm(0x03020100u, 0x0C080604u, sel_hi);
    const uint32_t neg_hi = __byte_perm(0xFDFEFF00u, 0xF4F8FAFCu, sel_hi);
    // byte i = 0xFF when nibble i (i + 4) has bit 3 set: selector bit 3 replicates the top bit of the selected byte
    const uint32_t q4 = q << 4;
    uint32_t m_lo, m_hi;
    asm("prmt.b32 %0, %1, %2, 0xD9C8;" : "=r"(m_lo) : "r"(q4), "r"(q));
    asm("prmt.b32 %0, %1, %2, 0xFBEA;" : "=r"(m_hi) : "r"(q4), "r"(q));
    asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(lo) : "r"(m_lo), "r"(neg_lo), "r"(pos_lo));
    asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(hi) : "r"(m_hi), "r"(neg_hi), "r"(pos_hi));
}

// kSeg: 0 one matrix (pair); 2 MoE slots resolved through the routing buffer, one output block per slot, x shared;
// 3 MoE down projection: the slots' matrices side by side along K, each with its own activation and
// routing weight, summed into one output (y += sum_s w_s W_s x_s)
template <int NS, int EPI, int kWarps, int kSeg>
__global__ void __launch_bounds__(kWarps * 32, 16 / kWarps) dmmv_mxfp4_warp_kernel(const WarpArgs a,
                                                                                   const uint8_t* a_end0,
                                                                                   const uint8_t* a_end1) {
    extern __shared__ uint8_t smem_raw[];
    pdl_begin(a);
    const uint32_t n_str = kSeg == 3 ? a.nseg : (uint32_t)NS;      // (matrix, activation range) streams per tile
    const uint32_t Kp_total = k_padded(a.K) * (kSeg == 3 ? a.nseg : 1u);
    const SmemX s = carve_x(smem_raw, Kp_total, kWarps);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t nb = a.K >> 5;                                // blocks per row
    const uint32_t row_bytes = nb * 17u;
    const uint32_t upt = (nb + kUnitBlocks - 1) / kUnitBlocks;  // units per row
    const uint32_t upt_all = upt * n_str;
    const uint32_t tpe = (a.M + 15) / 16;
    const uint32_t tiles = kSeg == 2 ? a.nseg * a.tiles_per_expert : tpe;
    const uint32_t U = tiles * upt_all, G = gridDim.x * kWarps;
    const uint32_t me = blockIdx.x * kWarps + warp;
    const uint32_t u0 = (uint32_t)part_begin(me, U, G), u1 = (uint32_t)part_begin(me + 1, U, G);
    const uint32_t n = u1 - u0;
    uint8_t* ring = s.ring + (size_t)warp * kRingX;

    // Matrix base, row bound for tile T in the indexing "row = T * 16 + r", and the first byte past the buffer
    // that holds the matrix. False: the slot names no expert on this rank (nothing to read, zeros contributed).
    auto locate = [&](uint32_t T, uint32_t strm, const uint8_t*& base, uint32_t& Mb, const uint8_t*& end) -> bool {
        if constexpr (kSeg == 2) {
            const uint32_t slot = T / a.tiles_per_expert, t0 = slot * a.tiles_per_expert * 16;
            const uint32_t e_raw = __ldg(a.routing + slot);
            if (e_raw == kSkipExpert) return false;
            const uint8_t* m = expert_matrix(a.A[strm], a.A_sh[strm], e_raw, a.expert_stride, a.n_experts_max, a.status);
            end = m == a.A_sh[strm] ? a.A_sh_end[strm] : (strm == 0 ? a_end0 : a_end1);
            base = m - (uint64_t)t0 * row_bytes;
            Mb = t0 + a.M;
            return true;
        } else if constexpr (kSeg == 3) {
            const uint32_t e_raw = __ldg(a.routing + strm);
            if (e_raw == kSkipExpert) return false;
            base = expert_matrix(a.A[0], a.A_sh[0], e_raw, a.expert_stride, a.n_experts_max, a.status);
            end = base == a.A_sh[0] ? a.A_sh_end[0] : a_end0;
            Mb = a.M;
            return true;
        } else {
            base = a.A[strm];
            end = strm == 0 ? a_end0 : a_end1;
            Mb = a.M;
            return true;
        }
    };

    uint32_t p_tile = u0 / upt_all, p_strm = (u0 % upt_all) / upt, p_kc = (u0 % upt_all) % upt;
    // per-lane constants of its nine pieces: row r, 16-byte column c, r * row_bytes + c * 16, and the row's
    // contribution to the byte offset inside the aligned superset (the unit start, and 272-byte steps
    // along K, add the same amount to every row)
    uint32_t pc_rc[kPiecesLane], pc_off[kPiecesLane];
#pragma unroll
    for (int i = 0; i < kPiecesLane; ++i) {
        const uint32_t p = i * 32 + lane;
        const uint32_t r = p / kPiecesRow, c = p - r * kPiecesRow;
        pc_rc[i] = r | (c << 8) | (((r * row_bytes) & 15u) << 16);
        pc_off[i] = r * row_bytes + c * 16;
    }
    auto request = [&](uint32_t slot) {
        const uint8_t* base = nullptr;
        const uint8_t* a_end = nullptr;  // first byte past this stream's weight buffer
        uint32_t Mb = 0;
        if (!locate(p_tile, p_strm, base, Mb, a_end)) {
            if (++p_kc == upt) {
                p_kc = 0;
                if (++p_strm == n_str) { p_strm = 0; ++p_tile; }
            }
            return;
        }
        const uint32_t seg = min((uint32_t)kUnitBlocks, nb - p_kc * kUnitBlocks) * 17u;  // bytes of this segment
        const uint32_t row0 = p_tile * 16;
        uint8_t* dst = ring + slot * kSlotBytesX;
        const uint8_t* ubase = base + (uint64_t)row0 * row_bytes + (uint64_t)p_kc * kSegBytes;  // row 0 of the unit
        if (row0 + 16 <= Mb && ubase + 16 * row_bytes + 32 <= a_end) {
            // whole tile inside the matrix and away from the end of the buffer
            const uint32_t tb = (uint32_t)(reinterpret_cast<uintptr_t>(ubase) & 15u);
#pragma unroll
            for (int i = 0; i < kPiecesLane; ++i) {
                const uint32_t c16 = (pc_rc[i] >> 4) & 0xFF0u;           // c * 16
                const uint32_t o = (tb + (pc_rc[i] >> 16)) & 15u;        // this row's offset in its superset
                if (c16 < o + seg)
                    cp_async16(dst + (pc_rc[i] & 0xFFu) * kRowSlot + c16, ubase + pc_off[i] - o);
            }
        } else {
#pragma unroll 1
            for (int i = 0; i < kPiecesLane; ++i) {
                const uint32_t p = i * 32 + lane;
                const uint32_t r = p / kPiecesRow, c = p - r * kPiecesRow;
                const uint32_t row = min(row0 + r, Mb - 1);
                const uint8_t* start = base + (uint64_t)row * row_bytes + (uint64_t)p_kc * kSegBytes;
                const uint32_t o = (uint32_t)(reinterpret_cast<uintptr_t>(start) & 15u);
                if (c * 16 < o + seg) {  // the piece holds bytes of the segment
                    const uint8_t* src = start - o + c * 16;
                    uint8_t* d = dst + r * kRowSlot + c * 16;
                    if (src + 16 <= a_end) {
                        cp_async16(d, src);
                    } else {  // the very end of the tensor: copy only the bytes that exist
                        for (const uint8_t* q = src; q < a_end; ++q) d[q - src] = __ldg(q);
                    }
                }
            }
        }
        if (++p_kc == upt) {
            p_kc = 0;
            if (++p_strm == n_str) { p_strm = 0; ++p_tile; }
        }
    };
    pdl_late(a);
    if (n) request(0);
    cp_async_commit();
    pdl_wait();
    XRegsX xr;
    load_x_x<kWarps>(xr, a.x, a.K, kSeg == 3 ? a.nseg : 1u, kSeg == 3 ? a.x_slot_stride : 0u,
                     kSeg == 3 ? a.routing + a.nseg : nullptr, warp, lane);
#pragma unroll
    for (int i = 1; i < kDepthX; ++i) {
        if ((uint32_t)i < n) request(i);
        cp_async_commit();
    }
    if (tid < kZeroUnitsX) s.zeros[tid] = make_uint4(0u, 0u, 0u, 0u);
    if (tid < kWarps) s.sflags[tid] = 0u;
    prep_x_x<kWarps>(s, xr, Kp_total, warp, lane);
    __syncthreads();

    uint32_t tile = u0 / upt_all, strm = (u0 % upt_all) / upt, kc = (u0 % upt_all) % upt;
    float acc0[2] = {0.f, 0.f}, acc1[2] = {0.f, 0.f};
    const bool b_live = (g >> 1) == t;
    const uint32_t xu_live = smem_u32(s.xf + (g & 1) * 4 + t);
    const uint32_t xu_dead = smem_u32(s.zeros + (g >> 1) + 1);
    const uint32_t ring_s = smem_u32(ring);

    for (uint32_t it = 0; it < n; ++it) {
        const uint32_t slot = it % kDepthX;
        cp_async_wait<kDepthX - 1>();
        __syncwarp();
        // byte offsets of this lane's two rows inside their row slots
        const uint8_t* base = a.A[0];  // (a slot without an expert: addresses formed below are never used)
        const uint8_t* unused_end;
        uint32_t Mb = 1;
        const bool live = locate(tile, strm, base, Mb, unused_end);
        const uint32_t rA = min(tile * 16 + g, Mb - 1), rB = min(tile * 16 + g + 8, Mb - 1);
        const uint32_t oA = (uint32_t)(reinterpret_cast<uintptr_t>(base + (uint64_t)rA * row_bytes + (uint64_t)kc * kSegBytes) & 15u);
        const uint32_t oB = (uint32_t)(reinterpret_cast<uintptr_t>(base + (uint64_t)rB * row_bytes + (uint64_t)kc * kSegBytes) & 15u);
        // shared-window byte addresses of the two rows' segments
        const uint32_t sA = ring_s + slot * kSlotBytesX + g * kRowSlot + oA;
        const uint32_t sB = ring_s + slot * kSlotBytesX + (g + 8) * kRowSlot + oB;
        const uint32_t nblk = live ? min((uint32_t)kUnitBlocks, nb - kc * kUnitBlocks) : 0u;
#pragma unroll 1
        for (uint32_t gq = 0; gq * 4 < nblk; ++gq) {
            const uint32_t bl = gq * 4 + t;              // this lane's block inside the unit
            // group of four blocks along the (concatenated) activation
            const uint32_t q = (kSeg == 3 ? strm * (k_padded(a.K) / 128) : 0u) + kc * (kUnitBlocks / 4) + gq;
            // 17 bytes per row at an arbitrary byte offset o (0..3) inside five aligned words: the scale is byte o,
            // nibble word i is bytes o + 1 + 4 i .. of them: one funnel shift by 8 (o + 1) bits (a shift of 32
            // hands back the upper word)
            uint32_t wa[5], wb[5];
            const uint32_t pa = sA + bl * 17, pb = sB + bl * 17;
            const uint32_t sha = (pa & 3u) * 8u + 8u, shb = (pb & 3u) * 8u + 8u;
#pragma unroll
            for (int i = 0; i < 5; ++i) {
                wa[i] = lds_u32((pa & ~3u) + 4 * i);
                wb[i] = lds_u32((pb & ~3u) + 4 * i);
            }
            const uint32_t xu = b_live ? xu_live + q * 512u : xu_dead;  // 32 units of 16 bytes per group
            int d01[4] = {0, 0, 0, 0}, d2[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t qa = __funnelshift_rc(wa[j], wa[j + 1], sha), qb = __funnelshift_rc(wb[j], wb[j + 1], shb);
                uint32_t a0, a1, a2, a3;
                e2m1x8_to_s8(qa, a0, a2);
                e2m1x8_to_s8(qb, a1, a3);
                const uint4 bx = lds_u128(xu + j * 128);
                mma_s8(d01, a0, a1, a2, a3, bx.x, bx.y);
                mma_s8(d2, a0, a1, a2, a3, bx.z, bx.w);
            }
            if (bl < nblk) {  // blocks past the row end hold stale bytes: their scale must not be used
                const float PA = (float)(d01[0] * 16384 + d01[1] * 128 + d2[0]);
                const float PB = (float)(d01[2] * 16384 + d01[3] * 128 + d2[2]);
                const float xs = s.xs[q >> 1];
                const uint32_t ea = (wa[0] >> (sha - 8u)) & 0xFFu, eb = (wb[0] >> (shb - 8u)) & 0xFFu;
                const float da = __uint_as_float(ea ? ea << 23 : 0x00400000u) * xs;
                const float db = __uint_as_float(eb ? eb << 23 : 0x00400000u) * xs;
                if (NS == 1 || strm == 0) { acc0[0] = fmaf(da, PA, acc0[0]); acc0[1] = fmaf(db, PB, acc0[1]); }  // NS == 1: every stream sums into acc0
                else { acc1[0] = fmaf(da, PA, acc1[0]); acc1[1] = fmaf(db, PB, acc1[1]); }
            }
        }
        __syncwarp();
        if (it + kDepthX < n) request(slot);
        cp_async_commit();
        const uint32_t T = tile;
        bool tile_done = false;
        if (++kc == upt) {
            kc = 0;
            if (++strm == n_str) { strm = 0; ++tile; tile_done = true; }
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
                const uint32_t slot_e = T / a.tiles_per_expert, t0 = slot_e * a.tiles_per_expert * 16;
                RowOut o{a.y + (size_t)slot_e * a.M - t0, a.y2 + (size_t)slot_e * a.M - t0, t0 + a.M, nullptr, nullptr};
                if (a.bias[0]) {  // the slot's expert's rows of the bias tables (none for a shared or absent expert)
                    const uint32_t e = __ldg(a.routing + slot_e);
                    if (e < a.n_experts_max) {
                        o.b0 = a.bias[0] + (size_t)e * a.M - t0;
                        o.b1 = a.bias[1] ? a.bias[1] + (size_t)e * a.M - t0 : nullptr;
                    }
                }
                finish_tile<NS, EPI, kWarps>(a, o, s.spartial, s.sflags, v, T, upt_all, u0, u1, U, G, me, warp, lane);
            } else {
                finish_tile<NS, EPI, kWarps>(a, row_out(a), s.spartial, s.sflags, v, T, upt_all, u0, u1, U, G, me, warp, lane);
            }
        }
    }
}

template <int NS, int EPI, int kWarps, int kSeg>
cudaError_t launch_x(const WarpArgs& a, const uint8_t* a_end, const uint8_t* a_end2, cudaStream_t st, int sm_count,
                     size_t smem) {
    auto kern = dmmv_mxfp4_warp_kernel<NS, EPI, kWarps, kSeg>;
    static std::atomic<uint64_t> attr_done{0};  // per device ordinal
    if (cudaError_t ea = ensure_dynamic_smem(kern, kWarps == 8 ? (int)kTwoPerSmX : 227 * 1024, attr_done); ea != cudaSuccess) return ea;
    const uint32_t nb = a.K >> 5;
    const uint64_t tiles = kSeg == 2 ? (uint64_t)a.nseg * a.tiles_per_expert : (a.M + 15) / 16;
    const uint64_t U = tiles * ((nb + kUnitBlocks - 1) / kUnitBlocks) * (kSeg == 3 ? a.nseg : (uint32_t)NS);
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
    return cudaLaunchKernelEx(&cfg, kern, a, a_end, a_end2);
}

template <int NS, int EPI, int kSeg>
cudaError_t launch_cfg_x(const WarpArgs& a, const uint8_t* a_end, const uint8_t* a_end2, cudaStream_t st,
                         int sm_count) {
    const uint32_t Kp = k_padded(a.K) * (kSeg == 3 ? a.nseg : 1u);
    const size_t s8 = smem_bytes_x(Kp, 8);
    if (s8 <= kTwoPerSmX && Kp / 256 <= (uint32_t)(kPrepX * 8)) return launch_x<NS, EPI, 8, kSeg>(a, a_end, a_end2, st, sm_count, s8);
    return launch_x<NS, EPI, 16, kSeg>(a, a_end, a_end2, st, sm_count, smem_bytes_x(Kp, 16));
}

bool common_ok(const DmmvArgs& a) {
    if (!a.scratch_partial || !a.status || !a.a_end) return false;
    // rows are fetched as 16-byte-aligned supersets: the buffers themselves must start on that boundary
    if ((reinterpret_cast<uintptr_t>(a.A) & 15u) || (a.A2 && (reinterpret_cast<uintptr_t>(a.A2) & 15u))) return false;
    if ((a.K & 31u) || a.K == 0) return false;
    if ((a.A_sh && ((reinterpret_cast<uintptr_t>(a.A_sh) & 15u) || !a.a_sh_end)) ||
        (a.A2_sh && ((reinterpret_cast<uintptr_t>(a.A2_sh) & 15u) || !a.a2_sh_end)))
        return false;
    if (smem_bytes_x(k_padded(a.K), 16) > 227 * 1024 || k_padded(a.K) / 256 > (uint32_t)(kPrepX * 8)) return false;
    return true;
}

}  // namespace

bool mxfp4_dmmv_eligible(uint32_t type, int mode, const DmmvArgs& a) {
    if (type != T_MXFP4 || mode != MODE_PLAIN || !common_ok(a)) return false;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * (((a.K >> 5) + kUnitBlocks - 1) / kUnitBlocks);
    return U >= 16 && U <= 0xFFFFFFFFull;
}

bool mxfp4_moe_gate_up_eligible(uint32_t type, const DmmvArgs& a) {
    if (type != T_MXFP4 || a.x_expert_stride != 0 || !a.routing || !a.A2 || (!a.y2 && !a.act) || !a.a2_end || !common_ok(a))
        return false;
    const uint64_t U = (uint64_t)a.n_used * ((a.M + 15) / 16) * (((a.K >> 5) + kUnitBlocks - 1) / kUnitBlocks) * 2;
    return a.n_used >= 1 && U >= 16 && U <= 0xFFFFFFFFull;
}

bool mxfp4_moe_down_acc_eligible(uint32_t type, const DmmvArgs& a) {
    if (type != T_MXFP4 || !a.routing || a.n_used == 0 || !common_ok(a)) return false;
    if ((a.x_expert_stride & 3u) || (reinterpret_cast<uintptr_t>(a.x) & 15u)) return false;  // float4 loads per slot
    const uint32_t Kp = k_padded(a.K) * a.n_used;
    if (smem_bytes_x(Kp, 16) > 227 * 1024 || Kp / 256 > (uint32_t)(kPrepX * 16)) return false;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * (((a.K >> 5) + kUnitBlocks - 1) / kUnitBlocks) * a.n_used;
    return U >= 16 && U <= 0xFFFFFFFFull;
}

static void fill_common(WarpArgs& wa, const DmmvArgs& a) {
    wa.A[0] = a.A;
    wa.A[1] = a.A2 ? a.A2 : a.A;
    wa.x = a.x;
    wa.y = a.y;
    wa.y2 = a.y2;
    wa.act = a.act;
    wa.gate = nullptr;
    wa.M = a.M;
    wa.K = a.K;
    wa.acc_mode = a.acc_mode;
    wa.gpartial = a.scratch_partial;
    wa.status = a.status;
    wa.spin_limit = a.spin_limit;
    wa.nseg = 0;
    wa.routing = a.routing;
    wa.n_experts_max = a.n_experts_max;
    wa.expert_stride = a.expert_stride;
    wa.tiles_per_expert = (a.M + 15) / 16;
    wa.x_slot_stride = 0;
    wa.A_sh[0] = a.A_sh;
    wa.A_sh[1] = a.A2_sh ? a.A2_sh : a.A_sh;
    wa.A_sh_end[0] = a.a_sh_end;
    wa.A_sh_end[1] = a.A2_sh ? a.a2_sh_end : a.a_sh_end;
    wa.bias[0] = a.bias;
    wa.bias[1] = a.bias2;
    wa.late = a.late;
}

cudaError_t launch_mxfp4_dmmv(const DmmvArgs& a, cudaStream_t st, uint64_t* launches) {
    WarpArgs wa;
    fill_common(wa, a);
    const cudaError_t e = launch_cfg_x<1, EPI_PLAIN, 0>(wa, a.a_end, a.a_end, st, a.sm_count);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

cudaError_t launch_mxfp4_moe_gate_up(const DmmvArgs& a, cudaStream_t st, uint64_t* launches) {
    WarpArgs wa;
    fill_common(wa, a);
    wa.nseg = a.n_used;
    wa.acc_mode = 0;
    const cudaError_t e = launch_cfg_x<2, EPI_PAIR, 2>(wa, a.a_end, a.a2_end, st, a.sm_count);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

cudaError_t launch_mxfp4_moe_down_acc(const DmmvArgs& a, cudaStream_t st, uint64_t* launches) {
    WarpArgs wa;
    fill_common(wa, a);
    wa.nseg = a.n_used;
    wa.x_slot_stride = a.x_expert_stride;
    const cudaError_t e = launch_cfg_x<1, EPI_ACC, 3>(wa, a.a_end, a.a_end, st, a.sm_count);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
