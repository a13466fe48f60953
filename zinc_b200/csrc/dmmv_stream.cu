// Streaming decode matvec for B200: quantized rows are pulled through shared memory with
// bulk asynchronous copies (1-D TMA, mbarrier pipeline), the nibbles are turned into exact
// small-integer f16 values with one logic op each and fed to the tensor cores as a 16-row
// dot-product engine with f32 accumulation; K is split across workers so that every SM
// streams the same number of bytes.
//
// Stands in for the reference's K-parallel decode shaders and their fused epilogues
// (src/shaders/dmmv_q4k.comp:59-240, dmmv_q4k_wide.comp, dmmv_q4k_fused_gate_up_swiglu.comp:195-218,
// dmmv_q8_0_sigmoid_acc.comp:95-132) for the Q4_K layout of src/compute/forward.zig:370-409.
//
// Arithmetic per 256-weight super-block of a row, sub-blocks s = 0..7 of 32 weights:
//   y += 2^e * sum_s ( d*sc_s * D_s - (64*d*sc_s + dmin*m_s) * SX_s ),   D_s = sum_i (64+q_i) * x'_i
// x' = x * 2^-e is the block of x scaled into (-1024, 1024) and split into two f16 terms
// (x' = h1 + h2, 22 bits), SX_s = sum_i x'_i in f32. 64+q_i is exact in f16, products are exact
// in f32, D_s is accumulated in f32 by the tensor core. Weights are never rounded.
//
// Tensor-core mapping (mma.sync m16n8k16, f16 in, f32 out): the 16 A rows are 16 weight rows;
// lane (g = lane/4, t = lane%4) owns the 32-byte qs group t of rows g and g+8, i.e. sub-blocks
// 2t (low nibbles) and 2t+1 (high nibbles). B is made block-diagonal: column 2t+term is non-zero
// only in lane t's k slots, so D column 2t+term holds sub-block dot products of group t alone
// and lands in lane t's own accumulator registers. Scales are applied per lane afterwards.
#include "kernels.h"
#include "common.cuh"
#include "stream_common.cuh"

namespace zc {

namespace {

constexpr int kGroups = 3;               // independent streaming workers per CTA (one CTA per SM)
constexpr int kCW = 4;                   // consumer warps per worker (one super-block of a stage each)
constexpr int kGroupWarps = kCW + 1;     // + one producer warp
constexpr int kThreads = kGroups * kGroupWarps * 32;
constexpr int kStages = 3;
constexpr int kChunkBlocks = 8;          // super-blocks per row per stage
constexpr int kRowSeg = kChunkBlocks * 144 + 16;  // 592: rows land 16 B apart mod 32 B -> conflict-free 128-bit reads
constexpr int kStageBytes = 16 * kRowSeg;
constexpr int kRingBytes = kStages * kStageBytes;

struct StreamArgs {
    const uint8_t* A[2];
    const float* x;
    float* y;
    const float* gate;
    uint32_t M, K, acc_mode;
    float* partial;      // [workers][2][32] split-K partial sums
    uint32_t* counters;  // [tiles] arrival counters, zero between launches
    uint32_t* status;    // [0] error code, [1] site
};

struct Smem {
    uint4* xf;      // x in B-operand order: unit ((blk*8 + wi)*2 + term)*4 + t = 8 halves
    float* sx;      // per 32-element sub-block sum of x'
    float* xs;      // per super-block 2^e
    uint8_t* ring;  // kGroups rings of kStages stages of 16 row segments
    float* red;     // [kGroups][kCW][NS][16] cross-warp reduction
    uint64_t* full;   // [kGroups][kStages]
    uint64_t* empty;  // [kGroups][kStages]
    volatile uint32_t* flags;  // [0] abort
};

__host__ __device__ inline size_t smem_bytes(uint32_t K, int ns) {
    size_t n = (size_t)K * 4;  // xf
    n += (size_t)(K / 32) * 4 + (size_t)(K / 256) * 4;
    n = (n + 127) & ~size_t(127);
    n += (size_t)kGroups * kRingBytes;
    n += (size_t)kGroups * kCW * ns * 16 * 4;
    n += 2 * kGroups * kStages * 8 + 16;
    return n + 128;  // slack for aligning the dynamic base
}

__device__ inline Smem carve(uint8_t* base, uint32_t K, int ns) {
    Smem s;
    uintptr_t p = (reinterpret_cast<uintptr_t>(base) + 127) & ~uintptr_t(127);
    s.xf = reinterpret_cast<uint4*>(p);
    p += (size_t)K * 4;
    s.sx = reinterpret_cast<float*>(p);
    p += (size_t)(K / 32) * 4;
    s.xs = reinterpret_cast<float*>(p);
    p += (size_t)(K / 256) * 4;
    p = (p + 127) & ~uintptr_t(127);
    s.ring = reinterpret_cast<uint8_t*>(p);
    p += (size_t)kGroups * kRingBytes;
    s.red = reinterpret_cast<float*>(p);
    p += (size_t)kGroups * kCW * ns * 16 * 4;
    s.full = reinterpret_cast<uint64_t*>(p);
    s.empty = s.full + kGroups * kStages;
    s.flags = reinterpret_cast<volatile uint32_t*>(s.empty + kGroups * kStages);
    return s;
}

__device__ __forceinline__ uint4 lds128(const void* p) { return *reinterpret_cast<const uint4*>(p); }

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float2 unpack_h2(uint32_t v) {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

// Convert x into the tensor-core operand layout. One warp per super-block; lane = wi*4 + t
// handles elements 64t + 4wi + {0..3} (low-nibble sub-block 2t) and +32 (high-nibble 2t+1).
// A unit holds (e0, e2, e1, e3) of the low-nibble elements, then the same of the high ones:
// the order in which and_or() leaves the nibbles of one 32-bit word in A registers.
__device__ inline void prep_x(const Smem& s, const float* __restrict__ x, uint32_t K, int warp, int n_warps,
                              int lane) {
    const int wi = lane >> 2, t = lane & 3;
    for (uint32_t blk = warp; blk < (K >> 8); blk += n_warps) {
        const float* xp = x + (size_t)blk * 256 + 64 * t + 4 * wi;
        const float4 lo = __ldg(reinterpret_cast<const float4*>(xp));
        const float4 hi = __ldg(reinterpret_cast<const float4*>(xp + 32));
        float mx = fmaxf(fmaxf(fmaxf(fabsf(lo.x), fabsf(lo.y)), fmaxf(fabsf(lo.z), fabsf(lo.w))),
                         fmaxf(fmaxf(fabsf(hi.x), fabsf(hi.y)), fmaxf(fabsf(hi.z), fabsf(hi.w))));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        // |x'| < 1024: x' = x * 2^(136 - E), E the biased exponent of the block maximum
        uint32_t E = (__float_as_uint(mx) >> 23) & 0xFFu;
        E = E < 32u ? 32u : E;
        const float scale = __uint_as_float((263u - E) << 23);
        const float v0 = lo.x * scale, v1 = lo.y * scale, v2 = lo.z * scale, v3 = lo.w * scale;
        const float v4 = hi.x * scale, v5 = hi.y * scale, v6 = hi.z * scale, v7 = hi.w * scale;
        uint4 a, b;
        a.x = pack_h2(v0, v2); a.y = pack_h2(v1, v3); a.z = pack_h2(v4, v6); a.w = pack_h2(v5, v7);
        const float2 f02 = unpack_h2(a.x), f13 = unpack_h2(a.y), f46 = unpack_h2(a.z), f57 = unpack_h2(a.w);
        b.x = pack_h2(v0 - f02.x, v2 - f02.y); b.y = pack_h2(v1 - f13.x, v3 - f13.y);
        b.z = pack_h2(v4 - f46.x, v6 - f46.y); b.w = pack_h2(v5 - f57.x, v7 - f57.y);
        const float2 r02 = unpack_h2(b.x), r13 = unpack_h2(b.y), r46 = unpack_h2(b.z), r57 = unpack_h2(b.w);
        s.xf[((blk * 8 + wi) * 2 + 0) * 4 + t] = a;
        s.xf[((blk * 8 + wi) * 2 + 1) * 4 + t] = b;
        // sub-block sums of exactly the values the tensor core multiplies (h1 + h2 is exact in f32)
        float slo = ((f02.x + r02.x) + (f02.y + r02.y)) + ((f13.x + r13.x) + (f13.y + r13.y));
        float shi = ((f46.x + r46.x) + (f46.y + r46.y)) + ((f57.x + r57.x) + (f57.y + r57.y));
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            slo += __shfl_xor_sync(0xFFFFFFFFu, slo, o);
            shi += __shfl_xor_sync(0xFFFFFFFFu, shi, o);
        }
        if (wi == 0) *reinterpret_cast<float2*>(s.sx + blk * 8 + 2 * t) = make_float2(slo, shi);
        if (lane == 0) s.xs[blk] = __uint_as_float((E - 9u) << 23);
    }
}

enum { EPI_PLAIN = 0, EPI_GATE_UP = 1, EPI_SIGMOID_ACC = 2 };

template <int NS, int EPI>
__device__ __forceinline__ void write_rows(const StreamArgs& a, uint32_t row, const float (&v)[NS]) {
    if (row >= a.M) return;
    if constexpr (EPI == EPI_GATE_UP) {
        a.y[row] = (v[0] / (1.0f + expf(-v[0]))) * v[1];
    } else if constexpr (EPI == EPI_SIGMOID_ACC) {
        a.y[row] += (1.0f / (1.0f + expf(-__ldg(a.gate)))) * v[0];
    } else {
        a.y[row] = a.acc_mode ? a.y[row] + v[0] : v[0];
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

template <int NS, int EPI>
__global__ void __launch_bounds__(kThreads, 1) dmmv_q4k_stream_kernel(const StreamArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const Smem s = carve(smem_raw, a.K, NS);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int grp = warp / kGroupWarps, gw = warp % kGroupWarps;  // worker group, warp within it
    const uint32_t bpr = a.K >> 8;
    const uint64_t row_bytes = (uint64_t)bpr * 144;
    const uint32_t upt = (bpr + kChunkBlocks - 1) / kChunkBlocks;  // k-chunks per row
    const uint32_t upt_all = upt * NS;                               // units per tile
    const uint32_t tiles = (a.M + 15) / 16;
    const uint32_t U = tiles * upt_all, G = gridDim.x * kGroups;    // units, workers (G <= U)
    const uint32_t me = blockIdx.x * kGroups + grp;
    const uint32_t u0 = (uint32_t)part_begin(me, U, G), u1 = (uint32_t)part_begin(me + 1, U, G);
    uint64_t* full = s.full + grp * kStages;
    uint64_t* empty = s.empty + grp * kStages;
    uint8_t* ring = s.ring + (size_t)grp * kRingBytes;

    if (tid == 0) {
        for (int i = 0; i < kGroups * kStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], kCW);
        }
        s.flags[0] = 0;
        mbar_fence_init();
    }
    __syncthreads();

    // first unit of this worker as (tile, stream, k-chunk); later units advance incrementally
    uint32_t tile = u0 / upt_all, strm = (u0 % upt_all) / upt, kc = (u0 % upt_all) % upt;
    auto advance = [&]() {
        if (++kc == upt) {
            kc = 0;
            if (++strm == NS) { strm = 0; ++tile; }
        }
    };

    if (gw == kCW) {
        // ---------------- producer warp: lane r copies the segment of row r ----------------
        auto produce = [&](uint32_t it) -> bool {
            const uint32_t st = it % kStages, ph = (it / kStages) & 1u;
            if (s.flags[0]) return false;
            if (!mbar_wait_bounded(&empty[st], ph ^ 1u)) {
                if (lane == 0) { a.status[0] = 1; a.status[1] = 1; s.flags[0] = 1; }
                return false;
            }
            const uint32_t nblk = min((uint32_t)kChunkBlocks, bpr - kc * kChunkBlocks);
            const uint32_t bytes = nblk * 144;
            const uint32_t rows = min(16u, a.M - tile * 16);
            if (lane == 0) mbar_expect_tx(&full[st], rows * bytes);
            __syncwarp();
            if (lane < rows) {
                const uint8_t* src = a.A[strm] + (uint64_t)(tile * 16 + lane) * row_bytes +
                                     (uint64_t)kc * kChunkBlocks * 144;
                bulk_g2s(ring + (size_t)st * kStageBytes + lane * kRowSeg, src, bytes, &full[st]);
            }
            advance();
            return true;
        };
        // fill the ring first (weights do not depend on x), help convert x, then keep streaming
        const uint32_t n = u1 - u0;
        uint32_t it = 0;
        bool ok = true;
        for (; ok && it < n && it < kStages; ++it) ok = produce(it);
        prep_x(s, a.x, a.K, warp, kGroups * kGroupWarps, lane);
        __syncthreads();
        for (; ok && it < n; ++it) ok = produce(it);
        return;
    }

    // ---------------- consumer warps ----------------
    prep_x(s, a.x, a.K, warp, kGroups * kGroupWarps, lane);
    __syncthreads();

    const int g = lane >> 2, t = lane & 3;
    float* red = s.red + (size_t)grp * kCW * NS * 16;
    const int bar_id = 1 + grp;
    float acc[NS][2];
#pragma unroll
    for (int i = 0; i < NS; ++i) acc[i][0] = acc[i][1] = 0.f;
    bool aborted = false;
    // B operand: lane (g, t) feeds column g, which is live only for g in {2t, 2t+1}
    const bool b_live = (g >> 1) == t;
    const uint4* xu_lane = s.xf + (g & 1) * 4 + t;

    auto flush = [&](uint32_t T) {
#pragma unroll
        for (int i = 0; i < NS; ++i) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float v = acc[i][r];
                v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
                v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
                if (t == 0) red[(gw * NS + i) * 16 + g + 8 * r] = v;
                acc[i][r] = 0.f;
            }
        }
        named_bar_sync(bar_id, kCW * 32);
        if (gw == 0) {
            float v[NS];
            if (lane < 16) {
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    v[i] = 0.f;
#pragma unroll
                    for (int w = 0; w < kCW; ++w) v[i] += red[(w * NS + i) * 16 + lane];
                }
            }
            const uint32_t first = T * upt_all, last = first + upt_all - 1;
            if (u0 <= first && last < u1) {
                if (lane < 16) write_rows<NS, EPI>(a, T * 16 + lane, v);
            } else {
                // partial tile: publish, count arrivals; the last arrival sums every part in worker order
                const uint32_t my_slot = (u0 / upt_all) == T ? 0u : 1u;
                float* mine = a.partial + ((size_t)me * 2 + my_slot) * 32;
                if (lane < 16) {
#pragma unroll
                    for (int i = 0; i < NS; ++i) mine[i * 16 + lane] = v[i];
                    __threadfence();
                }
                __syncwarp();
                const uint32_t cf = part_owner(first, U, G), cl = part_owner(last, U, G);
                uint32_t old = 0;
                if (lane == 0) old = atomicAdd(&a.counters[T], 1u);
                old = __shfl_sync(0xFFFFFFFFu, old, 0);
                if (old == cl - cf) {
                    __threadfence();
                    if (lane < 16) {
                        float tot[NS];
#pragma unroll
                        for (int i = 0; i < NS; ++i) tot[i] = 0.f;
                        for (uint32_t c = cf; c <= cl; ++c) {
                            const uint32_t slot = ((uint32_t)part_begin(c, U, G) / upt_all) == T ? 0u : 1u;
                            const float* p = a.partial + ((size_t)c * 2 + slot) * 32;
#pragma unroll
                            for (int i = 0; i < NS; ++i) tot[i] += ld_cg_f32(p + i * 16 + lane);
                        }
                        write_rows<NS, EPI>(a, T * 16 + lane, tot);
                    }
                    if (lane == 0) a.counters[T] = 0;
                }
            }
        }
        named_bar_sync(bar_id, kCW * 32);
    };

    const uint32_t n = u1 - u0;
    uint32_t cur_tile = tile;
    for (uint32_t it = 0; it < n; ++it) {
        const uint32_t st = it % kStages, ph = (it / kStages) & 1u;
        if (tile != cur_tile) {
            flush(cur_tile);
            cur_tile = tile;
        }
        if (!aborted && !mbar_wait_bounded(&full[st], ph)) {
            if (lane == 0) { a.status[0] = 1; a.status[1] = 2; s.flags[0] = 1; }
            aborted = true;
        }
        for (int bi = gw; bi < kChunkBlocks; bi += kCW) {
            const uint32_t blk = kc * kChunkBlocks + bi;  // this warp's super-block within the row
            if (aborted || blk >= bpr) break;
            const uint8_t* sb = ring + (size_t)st * kStageBytes + bi * 144;
            const uint8_t* rA = sb + g * kRowSeg;
            const uint8_t* rB = sb + (g + 8) * kRowSeg;
            const uint4 hA = lds128(rA), hB = lds128(rB);
            const uint4 qa0 = lds128(rA + 16 + 32 * t), qa1 = lds128(rA + 32 + 32 * t);
            const uint4 qb0 = lds128(rB + 16 + 32 * t), qb1 = lds128(rB + 32 + 32 * t);
            const uint32_t qa[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
            const uint32_t qb[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
            const uint4* xu = xu_lane + (size_t)blk * 64;
            float dlo[4] = {0.f, 0.f, 0.f, 0.f}, dhi[4] = {0.f, 0.f, 0.f, 0.f};
            constexpr uint32_t kMask = 0x00F000F0u, kMagic = 0x54005400u;  // f16 64.0 + nibble in mantissa bits 4..7
#pragma unroll
            for (int wi = 0; wi < 8; ++wi) {
                uint4 b = make_uint4(0u, 0u, 0u, 0u);
                if (b_live) b = xu[wi * 8];
                const uint32_t wa = qa[wi], wb = qb[wi];
                // low nibbles of bytes (0,2) and (1,3): shift them up into bits 4..7
                mma_f16(dlo, and_or(wa << 4, kMask, kMagic), and_or(wb << 4, kMask, kMagic),
                        and_or(wa >> 4, kMask, kMagic), and_or(wb >> 4, kMask, kMagic), b.x, b.y);
                // high nibbles already sit in bits 4..7
                mma_f16(dhi, and_or(wa, kMask, kMagic), and_or(wb, kMask, kMagic),
                        and_or(wa >> 8, kMask, kMagic), and_or(wb >> 8, kMask, kMagic), b.z, b.w);
            }
            // lane t's accumulator columns (2t, 2t+1) = the two f16 terms of x for its own sub-blocks
            const float DloA = dlo[0] + dlo[1], DloB = dlo[2] + dlo[3];
            const float DhiA = dhi[0] + dhi[1], DhiB = dhi[2] + dhi[3];
            uint32_t scA, mnA, scB, mnB;
            scales_mins_pair(hA.y, hA.z, hA.w, t, scA, mnA);
            scales_mins_pair(hB.y, hB.z, hB.w, t, scB, mnB);
            const float xs = s.xs[blk];
            const float2 sxv = *reinterpret_cast<const float2*>(s.sx + blk * 8 + 2 * t);
            const float dA = h2f(hA.x) * xs, dmA = h2f(hA.x >> 16) * xs;
            const float dB = h2f(hB.x) * xs, dmB = h2f(hB.x >> 16) * xs;
            const float cA0 = dA * (float)(scA & 0xFFu), cA1 = dA * (float)(scA >> 8);
            const float cB0 = dB * (float)(scB & 0xFFu), cB1 = dB * (float)(scB >> 8);
            float vA = cA0 * DloA + cA1 * DhiA;
            vA -= (64.f * cA0 + dmA * (float)(mnA & 0xFFu)) * sxv.x + (64.f * cA1 + dmA * (float)(mnA >> 8)) * sxv.y;
            float vB = cB0 * DloB + cB1 * DhiB;
            vB -= (64.f * cB0 + dmB * (float)(mnB & 0xFFu)) * sxv.x + (64.f * cB1 + dmB * (float)(mnB >> 8)) * sxv.y;
#pragma unroll
            for (int i = 0; i < NS; ++i) {
                acc[i][0] += (strm == (uint32_t)i) ? vA : 0.f;
                acc[i][1] += (strm == (uint32_t)i) ? vB : 0.f;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
        advance();
    }
    if (n) flush(cur_tile);
}

template <int NS, int EPI>
cudaError_t launch_cfg(const StreamArgs& a, cudaStream_t st, int sm_count) {
    auto kern = dmmv_q4k_stream_kernel<NS, EPI>;
    static bool attr_set = false;
    const size_t smem = smem_bytes(a.K, NS);
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    const uint32_t bpr = a.K >> 8;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * ((bpr + kChunkBlocks - 1) / kChunkBlocks) * NS;
    uint64_t grid = (uint64_t)sm_count;  // one CTA per SM, kGroups workers each
    if (grid * kGroups > U) grid = U / kGroups;
    if (grid * kGroups > kStreamMaxGrid) grid = kStreamMaxGrid / kGroups;
    if (grid == 0) return cudaErrorInvalidConfiguration;
    kern<<<(uint32_t)grid, kThreads, smem, st>>>(a);
    return cudaGetLastError();
}

}  // namespace

bool stream_dmmv_eligible(uint32_t type, int mode, const DmmvArgs& a) {
    if (type != T_Q4_K) return false;
    if (mode != MODE_PLAIN && mode != MODE_GATE_UP_SWIGLU && mode != MODE_SIGMOID_ACC) return false;
    if (!a.scratch_partial || !a.scratch_counters || !a.status) return false;
    if ((reinterpret_cast<uintptr_t>(a.A) & 15u) || (a.A2 && (reinterpret_cast<uintptr_t>(a.A2) & 15u))) return false;
    if (a.M < 64 || (a.M + 15) / 16 > kStreamMaxTiles) return false;
    const int ns = mode == MODE_GATE_UP_SWIGLU ? 2 : 1;
    if (smem_bytes(a.K, ns) > 227 * 1024) return false;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * (((a.K >> 8) + kChunkBlocks - 1) / kChunkBlocks) * ns;
    if (U < kGroups || U > 0xFFFFFFFFull) return false;
    return true;
}

cudaError_t launch_stream_dmmv(uint32_t type, int mode, const DmmvArgs& a, cudaStream_t st, uint64_t* launches) {
    (void)type;
    StreamArgs sa;
    sa.A[0] = a.A;
    sa.A[1] = a.A2 ? a.A2 : a.A;
    sa.x = a.x;
    sa.y = a.y;
    sa.gate = a.gate;
    sa.M = a.M;
    sa.K = a.K;
    sa.acc_mode = a.acc_mode;
    sa.partial = a.scratch_partial;
    sa.counters = a.scratch_counters;
    sa.status = a.status;
    cudaError_t e;
    switch (mode) {
        case MODE_PLAIN: e = launch_cfg<1, EPI_PLAIN>(sa, st, a.sm_count); break;
        case MODE_GATE_UP_SWIGLU: e = launch_cfg<2, EPI_GATE_UP>(sa, st, a.sm_count); break;
        case MODE_SIGMOID_ACC: e = launch_cfg<1, EPI_SIGMOID_ACC>(sa, st, a.sm_count); break;
        default: return cudaErrorInvalidValue;
    }
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
