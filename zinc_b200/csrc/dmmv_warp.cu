// Warp-autonomous streaming decode matvec for B200 (Q4_K).
//
// Every warp is an independent worker: it owns a contiguous range of work units
// (16 rows x one 256-weight super-block), prefetches them with 16-byte asynchronous copies
// (cp.async, lane-private shared-memory slots, depth kDepth), turns nibbles into exact small
// f16 integers with one logic op each and uses the tensor cores as a 16-row dot-product
// engine with f32 accumulation. There is no block-wide synchronisation after the activation
// vector has been converted. K is split across workers so that all SMs stream the same number
// of bytes; a tile that spans several workers is finished by the worker that owns its first
// unit, which adds the partial sums the later workers have published (shared memory inside a
// CTA, global memory across CTAs) in worker order, so results do not depend on timing.
//
// Stands in for the reference's K-parallel decode shaders and their fused epilogues
// (src/shaders/dmmv_q4k.comp:59-240, dmmv_q4k_wide.comp, dmmv_q4k_fused_gate_up_swiglu.comp:195-218,
// dmmv_q8_0_sigmoid_acc.comp:95-132) for the Q4_K layout of src/compute/forward.zig:370-409.
//
// Arithmetic per super-block of a row, sub-blocks s = 0..7 of 32 weights:
//   y += 2^e * sum_s ( d*sc_s * D_s - (64*d*sc_s + dmin*m_s) * SX_s ),   D_s = sum_i (64+q_i) * x'_i
// x' = x * 2^-e is the block of x scaled into (-1024, 1024) and split into two f16 terms
// (x' = h1 + h2, 22 bits), SX_s = sum_i x'_i in f32. 64+q_i is exact in f16, products are exact
// in f32, D_s is accumulated in f32 by the tensor core. Weights are never rounded.
//
// Tensor-core mapping (mma.sync m16n8k16, f16 in, f32 out): the 16 A rows are 16 weight rows;
// lane (g = lane/4, t = lane%4) owns the 32-byte qs group t of rows g and g+8, i.e. sub-blocks
// 2t (low nibbles) and 2t+1 (high nibbles). B is block-diagonal: column 2t+term is non-zero
// only in lane t's k slots, so D column 2t+term holds sub-block dot products of group t alone
// and lands in lane t's own accumulator registers. Scales are applied per lane afterwards.
#include "kernels.h"
#include "common.cuh"
#include "stream_common.cuh"

namespace zc {

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kDepth = 3;                  // prefetched units per warp
constexpr int kSlotBytes = 6 * 512;        // 6 pieces of 16 B per lane
constexpr int kWarpRing = kDepth * kSlotBytes;
constexpr int kZeroUnits = 64;             // 1 KB of zeros: B operand of the lanes whose column is dead

struct WarpArgs {
    const uint8_t* A[2];
    const float* x;
    float* y;
    const float* gate;
    uint32_t M, K, acc_mode;
    float* gpartial;     // [workers][32] partial sums published across CTAs
    uint32_t* gflags;    // [workers] 0 = empty, 1 = published; the reader clears it
    uint32_t* status;    // [0] error code, [1] site
};

struct Smem {
    uint4* xf;       // x in B-operand order: unit ((blk*8 + wi)*2 + term)*4 + t = 8 halves
    uint4* zeros;    // kZeroUnits zero units
    float* sx;       // per 32-element sub-block sum of x'
    float* xs;       // per super-block 2^e
    uint8_t* ring;   // [kWarps][kDepth][6][32] 16-byte pieces
    float* spartial; // [kWarps][32] partial sums published inside the CTA
    volatile uint32_t* sflags;  // [kWarps]
};

__host__ __device__ inline size_t smem_bytes(uint32_t K) {
    size_t n = (size_t)K * 4 + (size_t)kZeroUnits * 16;
    n += (size_t)(K / 32) * 4 + (size_t)(K / 256) * 4;
    n = (n + 127) & ~size_t(127);
    n += (size_t)kWarps * kWarpRing;
    n += (size_t)kWarps * 32 * 4 + (size_t)kWarps * 4;
    return n + 128;
}

__device__ inline Smem carve(uint8_t* base, uint32_t K) {
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

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
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
__device__ inline void prep_x(const Smem& s, const float* __restrict__ x, uint32_t K, int warp, int lane) {
    const int wi = lane >> 2, t = lane & 3;
    for (uint32_t blk = warp; blk < (K >> 8); blk += kWarps) {
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
__device__ __forceinline__ void write_row(const WarpArgs& a, uint32_t row, const float (&v)[NS]) {
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

constexpr uint32_t kSpinLimit = 1u << 26;

template <int NS, int EPI>
__global__ void __launch_bounds__(kThreads, 1) dmmv_q4k_warp_kernel(const WarpArgs a) {
    extern __shared__ uint8_t smem_raw[];
    const Smem s = carve(smem_raw, a.K);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t bpr = a.K >> 8;
    const uint64_t row_bytes = (uint64_t)bpr * 144;
    const uint32_t upt_all = bpr * NS;  // units per 16-row tile
    const uint32_t tiles = (a.M + 15) / 16;
    const uint32_t U = tiles * upt_all, G = gridDim.x * kWarps;  // units, workers (G <= U)
    const uint32_t me = blockIdx.x * kWarps + warp;
    const uint32_t u0 = (uint32_t)part_begin(me, U, G), u1 = (uint32_t)part_begin(me + 1, U, G);
    const uint32_t n = u1 - u0;
    uint8_t* ring = s.ring + (size_t)warp * kWarpRing + lane * 16;

    // ---- prefetch iterator: (tile, stream, block) of the next unit to request ----
    uint32_t p_tile = u0 / upt_all, p_strm = (u0 % upt_all) / bpr, p_blk = (u0 % upt_all) % bpr;
    auto request = [&](uint32_t slot) {
        const uint32_t rA = min(p_tile * 16 + g, a.M - 1), rB = min(p_tile * 16 + g + 8, a.M - 1);
        const uint8_t* base = a.A[p_strm] + (uint64_t)p_blk * 144;
        const uint8_t* pa = base + rA * row_bytes;
        const uint8_t* pb = base + rB * row_bytes;
        uint8_t* dst = ring + slot * kSlotBytes;
        cp_async16(dst, pa);
        cp_async16(dst + 512, pb);
        cp_async16(dst + 1024, pa + 16 + 32 * t);
        cp_async16(dst + 1536, pa + 32 + 32 * t);
        cp_async16(dst + 2048, pb + 16 + 32 * t);
        cp_async16(dst + 2560, pb + 32 + 32 * t);
        if (++p_blk == bpr) {
            p_blk = 0;
            if (++p_strm == NS) { p_strm = 0; ++p_tile; }
        }
    };
#pragma unroll
    for (int i = 0; i < kDepth; ++i) {
        if ((uint32_t)i < n) request(i);
        cp_async_commit();
    }

    // ---- activation vector -> B operand layout (all warps), zero region, flags ----
    if (tid < kZeroUnits) s.zeros[tid] = make_uint4(0u, 0u, 0u, 0u);
    if (tid < kWarps) s.sflags[tid] = 0u;
    prep_x(s, a.x, a.K, warp, lane);
    __syncthreads();

    // ---- consume ----
    uint32_t tile = u0 / upt_all, strm = (u0 % upt_all) / bpr, blk = (u0 % upt_all) % bpr;
    float acc[NS][2];
#pragma unroll
    for (int i = 0; i < NS; ++i) acc[i][0] = acc[i][1] = 0.f;
    const bool b_live = (g >> 1) == t;  // lane (g, t) feeds B column g, live only for g in {2t, 2t+1}
    const uint4* xu_live = s.xf + (g & 1) * 4 + t;

    auto finish_tile = [&](uint32_t T) {
        // rows g and g+8 of this warp: reduce over the four lanes of a row
        float v[NS][2];
#pragma unroll
        for (int i = 0; i < NS; ++i) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float w = acc[i][r];
                w += __shfl_xor_sync(0xFFFFFFFFu, w, 1);
                w += __shfl_xor_sync(0xFFFFFFFFu, w, 2);
                v[i][r] = w;
                acc[i][r] = 0.f;
            }
        }
        const uint32_t first = T * upt_all, last = first + upt_all - 1;
        if (u0 > first) {
            // not the first contributor: publish the partial sums for the worker that owns `first`
            const uint32_t fin = part_owner(first, U, G);
            const bool same_cta = fin / kWarps == blockIdx.x;
            float* dst = same_cta ? s.spartial + warp * 32 : a.gpartial + (size_t)me * 32;
            if (t == 0) {
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    dst[i * 16 + g] = v[i][0];
                    dst[i * 16 + g + 8] = v[i][1];
                }
                if (same_cta) __threadfence_block(); else __threadfence();
            }
            __syncwarp();
            if (lane == 0) {
                if (same_cta) s.sflags[warp] = 1u;
                else *reinterpret_cast<volatile uint32_t*>(a.gflags + me) = 1u;
            }
            return;
        }
        if (last >= u1) {
            // first contributor of a tile that continues in later workers: add their parts in order
            const uint32_t cl = part_owner(last, U, G);
            for (uint32_t c = me + 1; c <= cl; ++c) {
                const bool same_cta = c / kWarps == blockIdx.x;
                volatile uint32_t* flag = same_cta ? s.sflags + (c % kWarps)
                                                   : reinterpret_cast<volatile uint32_t*>(a.gflags + c);
                uint32_t spins = 0;
                while (*flag == 0u) {
                    if (++spins > kSpinLimit) {
                        if (lane == 0) { a.status[0] = 1; a.status[1] = 3; }
                        break;
                    }
                }
                if (same_cta) __threadfence_block(); else __threadfence();
                const float* src = same_cta ? s.spartial + (c % kWarps) * 32 : a.gpartial + (size_t)c * 32;
                if (t == 0) {
#pragma unroll
                    for (int i = 0; i < NS; ++i) {
                        v[i][0] += same_cta ? src[i * 16 + g] : ld_cg_f32(src + i * 16 + g);
                        v[i][1] += same_cta ? src[i * 16 + g + 8] : ld_cg_f32(src + i * 16 + g + 8);
                    }
                }
                __syncwarp();
                if (!same_cta && lane == 0) *flag = 0u;  // leave the global flags clear for the next launch
            }
        }
        if (t == 0) {
            float r0[NS], r1[NS];
#pragma unroll
            for (int i = 0; i < NS; ++i) { r0[i] = v[i][0]; r1[i] = v[i][1]; }
            write_row<NS, EPI>(a, T * 16 + g, r0);
            write_row<NS, EPI>(a, T * 16 + g + 8, r1);
        }
    };

    constexpr uint32_t kMask = 0x00F000F0u, kMagic = 0x54005400u;  // f16 64.0 + nibble in mantissa bits 4..7
    for (uint32_t it = 0; it < n; ++it) {
        cp_async_wait<kDepth - 1>();
        const uint8_t* sl = ring + (it % kDepth) * kSlotBytes;
        const uint4 hA = lds128(sl), hB = lds128(sl + 512);
        const uint4 qa0 = lds128(sl + 1024), qa1 = lds128(sl + 1536);
        const uint4 qb0 = lds128(sl + 2048), qb1 = lds128(sl + 2560);
        const uint32_t qa[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
        const uint32_t qb[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
        const uint4* xu = b_live ? xu_live + (size_t)blk * 64 : s.zeros;
        float dlo[4] = {0.f, 0.f, 0.f, 0.f}, dhi[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int wi = 0; wi < 8; ++wi) {
            const uint4 b = xu[wi * 8];
            const uint32_t wa = qa[wi], wb = qb[wi];
            // low nibbles of bytes (0,2) and (1,3): shift them into bits 4..7
            mma_f16(dlo, and_or(wa << 4, kMask, kMagic), and_or(wb << 4, kMask, kMagic),
                    and_or(wa >> 4, kMask, kMagic), and_or(wb >> 4, kMask, kMagic), b.x, b.y);
            // high nibbles already sit in bits 4..7
            mma_f16(dhi, and_or(wa, kMask, kMagic), and_or(wb, kMask, kMagic),
                    and_or(wa >> 8, kMask, kMagic), and_or(wb >> 8, kMask, kMagic), b.z, b.w);
        }
        // the slot's bytes are in registers now: request the unit kDepth ahead into it
        if (it + kDepth < n) request(it % kDepth);
        cp_async_commit();

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
        // advance; a tile ends with its last unit or with this worker's range
        const uint32_t T = tile;
        bool tile_done = false;
        if (++blk == bpr) {
            blk = 0;
            if (++strm == NS) { strm = 0; ++tile; tile_done = true; }
        }
        if (tile_done || it + 1 == n) finish_tile(T);
    }
    cp_async_wait<0>();
}

template <int NS, int EPI>
cudaError_t launch_cfg(const WarpArgs& a, cudaStream_t st, int sm_count) {
    auto kern = dmmv_q4k_warp_kernel<NS, EPI>;
    static bool attr_set = false;
    const size_t smem = smem_bytes(a.K);
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * (a.K >> 8) * NS;
    uint64_t grid = (uint64_t)sm_count;  // one CTA per SM, kWarps workers each
    if (grid * kWarps > U) grid = U / kWarps;
    if (grid * kWarps > kStreamMaxWorkers) grid = kStreamMaxWorkers / kWarps;
    if (grid == 0) return cudaErrorInvalidConfiguration;
    kern<<<(uint32_t)grid, kThreads, smem, st>>>(a);
    return cudaGetLastError();
}

}  // namespace

bool warp_dmmv_eligible(uint32_t type, int mode, const DmmvArgs& a) {
    if (type != T_Q4_K) return false;
    if (mode != MODE_PLAIN && mode != MODE_GATE_UP_SWIGLU && mode != MODE_SIGMOID_ACC) return false;
    if (!a.scratch_partial || !a.scratch_flags || !a.status) return false;
    if ((reinterpret_cast<uintptr_t>(a.A) & 15u) || (a.A2 && (reinterpret_cast<uintptr_t>(a.A2) & 15u))) return false;
    if (smem_bytes(a.K) > 227 * 1024) return false;
    const int ns = mode == MODE_GATE_UP_SWIGLU ? 2 : 1;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * (a.K >> 8) * ns;
    if (U < kWarps || U > 0xFFFFFFFFull) return false;
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

}  // namespace zc
