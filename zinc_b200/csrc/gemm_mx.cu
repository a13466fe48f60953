// MXFP4 prefill GEMM on the block-scaled tensor-core path: D[t][m] = sum_k W[m][k] X[t][k] with the GGUF MXFP4
// weights as they are (E2M1 nibbles, one E8M0 scale byte per 32 elements: exactly the operand format of
// tcgen05.mma kind::mxf8f6f4 with block scaling) and the bf16 activations split into two FP8 terms.
//
//   x = x_hi + x_lo, both E4M3 with their own power-of-two scale per 32 elements. A bf16 value has 8 significant
//   bits and an E4M3 value 4, so x_hi (x rounded to 4 significant bits) and x_lo (the remainder, again at most 4
//   significant bits) reproduce x exactly unless an element lies more than 2^14 below its block's maximum;
//   the two products accumulate into the same f32 accumulator. No weight is dequantised: a row's nibbles are only
//   re-ordered (GGUF keeps element j and j + 16 in one byte, the tensor core wants 16 consecutive elements in 8
//   bytes of a 16-byte chunk), about 0.6 integer operations per weight instead of 3.6 for the bf16 route.
//
//   1. mx_split_kernel   X bf16 [T][K] -> x_hi, x_lo (bytes [T][K]) and their scale bytes in the 512-byte atoms the
//                        tensor core reads (128 tokens x 4 blocks: byte (t % 32) * 16 + (t / 32) * 4 + block)
//   2. gemm_mx_kernel    persistent CTAs over (128 weight rows, 128 tokens) items; per 128-column stage: the weight
//                        stage (16 KB, K-major, 128-byte swizzle) and its 512 scale bytes written by the slot's 128
//                        producer threads (one per row) from raw bytes they copied into a private slot a stage ahead, x_hi / x_lo tiles
//                        by TMA, their scale atoms by bulk copies; one thread copies the three scale atoms into tensor
//                        memory (tcgen05.cp) and issues eight MMAs (four 32-column steps x two terms); two
//                        accumulators let the epilogue of an item overlap the next item's MMAs.
// Every mbarrier wait is bounded; a wait that gives up records {1, site}, raises the CTA's flag, and every role
// drains to the common exit where tensor memory is released.
//
// Replaces the tiled prefill GEMM dispatch for MXFP4 weights (src/compute/dmmv.zig:1045-1094 recordMulMmQ4K is
// its Q4_K form; element order and scale rule of MXFP4: src/compute/forward.zig:441-459).
#include <cuda_fp8.h>

#include "kernels.h"
#include "tc_common.cuh"

namespace zc {
namespace {

constexpr int kMxBN = 128;                 // tokens per item
constexpr int kMxStageK = 128;             // columns per stage: four MXFP4 blocks, one scale atom
constexpr int kMxStages = 3;
constexpr uint32_t kMxABytes = kBM * 128;  // 16 KB: 128 rows x 128 padded-FP4 bytes
constexpr uint32_t kMxXBytes = kMxBN * 128;
constexpr uint32_t kMxSfBytes = 512;
// A | x_hi | x_lo | sfa | sfb_hi | sfb_lo, padded to the 1024-byte alignment the swizzled tiles of the next stage need
constexpr uint32_t kMxStageBytes = (kMxABytes + 2 * kMxXBytes + 3 * kMxSfBytes + 1023u) & ~1023u;
// Warps: 0 tensor memory + MMA issue, 1 loader, then one group of four producer warps per stage slot (a thread
// per weight row; group j always fills slot j, so the groups work on different stages at the same time: a
// thread's chain of loads, shifts and stores per stage is latency-bound and four times the issuing thread's time
// per stage), then four epilogue warps.
constexpr int kMxProdWarp0 = 2, kMxGroupWarps = 4, kMxEpiWarp0 = kMxProdWarp0 + kMxStages * kMxGroupWarps;
constexpr int kMxThreads = (kMxEpiWarp0 + 4) * 32;
constexpr uint32_t kMxRawSlot = 96;        // bytes per producer thread: the 16-byte aligned superset of a row's 68
constexpr uint32_t kMxRawOffset = kMxStages * kMxStageBytes;
constexpr uint32_t kMxBarOffset = kMxRawOffset + kMxStages * 128 * kMxRawSlot;
constexpr uint32_t kMxSmemBytes = kMxBarOffset + 256 + 1024;
constexpr uint32_t kMxTmemCols = 512;      // two 128-column accumulators, then 12 scale columns per stage
constexpr uint32_t kMxSfCol0 = 2 * kMxBN;

struct MxBars {
    uint64_t full[kMxStages];    // the slot's four producer warps + the loader's expect_tx
    uint64_t empty[kMxStages];   // the issuing thread's commit
    uint64_t accum_full[2];
    uint64_t accum_empty[2];     // one arrival per epilogue warp
    uint32_t tmem_base;
    volatile uint32_t failed;
};

struct MxArgs {
    const uint8_t* A;        // MXFP4 rows, K / 32 blocks of 17 bytes
    const uint8_t* a_end;
    const uint8_t* sf_hi;    // scale atoms of x_hi: [token tiles][k atoms][512]
    const uint8_t* sf_lo;
    float* D;
    uint32_t M, N, K, stride_d, row_tiles, tok_tiles;
    uint32_t* status;
};

template <bool kSleep = true>
__device__ __forceinline__ bool mx_wait(uint64_t* bar, uint32_t parity, MxBars* bars, uint32_t* status, uint32_t site) {
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

// Shared-memory descriptor of a scale atom for tcgen05.cp: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes
// apart.
__device__ __forceinline__ uint64_t sf_desc(uint32_t saddr) {
    const uint32_t lo = ((saddr >> 4) & 0x3FFFu) | (1u << 16);
    const uint32_t hi = (128u >> 4) | (1u << 14);
    return ((uint64_t)hi << 32) | lo;
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t tmem_col, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(desc) : "memory");
}

// Instruction descriptor of the block-scaled MMA: A = E2M1, B = E4M3, both K-major, E8M0 scales, M = 128, N = 128,
// K = 32; sfa / sfb: which byte of the scale words this step uses.
__device__ __forceinline__ uint32_t mx_idesc(uint32_t sfa, uint32_t sfb) {
    return (sfb << 4) | (5u << 7) | (0u << 10) | ((uint32_t)(kMxBN >> 3) << 17) | (1u << 23) |
           ((uint32_t)(kBM >> 4) << 24) | (sfa << 29);
}
__device__ __forceinline__ void umma_mx(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Sixteen nibble bytes of a block (four words) -> the two 8-byte halves the tensor core reads: elements 0..15 (the
// low nibbles) and 16..31 (the high nibbles), two elements per byte, the lower element in the low nibble.
__device__ __forceinline__ void repack_block(const uint32_t (&q)[4], uint2& lo, uint2& hi) {
    uint32_t l[4], h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t a = q[i] & 0x0F0F0F0Fu, b = (q[i] >> 4) & 0x0F0F0F0Fu;
        l[i] = a | (a >> 4);  // bytes 0 and 2 hold the pairs (0,1) and (2,3)
        h[i] = b | (b >> 4);
    }
    lo = make_uint2(__byte_perm(l[0], l[1], 0x6420), __byte_perm(l[2], l[3], 0x6420));
    hi = make_uint2(__byte_perm(h[0], h[1], 0x6420), __byte_perm(h[2], h[3], 0x6420));
}

__global__ void __launch_bounds__(kMxThreads, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tmap_hi, const __grid_constant__ CUtensorMap tmap_lo, const MxArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    MxBars* bars = reinterpret_cast<MxBars*>(smem + kMxBarOffset);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t n_items = g.row_tiles * g.tok_tiles;
    const uint32_t nb = g.K >> 5;                          // blocks per row
    const int n_stages = (int)((nb + 3) >> 2);             // the last one may hold fewer than four blocks
    const uint64_t row_bytes = (uint64_t)nb * 17u;

    if (tid == 0) {
        for (int s = 0; s < kMxStages; ++s) {
            mbar_init(&bars->full[s], kMxGroupWarps + 1);
            mbar_init(&bars->empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars->accum_full[s], 1);
            mbar_init(&bars->accum_empty[s], 4);
        }
        bars->failed = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                     "r"(kMxTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        if (lane == 0) {  // ---- scale copies + MMA issuer ----
            uint32_t gs = 0, i = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++i) {
                const uint32_t ab = i & 1;
                ok = mx_wait<false>(&bars->accum_empty[ab], ((i >> 1) & 1) ^ 1, bars, g.status, 141);
                if (!ok) break;
                tc_fence_after();
                for (int s = 0; s < n_stages; ++s, ++gs) {
                    const uint32_t st = gs % kMxStages, ph = (gs / kMxStages) & 1;
                    ok = mx_wait<false>(&bars->full[st], ph, bars, g.status, 142);
                    if (!ok) break;
                    tc_fence_after();
                    uint8_t* stage = smem + st * kMxStageBytes;
                    const uint32_t sf_col = tmem + kMxSfCol0 + st * 12;
                    const uint32_t sf_s = smem_u32(stage + kMxABytes + 2 * kMxXBytes);
                    tmem_cp_sf(sf_col, sf_desc(sf_s));
                    tmem_cp_sf(sf_col + 4, sf_desc(sf_s + kMxSfBytes));
                    tmem_cp_sf(sf_col + 8, sf_desc(sf_s + 2 * kMxSfBytes));
                    const uint64_t da = smem_desc(smem_u32(stage));
                    const uint64_t dh = smem_desc(smem_u32(stage + kMxABytes));
                    const uint64_t dl = smem_desc(smem_u32(stage + kMxABytes + kMxXBytes));
                    const int steps = min(4, (int)nb - 4 * s);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (k < steps) {
                            umma_mx(tmem + ab * kMxBN, da + 2 * k, dh + 2 * k, mx_idesc(k, k), sf_col, sf_col + 4,
                                    (s | k) ? 1u : 0u);
                            umma_mx(tmem + ab * kMxBN, da + 2 * k, dl + 2 * k, mx_idesc(k, k), sf_col, sf_col + 8, 1u);
                        }
                    }
                    umma_commit(&bars->empty[st]);
                }
                if (ok) umma_commit(&bars->accum_full[ab]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // ---- loader of the activation terms and their scale atoms ----
            uint32_t gs = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
                const uint32_t tt = w / g.row_tiles;
                for (int s = 0; s < n_stages; ++s, ++gs) {
                    const uint32_t st = gs % kMxStages;
                    ok = mx_wait(&bars->empty[st], ((gs / kMxStages) & 1) ^ 1, bars, g.status, 143);
                    if (!ok) break;
                    uint8_t* stage = smem + st * kMxStageBytes;
                    mbar_expect_tx(&bars->full[st], 2 * kMxXBytes + 2 * kMxSfBytes);
                    tma_load_2d(stage + kMxABytes, &tmap_hi, s * kMxStageK, (int)(tt * kMxBN), &bars->full[st]);
                    tma_load_2d(stage + kMxABytes + kMxXBytes, &tmap_lo, s * kMxStageK, (int)(tt * kMxBN), &bars->full[st]);
                    const size_t atom = ((size_t)tt * n_stages + s) * kMxSfBytes;
                    bulk_load(stage + kMxABytes + 2 * kMxXBytes + kMxSfBytes, g.sf_hi + atom, kMxSfBytes, &bars->full[st]);
                    bulk_load(stage + kMxABytes + 2 * kMxXBytes + 2 * kMxSfBytes, g.sf_lo + atom, kMxSfBytes, &bars->full[st]);
                }
            }
        }
    } else if (warp >= kMxProdWarp0 && warp < kMxEpiWarp0) {
        // ---- weight producers: group = stage slot, thread = weight row; four blocks (68 bytes) per stage ----
        const int p = tid - kMxProdWarp0 * 32;
        const int row = p & 127;
        const uint32_t grp = (uint32_t)p >> 7;
        const uint32_t my_items = blockIdx.x < n_items ? (n_items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
        const uint32_t total = my_items * (uint32_t)n_stages;  // stages this CTA walks, in order
        uint8_t* my_raw = smem + kMxRawOffset + (size_t)p * kMxRawSlot;
        // byte offset (into A) of this thread's row segment for flat stage gs
        auto seg_off = [&](uint32_t gs) -> uint64_t {
            const uint32_t it = gs / (uint32_t)n_stages, s = gs - it * (uint32_t)n_stages;
            const uint32_t w = blockIdx.x + it * gridDim.x;
            const uint32_t grow = min((w % g.row_tiles) * kBM + (uint32_t)row, g.M - 1);  // rows past M: computed, dropped
            return (uint64_t)grow * row_bytes + (uint64_t)s * 68u;
        };
        // the segment's 16-byte aligned superset -> this thread's slot; bytes at or beyond the end of the buffer are
        // not read (zeros are written)
        auto fetch = [&](uint64_t off) {
            const uint8_t* src = g.A + (off & ~(uint64_t)15);
#pragma unroll
            for (int pc = 0; pc < (int)kMxRawSlot / 16; ++pc) {
                const uint8_t* sp = src + pc * 16;
                const uint32_t n = sp + 16 <= g.a_end ? 16u : (sp < g.a_end ? (uint32_t)(g.a_end - sp) : 0u);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(my_raw + pc * 16)),
                             "l"(n ? sp : g.A), "r"(n)
                             : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        uint64_t off = 0;
        if (grp < total) {
            off = seg_off(grp);
            fetch(off);
        }
        bool dead = false;
        for (uint32_t gs = grp; gs < total; gs += kMxStages) {
            // this stage's bytes out of the slot (shifted to the segment's first byte); then the slot is free for
            // the next own stage, whose copies fly while this one is repacked
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            const uint32_t o = (uint32_t)(off & 15u);
            uint32_t wd[17];
            lds_shifted<17>(reinterpret_cast<const uint32_t*>(my_raw + (o & ~3u)), (o & 3u) * 8u, wd);
            const uint32_t s = gs % (uint32_t)n_stages;
            if (gs + kMxStages < total) {
                off = seg_off(gs + kMxStages);
                fetch(off);
            }
            const uint32_t use = gs / kMxStages;  // slot grp, use number
            if (!dead) dead = !mx_wait(&bars->empty[grp], (use & 1) ^ 1, bars, g.status, 144);
            if (!dead) {
                uint8_t* stage = smem + grp * kMxStageBytes;
                uint8_t* rowp = stage + row * 128;
                const int sw = row & 7;
                uint32_t sf = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    // block b: scale byte at 17 b, nibble bytes 17 b + 1 .. 17 b + 16
                    constexpr int kW[4] = {0, 4, 8, 13};
                    constexpr int kS[4] = {8, 16, 24, 0};
                    const bool live = 4u * s + (uint32_t)b < nb;  // the last stage of a row may be short
                    uint32_t q[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        q[i] = kS[b] ? __funnelshift_r(wd[kW[b] + i], wd[kW[b] + i + 1], kS[b]) : wd[kW[b] + i];
                    const uint32_t e = (wd[(17 * b) >> 2] >> (8 * ((17 * b) & 3))) & 0xFFu;
                    uint2 lo, hi;
                    repack_block(q, lo, hi);
                    if (!live) lo = hi = make_uint2(0u, 0u);
                    *reinterpret_cast<uint4*>(rowp + (((2 * b) ^ sw) << 4)) = make_uint4(lo.x, lo.y, 0u, 0u);
                    *reinterpret_cast<uint4*>(rowp + (((2 * b + 1) ^ sw) << 4)) = make_uint4(hi.x, hi.y, 0u, 0u);
                    sf |= (live ? e : 127u) << (8 * b);
                }
                *reinterpret_cast<uint32_t*>(stage + kMxABytes + 2 * kMxXBytes + (row & 31) * 16 + (row >> 5) * 4) = sf;
                fence_proxy_async();
            }
            __syncwarp();
            if (lane == 0 && !dead) mbar_arrive(&bars->full[grp]);
        }
    } else if (warp >= kMxEpiWarp0) {
        // ---- epilogue: lane = weight row, column = token ----
        const uint32_t q = warp & 3;
        uint32_t i = 0;
        for (uint32_t w = blockIdx.x; w < n_items; w += gridDim.x, ++i) {
            const uint32_t ab = i & 1;
            const uint32_t tt = w / g.row_tiles;
            const uint32_t m = (w % g.row_tiles) * kBM + q * 32 + lane;
            const uint32_t t0 = tt * kMxBN, nt = min((uint32_t)kMxBN, g.N - t0);
            if (!mx_wait(&bars->accum_full[ab], (i >> 1) & 1, bars, g.status, 145)) break;
            __syncwarp();
            tc_fence_after();
#pragma unroll 1
            for (uint32_t c = 0; c * 32 < nt; ++c) {
                uint32_t v[32];
                const uint32_t taddr = tmem + ((q * 32u) << 16) + ab * kMxBN + c * 32;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                    "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
                      "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
                      "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
                      "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
                      "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (m < g.M) {
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj)
                        if (c * 32 + jj < nt)
                            g.D[(uint64_t)(t0 + c * 32 + jj) * g.stride_d + m] = __uint_as_float(v[jj]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->accum_empty[ab]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kMxTmemCols) : "memory");
    }
}

// ---- activation split ---------------------------------------------------------------------------------
// One thread per (token, 32-element block). Tokens at or beyond T (the padding of the last 128-token tile) only
// write neutral scale bytes; their x rows do not exist (the tensor map fills them with zeros).
__device__ __forceinline__ uint32_t scale_exp(float maxabs) {
    // power of two s = 2^(e - 127) with maxabs / s in [128, 256): inside E4M3's range (448), four bits kept
    const uint32_t E = (__float_as_uint(maxabs) >> 23) & 0xFFu;
    if (maxabs == 0.f) return 127u;
    return E < 8u ? 1u : (E - 7u > 254u ? 254u : E - 7u);
}
__device__ __forceinline__ float pow2_neg(uint32_t e) { return __uint_as_float((254u - e) << 23); }  // 2^(127 - e)
__device__ __forceinline__ float pow2_pos(uint32_t e) { return __uint_as_float(e << 23); }           // 2^(e - 127)
__device__ __forceinline__ float fp8_to_float(uint8_t v) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(v, __NV_E4M3)));
}

__global__ void __launch_bounds__(256) mx_split_kernel(const __nv_bfloat16* __restrict__ X, uint32_t stride_b,
                                                       uint8_t* __restrict__ x_hi, uint8_t* __restrict__ x_lo,
                                                       uint8_t* __restrict__ sf_hi, uint8_t* __restrict__ sf_lo,
                                                       uint32_t T, uint32_t K, uint32_t n_katoms) {
    const uint32_t nb = K >> 5;
    const uint64_t id = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t Tp = ((T + 127) / 128) * 128;
    if (id >= (uint64_t)Tp * n_katoms * 4) return;
    const uint32_t t = (uint32_t)(id / (n_katoms * 4)), b = (uint32_t)(id - (uint64_t)t * (n_katoms * 4));
    const size_t sf_at = ((size_t)(t >> 7) * n_katoms + (b >> 2)) * 512 + ((t & 127) & 31) * 16 + ((t & 127) >> 5) * 4 + (b & 3);
    if (t >= T || b >= nb) {
        sf_hi[sf_at] = 127;
        sf_lo[sf_at] = 127;
        return;
    }
    const uint4* src = reinterpret_cast<const uint4*>(X + (size_t)t * stride_b + (size_t)b * 32);
    float v[32];
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 w = __ldg(src + i);
        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v[i * 8 + 2 * j] = __uint_as_float(ww[j] << 16);
            v[i * 8 + 2 * j + 1] = __uint_as_float(ww[j] & 0xFFFF0000u);
        }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fabsf(v[i]));
    const uint32_t eh = scale_exp(mx);
    const float ih = pow2_neg(eh), sh = pow2_pos(eh);
    uint32_t hi[8], lo[8];
    float r[32];
    float mr = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const uint8_t q = (uint8_t)__nv_cvt_float_to_fp8(v[i] * ih, __NV_SATFINITE, __NV_E4M3);
        r[i] = v[i] - fp8_to_float(q) * sh;
        mr = fmaxf(mr, fabsf(r[i]));
        if ((i & 3) == 0) hi[i >> 2] = 0;
        hi[i >> 2] |= (uint32_t)q << (8 * (i & 3));
    }
    const uint32_t el = scale_exp(mr);
    const float il = pow2_neg(el);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const uint8_t q = (uint8_t)__nv_cvt_float_to_fp8(r[i] * il, __NV_SATFINITE, __NV_E4M3);
        if ((i & 3) == 0) lo[i >> 2] = 0;
        lo[i >> 2] |= (uint32_t)q << (8 * (i & 3));
    }
    uint4* dh = reinterpret_cast<uint4*>(x_hi + (size_t)t * K + (size_t)b * 32);
    uint4* dl = reinterpret_cast<uint4*>(x_lo + (size_t)t * K + (size_t)b * 32);
    dh[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    dh[1] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
    dl[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    dl[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
    sf_hi[sf_at] = (uint8_t)eh;
    sf_lo[sf_at] = (uint8_t)el;
}

struct MxLayout {
    uint64_t x_bytes, sf_bytes, total;
    uint32_t n_katoms, tok_tiles;
};
MxLayout mx_layout(uint32_t N, uint32_t K) {
    MxLayout l;
    l.n_katoms = (K + 127) / 128;
    l.tok_tiles = (N + kMxBN - 1) / kMxBN;
    l.x_bytes = (((uint64_t)N * K) + 1023) & ~1023ull;
    l.sf_bytes = (uint64_t)l.tok_tiles * l.n_katoms * 512;
    l.total = 2 * l.x_bytes + 2 * l.sf_bytes;
    return l;
}

}  // namespace

uint64_t mul_mm_mx_workspace_bytes(uint32_t N, uint32_t K) { return mx_layout(N, K).total; }

bool mul_mm_mx_eligible(uint32_t type, const uint8_t* A, const void* B, uint32_t N, uint32_t K, uint32_t stride_b,
                        const void* workspace, uint64_t workspace_size) {
    if (type != T_MXFP4 || (K & 31u) || K < 128 || N < 64) return false;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255u) || workspace_size < mx_layout(N, K).total) return false;
    return !(reinterpret_cast<uintptr_t>(A) & 15u) && !(reinterpret_cast<uintptr_t>(B) & 15u) && !(stride_b & 7u);
}

cudaError_t launch_mul_mm_mx(const uint8_t* A, uint64_t a_bytes, const void* B, float* D, uint32_t M, uint32_t N,
                             uint32_t K, uint32_t stride_b, uint32_t stride_d, void* workspace, uint32_t* status,
                             int sm_count, cudaStream_t s, uint64_t* launches) {
    EncodeFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    const MxLayout l = mx_layout(N, K);
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    uint8_t* x_hi = ws;
    uint8_t* x_lo = ws + l.x_bytes;
    uint8_t* sf_hi = ws + 2 * l.x_bytes;
    uint8_t* sf_lo = sf_hi + l.sf_bytes;
    CUtensorMap maps[2];
    for (int i = 0; i < 2; ++i) {
        const cuuint64_t dims[2] = {K, N};
        const cuuint64_t strides[1] = {(cuuint64_t)K};
        const cuuint32_t box[2] = {(cuuint32_t)kMxStageK, (cuuint32_t)kMxBN};
        const cuuint32_t estr[2] = {1, 1};
        if (enc(&maps[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, i == 0 ? x_hi : x_lo, dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorNotSupported;
    }
    const uint32_t Tp = l.tok_tiles * kMxBN;
    const uint64_t threads = (uint64_t)Tp * l.n_katoms * 4;
    mx_split_kernel<<<(uint32_t)((threads + 255) / 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(B), stride_b, x_hi,
                                                                      x_lo, sf_hi, sf_lo, N, K, l.n_katoms);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (launches) ++*launches;
    static std::atomic<uint64_t> attr_done{0};
    if ((e = ensure_dynamic_smem(gemm_mx_kernel, (int)kMxSmemBytes, attr_done)) != cudaSuccess) return e;
    MxArgs g;
    g.A = A;
    g.a_end = A + a_bytes;
    g.sf_hi = sf_hi;
    g.sf_lo = sf_lo;
    g.D = D;
    g.M = M;
    g.N = N;
    g.K = K;
    g.stride_d = stride_d;
    g.row_tiles = (M + kBM - 1) / kBM;
    g.tok_tiles = l.tok_tiles;
    g.status = status;
    const uint32_t items = g.row_tiles * g.tok_tiles;
    const uint32_t grid = items < (uint32_t)sm_count ? items : (uint32_t)sm_count;
    gemm_mx_kernel<<<grid, kMxThreads, kMxSmemBytes, s>>>(maps[0], maps[1], g);
    e = cudaGetLastError();
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
