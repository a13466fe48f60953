// Prefill dequant-GEMM on the 5th-generation tensor cores: D[n][m] = sum_k W[m][k] * X[n][k].
//
//   W  quantised GGUF rows (Q4_K or Q6_K), read in place and dequantised to bf16 by producer warps straight
//      into the shared-memory layout tcgen05.mma consumes (K-major, 128-byte swizzle)
//   X  bf16 activations [N][stride_b], fetched by TMA (cp.async.bulk.tensor, 128-byte swizzle)
//   D  f32 [N][stride_d]; accumulators live in tensor memory and are read back with tcgen05.ld
//
// Three kernels. More than 256 tokens: gemm_tc_pair_kernel, persistent CTA pairs (cta_group::2, one MMA of 256
// rows x 256 tokens per pair and accumulator, K streamed over the pairs). Up to 256 tokens (and the few shapes the
// pair kernel leaves): gemm_tc_kernel, one CTA per 128-row x (NACC x BN)-token tile. At most 128 tokens of Q4_K:
// gemm_tc_small_kernel, tokens on the MMA's M side. In all of them a dequantised weight stage is used for every
// accumulator of the tile, so with 512 tokens per tile every weight is unpacked once per 512 tokens and tensor
// memory is fully used. Warp roles of the first two (19 warps):
//   warp 0       allocates tensor memory; lane 0 issues the tcgen05.mma and commits of accumulator 0
//   warp 1       lane 0 issues the TMA loads of X; with two accumulators also those of the raw weight blocks
//   warp 2       one accumulator: lane 0 issues the TMA loads of the raw weight blocks (one 256-column block of
//                128 rows per box); two accumulators: lane 0 issues the MMAs and commits of accumulator 1
//   warps 3-18   dequantise: set j (4 warps, one thread per row) owns 64-column group j of every
//                256-column block, i.e. stage j of the bf16 weight ring; all of them also run the epilogue
// Rings: 3 raw-block slots of 18 KB (Q4_K) or 2 of 30 KB (Q6_K), 4 bf16 weight stages of 16 KB, 3 (BN = 256) or 6 (BN = 128)
// activation slots of BN x 64 bf16. Every wait on an mbarrier
// is bounded; a wait that gives up records {1, site} in the status words, raises a CTA-wide flag
// and lets every role fall through to the common exit, where tensor memory is released.
//
// Replaces the reference's mul_mm_q4k.comp / gemm_q4k.metal tile kernels
// (src/compute/dmmv.zig:1045 recordMulMmQ4K).
#include "kernels.h"
#include "tc_common.cuh"

namespace zc {
namespace {

// The persistent CTA-pair kernel takes launches of more than 256 tokens; ZC_GEMM_PAIRS=0 in the environment keeps
// them on the one-CTA-per-tile kernel (for comparisons).
const bool g_pair_mode = [] {
    const char* e = getenv("ZC_GEMM_PAIRS");
    return !(e && e[0] == '0');
}();

struct GemmArgs {
    const uint8_t* A;
    float* D;
    uint32_t M, N, K;
    uint32_t stride_d;
    uint32_t* status;
};

template <int TYPE, int BN, int NACC>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_w,
                   const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // swizzle atoms: 1024-byte aligned
    uint8_t* smem_b = smem + Tile<TYPE, BN>::kBOffset;
    uint8_t* smem_w = smem + Tile<TYPE, BN>::kWOffset;
    constexpr int kBSlots = Tile<TYPE, BN>::kBSlots;
    constexpr uint32_t kBSlotBytes = Tile<TYPE, BN>::kBBytes;
    // With an odd number of slots two issuers take the fills of a slot in turn, and a parity wait only tells the
    // current phase from the one before it: a thread that waited on a barrier it visits every other phase could
    // not tell "not filled yet" from "filled twice since". Such a slot has two "full" barriers, used by its even
    // and odd fills: each is then waited on by one thread only, phase after phase. With an even number of slots
    // every slot belongs to one issuer.
    constexpr int kFullSets = (NACC == 2 && kBSlots % 2 == 1) ? 2 : 1;
    static_assert(kBSlots * kFullSets <= 6, "full_b / empty_b hold six barriers");
    constexpr int kWSlots = Tile<TYPE, BN>::kWSlots;
    constexpr uint32_t kWBytes = Tile<TYPE, BN>::kWBytes;
    Bars* bars = reinterpret_cast<Bars*>(smem + Tile<TYPE, BN>::kBarOffset);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t m0 = blockIdx.x * kBM, n0 = blockIdx.y * (BN * NACC);
    // split-K: CTA z handles blocks [b_begin, b_end) of every row and adds its partial tile into D
    const int nblk_all = g.K >> 8;
    const int b_begin = (int)((long long)blockIdx.z * nblk_all / gridDim.z);
    const int b_end = (int)((long long)(blockIdx.z + 1) * nblk_all / gridDim.z);
    const int n_it = (b_end - b_begin) * 4;
    const int it0 = b_begin * 4;
    // accumulators of this tile that hold at least one real token
    const int nacc = min(NACC, (int)((g.N - n0 + BN - 1) / BN));
    const int n_iss = NACC == 1 ? 1 : nacc;  // issuing threads at work: one per accumulator in use

    if (tid == 0) {
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&bars->full_a[s], 4);  // one arrival per producer warp of the owning set
            mbar_init(&bars->empty_a[s], n_iss);  // one commit per issuing thread
        }
        for (int s = 0; s < kBSlots; ++s) mbar_init(&bars->empty_b[s], 1);
        for (int s = 0; s < kBSlots * kFullSets; ++s) mbar_init(&bars->full_b[s], 1);
        for (int s = 0; s < kWSlots; ++s) {
            mbar_init(&bars->full_w[s], 1);
            mbar_init(&bars->empty_w[s], 16);  // one arrival per producer warp
        }
        mbar_init(&bars->accum, n_iss);
        bars->failed = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&bars->tmem_base)),
                     "r"((uint32_t)(BN * NACC))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0 || (NACC == 2 && warp == 2)) {
        // ---- MMA issuers: one thread per accumulator (an issue costs the thread about as many cycles as the
        // tensor core needs for half the instruction, waits and commits not counted, so one thread alone
        // cannot keep two accumulators fed); both read every weight stage, each its own activation slots ----
        const int w = warp == 0 ? 0 : 1;
        if (lane == 0 && w < n_iss) {
            constexpr uint32_t idesc = instr_desc<BN>();
            int sb = w;  // slots are used in the order (iteration, accumulator)
            uint32_t fill = 0;  // how often the ring has wrapped = the number of this slot's fill
            bool ok = true;
            for (int it = 0; it < n_it && ok; ++it) {
                const int sa = it & 3;
                ok = wait_or_fail<false>(&bars->full_a[sa], (it >> 2) & 1, bars, g.status, 101);
                const uint64_t da = smem_desc(smem_u32(smem + sa * kABytes));
                for (int acc = w; acc < nacc && ok; acc += n_iss) {
                    ok = wait_or_fail<false>(&bars->full_b[sb + kBSlots * (fill & kFullSets - 1)], (fill / kFullSets) & 1, bars,
                                             g.status, 102);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t db = smem_desc(smem_u32(smem_b + sb * kBSlotBytes));
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)  // 16 columns = 32 bytes per instruction
                        umma_bf16(tmem + acc * BN, da + 2 * k, db + 2 * k, idesc, (it | k) ? 1u : 0u);
                    umma_commit(&bars->empty_b[sb]);
                    sb += n_iss;
                    if (sb >= kBSlots) {
                        sb -= kBSlots;
                        ++fill;
                    }
                }
                if (!ok) break;
                umma_commit(&bars->empty_a[sa]);
            }
            umma_commit(&bars->accum);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- TMA loader of X and, with two accumulators (whose second issuer has the third control warp),
            // of the raw weight blocks too: polls both rings without suspending on either ----
            int sb = 0, it = 0, acc = 0;
            uint32_t pb = 1, fill = 0;
            int sw = 0, b = NACC == 2 ? b_begin : b_end;
            uint32_t pw = 1, idle = 0;
            while (it < n_it || b < b_end) {
                bool moved = false;
                if (it < n_it && mbar_test_wait(&bars->empty_b[sb], pb)) {
                    uint64_t* full = &bars->full_b[sb + kBSlots * (fill & kFullSets - 1)];
                    mbar_expect_tx(full, kBSlotBytes);
                    tma_load_2d(smem_b + sb * kBSlotBytes, &tmap_b, (it0 + it) * kBK, (int)(n0 + acc * BN), full);
                    if (++sb == kBSlots) {
                        sb = 0;
                        pb ^= 1;
                        ++fill;
                    }
                    if (++acc == nacc) {
                        acc = 0;
                        ++it;
                    }
                    moved = true;
                }
                if (NACC == 2 && b < b_end && mbar_test_wait(&bars->empty_w[sw], pw)) {
                    mbar_expect_tx(&bars->full_w[sw], kWBytes);
                    tma_load_2d(smem_w + sw * kWBytes, &tmap_w, (int)((b * Raw<TYPE>::kBlock) & ~15u), (int)m0,
                                &bars->full_w[sw]);
                    if (++sw == kWSlots) {
                        sw = 0;
                        pw ^= 1;
                    }
                    ++b;
                    moved = true;
                }
                if (moved) {
                    idle = 0;
                } else {  // bounded like every other wait
                    __nanosleep(32);
                    ++idle;
                    if ((idle & 63u) == 63u && bars->failed) break;
                    if (idle >= kWaitLimit) {
                        bars->failed = 1;
                        if (g.status) {
                            g.status[0] = 1;
                            g.status[1] = 103;
                        }
                        break;
                    }
                }
            }
        }
    } else if (NACC == 1 && warp == 2) {
        if (lane == 0) {  // ---- TMA loader of the raw weight blocks ----
            int sw = 0;
            uint32_t pw = 1;
            for (int b = b_begin; b < b_end; ++b) {
                if (!wait_or_fail(&bars->empty_w[sw], pw, bars, g.status, 106)) break;
                mbar_expect_tx(&bars->full_w[sw], kWBytes);
                tma_load_2d(smem_w + sw * kWBytes, &tmap_w, (int)((b * Raw<TYPE>::kBlock) & ~15u), (int)m0,
                            &bars->full_w[sw]);
                if (++sw == kWSlots) {
                    sw = 0;
                    pw ^= 1;
                }
            }
        }
    } else {
        // ---- dequant producers: thread = one row; set j owns group j of every block = weight stage j ----
        const int p = tid - kCtlWarps * 32;  // with three control warps the quarters come in the order 3, 0, 1, 2
        const int row = p & 127, j = p >> 7;
        uint8_t* a_stage = smem + j * kABytes;
        int sw = 0;
        uint32_t pw = 0;
        for (int b = b_begin; b < b_end; ++b) {
            if (!wait_or_fail(&bars->full_w[sw], pw, bars, g.status, 107)) break;
            if constexpr (TYPE == T_Q4_K) {
                const uint8_t* wp = smem_w + sw * kWBytes + row * 144;  // rows past M arrive as zeros
                const uint4 chdr = *reinterpret_cast<const uint4*>(wp);
                const uint4 c0 = *reinterpret_cast<const uint4*>(wp + 16 + j * 32);
                const uint4 c1 = *reinterpret_cast<const uint4*>(wp + 32 + j * 32);
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->empty_w[sw]);
                const __half2 dd = *reinterpret_cast<const __half2*>(&chdr.x);
                const float d = __low2float(dd), dmin = __high2float(dd);
                uint32_t s0, mn0, s1, mn1;
                scale_min_k4(2 * j, chdr.y, chdr.z, chdr.w, s0, mn0);
                scale_min_k4(2 * j + 1, chdr.y, chdr.z, chdr.w, s1, mn1);
                if (!wait_or_fail(&bars->empty_a[j], ((b - b_begin) & 1) ^ 1, bars, g.status, 104)) break;
                dequant_group_q4k(c0, c1, d * (float)s0, dmin * (float)mn0, d * (float)s1, dmin * (float)mn1,
                                  a_stage, row);
            } else {
                // the block starts (b * 210) & 15 bytes into the box; that offset is even
                const uint32_t off = ((uint32_t)b * 210u) & 15u;
                const uint8_t* wp = smem_w + sw * kWBytes + row * 240 + (off & ~3u);
                if (!wait_or_fail(&bars->empty_a[j], ((b - b_begin) & 1) ^ 1, bars, g.status, 104)) break;
                dequant_group_q6k(reinterpret_cast<const uint32_t*>(wp), (off & 2u) * 8u, j, a_stage, row);
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->empty_w[sw]);
            }
            if (++sw == kWSlots) {
                sw = 0;
                pw ^= 1;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->full_a[j]);
        }
        // ---- epilogue: all sixteen producer warps (the stores take the time: the more in flight the better);
        // TMEM lane quarter = warp % 4, set j takes the column chunks c = j mod 4 ----
        {
            if (wait_or_fail(&bars->accum, 0, bars, g.status, 105)) {
                __syncwarp();
                tc_fence_after();
                const uint32_t q = warp & 3;
                const uint32_t m = m0 + q * 32 + lane;
#pragma unroll 1
                for (int c = j; c < nacc * (BN / 32); c += 4) {
                    uint32_t v[32];
                    const uint32_t taddr = tmem + ((q * 32u) << 16) + c * 32;
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
                        for (int jj = 0; jj < 32; ++jj) {
                            const uint32_t n = n0 + c * 32 + jj;
                            if (n < g.N) {
                                float* dst = g.D + (uint64_t)n * g.stride_d + m;
                                if (gridDim.z == 1)
                                    *dst = __uint_as_float(v[jj]);
                                else
                                    atomicAdd(dst, __uint_as_float(v[jj]));
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(BN * NACC))
                     : "memory");
    }
}

// ---- CTA pairs, persistent, K streamed over the pairs ------------------------------------------------------
// Tiles of 256 weight rows (128 per CTA of a pair) x 512 tokens (two accumulators). Their (tile, 256-column
// block) units, tile-major, are dealt in contiguous ranges to as many pairs as the GPU holds at once, so every
// pair has the same amount of work whatever the tile count: a pair works through a list of segments (tile, block
// range), all rings running on across segment boundaries. A tile whose blocks are split over pairs is finished
// through memory: the pair with the tile's last blocks (always the first segment of its range, so nobody waits
// long for it) stores its partial sums and raises the tile's flag; the others add theirs once the flag is up.
struct PairArgs {
    GemmArgs g;
    uint32_t* flags;  // [tile][CTA rank]: number of epilogue warps (of 16) of the storing CTA that are done; zero at launch
    uint32_t n_row_pairs, n_tiles;
    const uint8_t* a_end;  // MXFP4: first byte past the matrix (its rows are fetched as 16-byte aligned supersets)
    uint32_t zeroed;       // D was zeroed before the launch: the parts of a split tile all add, without an order
};

struct Segment {
    uint32_t tile, b0, b1;
};
__device__ __forceinline__ bool next_segment(uint32_t& u, uint32_t u1, uint32_t nblk, Segment& sg) {
    if (u >= u1) return false;
    sg.tile = u / nblk;
    sg.b0 = u - sg.tile * nblk;
    sg.b1 = min(nblk, sg.b0 + (u1 - u));
    u += sg.b1 - sg.b0;
    return true;
}

constexpr uint32_t kFlagSpinLimit = 1u << 21;

// kFetch: the dequant threads copy the raw blocks themselves (rows a tensor map cannot describe: MXFP4 always, Q6_K
// when the row pitch is not a multiple of 16 bytes); else one thread fetches them as TMA boxes.
template <int TYPE, bool kFetch = TYPE == T_MXFP4>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_w,
                    const PairArgs p) {
    static_assert(TYPE != T_MXFP4 || kFetch, "MXFP4 rows have no tensor map");
    static_assert(TYPE != T_Q4_K || !kFetch, "Q4_K rows always have a 16-byte pitch");
    constexpr int BN = 256, NACC = 2;
    using T = Tile<TYPE, BN>;
    // A CTA's activation slot holds 256 consecutive tokens, n0 + 256 * rank ..: its first 128 are this CTA's half
    // of accumulator 0's operand, the other 128 of accumulator 1's, so one copy per 64-column step feeds both.
    // Accumulator a therefore holds the tokens n0 + 128 a .. (columns 0..127) and n0 + 256 + 128 a .. (128..255).
    constexpr int kRing = T::kBSlots;
    constexpr uint32_t kBSlotBytes = T::kBBytes;
    constexpr int kWSlots = T::kWSlots;
    constexpr uint32_t kWBytes = T::kWBytes;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* smem_b = smem + T::kBOffset;
    uint8_t* smem_w = smem + T::kWOffset;
    Bars* bars = reinterpret_cast<Bars*>(smem + T::kBarOffset);
    const GemmArgs& g = p.g;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    // MXFP4: K is a multiple of 64 only; the columns past K of the last 256-column block are zeros on both sides
    // (the dequant warps write zero rows, the activation boxes past K are filled with zeros by the copy engine)
    const uint32_t nblk = TYPE == T_MXFP4 ? (g.K + 255) >> 8 : g.K >> 8;
    const uint32_t U = p.n_tiles * nblk, G = gridDim.x >> 1, slot = blockIdx.x >> 1;
    const uint32_t u_begin = (uint32_t)part_begin(slot, U, G), u_end = (uint32_t)part_begin(slot + 1, U, G);
    auto tile_m0 = [&](uint32_t tile) { return ((tile % p.n_row_pairs) * 2 + rank) * (uint32_t)kBM; };
    auto tile_n0 = [&](uint32_t tile) { return (tile / p.n_row_pairs) * (uint32_t)(BN * NACC); };
    // accumulators with at least one real token
    auto tile_nacc = [&](uint32_t tile) { return g.N - tile_n0(tile) > (uint32_t)(BN / 2) ? 2 : 1; };

    if (tid == 0) {
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&bars->full_a[s], 8);   // one arrival per producer warp of the owning set, both CTAs
            mbar_init(&bars->empty_a[s], NACC);  // one commit per issuing thread
        }
        for (int s = 0; s < kRing; ++s) {
            mbar_init(&bars->full_b[s], 2);      // one loader per CTA
            mbar_init(&bars->empty_b[s], NACC);  // one commit per issuing thread
        }
        for (int s = 0; s < kWSlots; ++s) {
            // filled by one TMA box, or (MXFP4) by the 512 dequant threads, whose copies report by themselves
            mbar_init(&bars->full_w[s], kFetch ? 512 : 1);
            mbar_init(&bars->empty_w[s], 16);  // one arrival per producer warp
        }
        mbar_init(&bars->accum, NACC);
        mbar_init(&bars->tmem_free, 32);     // the sixteen epilogue warps of both CTAs
        bars->failed = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                     "r"((uint32_t)(BN * NACC))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0 || warp == 2) {
        // ---- MMA issuers (even CTA): one thread per accumulator. A thread whose accumulator lies past the last
        // token of a tile still takes part in every hand-off (its commits follow no MMA and arrive at once). ----
        const int w = warp == 0 ? 0 : 1;
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = instr_desc_pair<BN>();
            uint32_t git = 0, fill = 0, seg_i = 0, u = u_begin;
            int sb = 0;
            bool ok = true;
            Segment sg;
            while (ok && next_segment(u, u_end, nblk, sg)) {
                const bool live = w < tile_nacc(sg.tile);
                if (seg_i > 0) {  // the epilogue has read the previous segment's sums out of tensor memory
                    ok = wait_or_fail<false>(&bars->tmem_free, (seg_i - 1) & 1, bars, g.status, 109);
                    if (!ok) break;
                    tc_fence_after();
                }
                const int n_it = (int)(sg.b1 - sg.b0) * 4;
                for (int it = 0; it < n_it; ++it, ++git) {
                    const int sa = git & 3;
                    ok = wait_or_fail<false>(&bars->full_a[sa], (git >> 2) & 1, bars, g.status, 101);
                    if (!ok) break;
                    ok = wait_or_fail<false>(&bars->full_b[sb], fill & 1, bars, g.status, 102);
                    if (!ok) break;
                    if (live) {
                        tc_fence_after();
                        const uint64_t da = smem_desc(smem_u32(smem + sa * kABytes));
                        const uint64_t db = smem_desc(smem_u32(smem_b + sb * kBSlotBytes + w * (kBSlotBytes / 2)));
#pragma unroll
                        for (int k = 0; k < kBK / 16; ++k)
                            umma_bf16_pair(tmem + w * BN, da + 2 * k, db + 2 * k, idesc, (it | k) ? 1u : 0u);
                    }
                    umma_commit_pair(&bars->empty_b[sb]);
                    if (++sb == kRing) {
                        sb = 0;
                        ++fill;
                    }
                    umma_commit_pair(&bars->empty_a[sa]);
                }
                if (!ok) break;
                umma_commit_pair(&bars->accum);
                ++seg_i;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- loader of both rings (each CTA its own half of the activation boxes and its own weight rows):
            // polls without suspending on either ----
            uint32_t ub = u_begin, uw = u_begin;
            Segment sb_seg, sw_seg;
            bool b_live = next_segment(ub, u_end, nblk, sb_seg);
            bool w_live = !kFetch && next_segment(uw, u_end, nblk, sw_seg);
            uint32_t b_it = 0;                   // 64-column step inside the activation segment
            uint32_t w_b = w_live ? sw_seg.b0 : 0;
            // per segment (the divisions stay out of the per-copy path)
            uint32_t b_n0 = 0, b_k0 = 0, b_nit = 0, w_m0 = 0;
            auto b_enter = [&]() {
                b_n0 = tile_n0(sb_seg.tile) + rank * BN;
                b_k0 = sb_seg.b0 * 4;
                b_nit = (sb_seg.b1 - sb_seg.b0) * 4;
            };
            if (b_live) b_enter();
            if (w_live) w_m0 = tile_m0(sw_seg.tile);
            int sbl = 0, sw = 0;
            uint32_t pbl = 1, pw = 1, idle = 0;
            while (b_live || w_live) {
                bool moved = false;
                if (b_live && mbar_test_wait(&bars->empty_b[sbl], pbl)) {
                    const uint32_t fb = leader_addr(&bars->full_b[sbl]);
                    mbar_expect_tx_cluster(fb, kBSlotBytes);
                    tma_load_2d_pair(smem_b + sbl * kBSlotBytes, &tmap_b, (int)((b_k0 + b_it) * kBK), (int)b_n0, fb);
                    if (++sbl == kRing) {
                        sbl = 0;
                        pbl ^= 1;
                    }
                    if (++b_it == b_nit) {
                        b_it = 0;
                        b_live = next_segment(ub, u_end, nblk, sb_seg);
                        if (b_live) b_enter();
                    }
                    moved = true;
                }
                if (w_live && mbar_test_wait(&bars->empty_w[sw], pw)) {
                    mbar_expect_tx(&bars->full_w[sw], kWBytes);
                    tma_load_2d(smem_w + sw * kWBytes, &tmap_w, (int)((w_b * Raw<TYPE>::kBlock) & ~15u),
                                (int)w_m0, &bars->full_w[sw]);
                    if (++sw == kWSlots) {
                        sw = 0;
                        pw ^= 1;
                    }
                    if (++w_b == sw_seg.b1) {
                        w_live = next_segment(uw, u_end, nblk, sw_seg);
                        w_b = sw_seg.b0;
                        if (w_live) w_m0 = tile_m0(sw_seg.tile);
                    }
                    moved = true;
                }
                if (moved) {
                    idle = 0;
                } else {  // bounded like every other wait
                    __nanosleep(32);
                    ++idle;
                    if ((idle & 63u) == 63u && bars->failed) break;
                    if (idle >= kWaitLimit) {
                        bars->failed = 1;
                        if (g.status) {
                            g.status[0] = 1;
                            g.status[1] = 103;
                        }
                        break;
                    }
                }
            }
        }
    } else {
        // ---- dequant producers: thread = one row; set j owns group j of every block = weight stage j ----
        const int pi = tid - kCtlWarps * 32;
        const int row = pi & 127, j = pi >> 7;
        uint8_t* a_stage = smem + j * kABytes;
        const uint32_t full_a_leader = leader_addr(&bars->full_a[j]);
        const uint32_t free_leader = leader_addr(&bars->tmem_free);
        int sw = 0;
        uint32_t pw = 0, gb = 0, seg_i = 0, u = u_begin;
        bool ok = true;
        Segment sg;
        // kFetch: the dequant threads fetch the raw blocks themselves, one ring slot (a block) ahead: thread (row, j)
        // copies the 16-byte pieces j, j + 4, ... of the aligned superset of its row's block (136 or 210 bytes)
        constexpr uint32_t kRawBlock = Raw<TYPE>::kBlock, kRawRow = Raw<TYPE>::kBox;
        constexpr int kRawPieces = TYPE == T_MXFP4 ? 10 : 15;  // (15 + block bytes) / 16 rounded up
        const uint64_t mx_row_bytes = TYPE == T_MXFP4 ? (uint64_t)(g.K >> 5) * 17u : (uint64_t)(g.K >> 8) * kRawBlock;
        uint32_t uf = u_begin, f_b = 0, f_pw = 1;
        int f_sw = 0;
        Segment f_seg{0, 0, 0};
        bool f_live = false;
        uint64_t f_row_off = 0, c_row_off = 0;
        auto mx_row_off = [&](uint32_t tile) {
            return (uint64_t)min(tile_m0(tile) + (uint32_t)row, g.M - 1) * mx_row_bytes;  // rows past M: computed, dropped
        };
        auto mx_fetch = [&]() -> bool {
            if (!f_live) return true;
            if (!wait_or_fail(&bars->empty_w[f_sw], f_pw, bars, g.status, 111)) return false;
            const uint64_t o = f_row_off + (uint64_t)f_b * kRawBlock;
            const uint8_t* src = g.A + (o & ~(uint64_t)15);
            uint8_t* dst = smem_w + f_sw * kWBytes + row * kRawRow;
#pragma unroll
            for (int pc = 0; pc < 16; pc += 4) {
                const int piece = pc + j;
                if (piece < kRawPieces) {
                    const uint8_t* sp = src + piece * 16;
                    const uint32_t nbytes = sp + 16 <= p.a_end ? 16u : (sp < p.a_end ? (uint32_t)(p.a_end - sp) : 0u);
                    cp_async16_zfill(dst + piece * 16, nbytes ? sp : g.A, nbytes);
                }
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bars->full_w[f_sw])) : "memory");
            if (++f_sw == kWSlots) {
                f_sw = 0;
                f_pw ^= 1;
            }
            if (++f_b == f_seg.b1) {
                f_live = next_segment(uf, u_end, nblk, f_seg);
                f_b = f_seg.b0;
                if (f_live) f_row_off = mx_row_off(f_seg.tile);
            }
            return true;
        };
        if constexpr (kFetch) {
            f_live = next_segment(uf, u_end, nblk, f_seg);
            f_b = f_seg.b0;
            if (f_live) f_row_off = mx_row_off(f_seg.tile);
            for (int d = 0; d < kWSlots - 1 && ok; ++d) ok = mx_fetch();
        }
        while (ok && next_segment(u, u_end, nblk, sg)) {
            if constexpr (kFetch) c_row_off = mx_row_off(sg.tile);
            for (uint32_t b = sg.b0; b < sg.b1; ++b, ++gb) {
                if (!wait_or_fail(&bars->full_w[sw], pw, bars, g.status, 107)) { ok = false; break; }
                if constexpr (kFetch) {
                    if (!mx_fetch()) { ok = false; break; }  // the next block, into the slot the previous one left
                }
                if constexpr (TYPE == T_MXFP4) {
                    if (!wait_or_fail(&bars->empty_a[j], (gb & 1) ^ 1, bars, g.status, 104)) { ok = false; break; }
                    if (4 * b + (uint32_t)j < (g.K >> 6)) {
                        const uint32_t off = (uint32_t)((c_row_off + (uint64_t)b * 136u) & 15u) + 34u * (uint32_t)j;
                        const uint8_t* wp = smem_w + sw * kWBytes + row * 176;
                        dequant_group_mxfp4(reinterpret_cast<const uint32_t*>(wp + (off & ~3u)), (off & 3u) * 8u, a_stage, row);
                    } else {  // past K: a zero row (the swizzle permutes 16-byte chunks of zeros)
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<uint4*>(a_stage + row * 128 + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->empty_w[sw]);
                } else if constexpr (TYPE == T_Q4_K) {
                    const uint8_t* wp = smem_w + sw * kWBytes + row * 144;  // rows past M arrive as zeros
                    const uint4 chdr = *reinterpret_cast<const uint4*>(wp);
                    const uint4 c0 = *reinterpret_cast<const uint4*>(wp + 16 + j * 32);
                    const uint4 c1 = *reinterpret_cast<const uint4*>(wp + 32 + j * 32);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->empty_w[sw]);
                    const __half2 dd = *reinterpret_cast<const __half2*>(&chdr.x);
                    const float d = __low2float(dd), dmin = __high2float(dd);
                    uint32_t s0, mn0, s1, mn1;
                    scale_min_k4(2 * j, chdr.y, chdr.z, chdr.w, s0, mn0);
                    scale_min_k4(2 * j + 1, chdr.y, chdr.z, chdr.w, s1, mn1);
                    if (!wait_or_fail(&bars->empty_a[j], (gb & 1) ^ 1, bars, g.status, 104)) { ok = false; break; }
                    dequant_group_q4k(c0, c1, d * (float)s0, dmin * (float)mn0, d * (float)s1, dmin * (float)mn1, a_stage,
                                      row);
                } else {
                    // the block starts `off` bytes into the box or (fetched by the threads) into the row's aligned
                    // superset; that offset is even
                    const uint32_t off = kFetch ? (uint32_t)((c_row_off + (uint64_t)b * 210u) & 15u) : (b * 210u) & 15u;
                    const uint8_t* wp = smem_w + sw * kWBytes + row * 240 + (off & ~3u);
                    if (!wait_or_fail(&bars->empty_a[j], (gb & 1) ^ 1, bars, g.status, 104)) { ok = false; break; }
                    dequant_group_q6k(reinterpret_cast<const uint32_t*>(wp), (off & 2u) * 8u, j, a_stage, row);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->empty_w[sw]);
                }
                if (++sw == kWSlots) {
                    sw = 0;
                    pw ^= 1;
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(full_a_leader);
            }
            if (!ok) break;
            // ---- epilogue of the segment: all sixteen producer warps (the stores, not the tensor memory reads, take
            // the time: the more in flight the better). TMEM lane quarter = warp % 4; set j takes the column chunks
            // c = j mod 4. ----
            {
                if (!wait_or_fail(&bars->accum, seg_i & 1, bars, g.status, 105)) { ok = false; break; }
                __syncwarp();
                tc_fence_after();
                // A tile split over pairs. Long ranges (flags): the pair with the tile's last blocks stores, the others add
                // once its flag is up. Short ranges (D zeroed before the launch): every part adds, nobody waits.
                const bool whole = sg.b0 == 0 && sg.b1 == nblk;
                const bool store = p.zeroed ? whole : sg.b1 == nblk;
                uint32_t* flag = p.flags + 2 * sg.tile + rank;
                bool go = true;
                if (!store && !p.zeroed) {
                    if (lane == 0) {
                        uint32_t n = 0;
                        while (ld_acquire_u32(flag) < 16u) {
                            __nanosleep(64);
                            if (++n >= kFlagSpinLimit || ((n & 63u) == 63u && bars->failed)) {
                                bars->failed = 1;
                                if (g.status) {
                                    g.status[0] = 1;
                                    g.status[1] = 110;
                                }
                                go = false;
                                break;
                            }
                        }
                    }
                    go = __shfl_sync(0xFFFFFFFFu, go ? 1 : 0, 0) != 0;
                }
                const uint32_t q = warp & 3;
                const uint32_t m = tile_m0(sg.tile) + q * 32 + lane, n0 = tile_n0(sg.tile);
                // this warp's chunks j, j + 4 (accumulator 0) and j + 8, j + 12 (accumulator 1), two reads in flight;
                // columns 32 c .. of tensor memory are accumulator c / 8, its columns 32 (c % 8) ..
                auto first_token = [&](int c) {
                    const uint32_t col = (uint32_t)(c & 7) * 32u;
                    return n0 + (uint32_t)(c >> 3) * (BN / 2) + col + (col >= (uint32_t)(BN / 2) ? BN / 2 : 0);
                };
                auto put = [&](uint32_t nc, const uint32_t (&v)[32]) {
                    if (m < g.M && go && nc < g.N) {
#pragma unroll
                        for (int jj = 0; jj < 32; ++jj) {
                            const uint32_t n = nc + jj;
                            if (n < g.N) {
                                float* dst = g.D + (uint64_t)n * g.stride_d + m;
                                if (store)
                                    *dst = __uint_as_float(v[jj]);
                                else
                                    atomicAdd(dst, __uint_as_float(v[jj]));
                            }
                        }
                    }
                };
#pragma unroll 1
                for (int c = j; c < NACC * (BN / 32); c += 8) {
                    const uint32_t na = first_token(c), nb = first_token(c + 4);
                    if (na >= g.N && nb >= g.N) continue;  // no real token (an accumulator nobody fed holds stale sums)
                    uint32_t va[32], vb[32];
                    tmem_ld32(tmem + ((q * 32u) << 16) + c * 32, va);
                    tmem_ld32(tmem + ((q * 32u) << 16) + (c + 4) * 32, vb);
                    tmem_ld_wait();
                    put(na, va);
                    put(nb, vb);
                }
                // tensor memory is free for the next segment
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(free_leader);
                if (store && sg.b0 > 0 && !p.zeroed) {  // others add to this tile: publish the stores
                    __threadfence();
                    __syncwarp();
                    if (lane == 0) atomicAdd(flag, 1u);
                }
            }
            ++seg_i;
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's MMAs read this CTA's stages, its commits arrive here
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(BN * NACC)) : "memory");
    }
}

// ---- few tokens (N <= 128): tokens on the TMEM lanes, weight rows on the columns ------------------------
// With at most 128 tokens a 128-row x 128-token tile issues tcgen05.mma with N = 128, and the issuing
// thread (about 73 cycles per instruction) cannot keep up with 64-cycle instructions. Here the roles are
// swapped: the MMA's M operand is the activation tile (128 tokens x 64 columns, TMA), its N operand the
// dequantised weights (256 rows x 64 columns per stage), so every instruction is a full 128 x 256 x 16.
// Q4_K only; weights are read straight from global memory into registers one block ahead (no raw
// staging ring: the 32 KB weight stages need the room); split K over up to 8 CTAs per tile.
constexpr int kSmRows = 256;                                   // weight rows per tile = accumulator columns
constexpr uint32_t kSmWBytes = kSmRows * kBK * 2;              // 32 KB per weight stage
constexpr uint32_t kSmXBytes = 128 * kBK * 2;                  // 16 KB per activation stage
constexpr int kSmXSlots = 4;
constexpr uint32_t kSmXOffset = kAStages * kSmWBytes;
constexpr uint32_t kSmBarOffset = kSmXOffset + kSmXSlots * kSmXBytes;
constexpr uint32_t kSmSmemBytes = kSmBarOffset + 256 + 1024;
constexpr int kSmThreads = 64 + 512;                           // MMA warp, TMA warp, 16 dequant warps

__global__ void __launch_bounds__(kSmThreads, 1)
gemm_tc_small_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* smem_x = smem + kSmXOffset;
    Bars* bars = reinterpret_cast<Bars*>(smem + kSmBarOffset);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t m0 = blockIdx.x * kSmRows, n0 = blockIdx.y * 128;
    const int nblk_all = g.K >> 8;
    const int b_begin = (int)((long long)blockIdx.z * nblk_all / gridDim.z);
    const int b_end = (int)((long long)(blockIdx.z + 1) * nblk_all / gridDim.z);
    const int n_it = (b_end - b_begin) * 4;

    if (tid == 0) {
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&bars->full_a[s], 9);   // one arrival per warp of the owning half + the activation box (TMA)
            mbar_init(&bars->empty_a[s], 1);
        }
        mbar_init(&bars->accum, 1);
        bars->failed = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&bars->tmem_base)),
                     "r"((uint32_t)kSmRows)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        if (lane == 0) {  // ---- MMA issuer: activation stage it & 3, weight stage it & 3 ----
            constexpr uint32_t idesc = instr_desc<kSmRows>();  // M = 128 tokens, N = 256 weight rows
            bool ok = true;
            for (int it = 0; it < n_it && ok; ++it) {
                const int st = it & 3;
                const uint32_t ph = (it >> 2) & 1;
                ok = wait_or_fail<false>(&bars->full_a[st], ph, bars, g.status, 111);  // weights and activations
                if (!ok) break;
                tc_fence_after();
                const uint64_t dx = smem_desc(smem_u32(smem_x + st * kSmXBytes));
                const uint64_t dw = smem_desc(smem_u32(smem + st * kSmWBytes));
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k) umma_bf16(tmem, dx + 2 * k, dw + 2 * k, idesc, (it | k) ? 1u : 0u);
                umma_commit(&bars->empty_a[st]);  // frees the weight stage and the activation slot
            }
            umma_commit(&bars->accum);
        }
    } else if (warp == 1) {
        if (lane == 0) {  // ---- TMA loader of the activations ----
            for (int it = 0; it < n_it; ++it) {
                const int st = it & 3;
                if (!wait_or_fail(&bars->empty_a[st], ((it >> 2) & 1) ^ 1, bars, g.status, 113)) break;
                mbar_expect_tx(&bars->full_a[st], kSmXBytes);
                tma_load_2d(smem_x + st * kSmXBytes, &tmap_x, (b_begin * 4 + it) * kBK, (int)n0, &bars->full_a[st]);
            }
        }
    } else {
        // ---- dequant producers: thread = (row, half); half h owns groups h and h + 2 of every block ----
        const int p = tid - 64;
        const int row = p & 255, h = p >> 8;
        const uint32_t grow = min(m0 + (uint32_t)row, g.M - 1);  // rows past M are computed and dropped
        const uint8_t* rp = g.A + (uint64_t)grow * nblk_all * 144u + (uint64_t)b_begin * 144u;
        uint4 hdr = __ldg(reinterpret_cast<const uint4*>(rp));
        uint4 qa0 = __ldg(reinterpret_cast<const uint4*>(rp + 16 + h * 32));
        uint4 qa1 = __ldg(reinterpret_cast<const uint4*>(rp + 32 + h * 32));
        uint4 qb0 = __ldg(reinterpret_cast<const uint4*>(rp + 80 + h * 32));
        uint4 qb1 = __ldg(reinterpret_cast<const uint4*>(rp + 96 + h * 32));
        bool ok = true;
        for (int b = 0; b < b_end - b_begin && ok; ++b) {
            const uint4 chdr = hdr, ca0 = qa0, ca1 = qa1, cb0 = qb0, cb1 = qb1;
            if (b + 1 < b_end - b_begin) {
                const uint8_t* np = rp + (uint64_t)(b + 1) * 144u;
                hdr = __ldg(reinterpret_cast<const uint4*>(np));
                qa0 = __ldg(reinterpret_cast<const uint4*>(np + 16 + h * 32));
                qa1 = __ldg(reinterpret_cast<const uint4*>(np + 32 + h * 32));
                qb0 = __ldg(reinterpret_cast<const uint4*>(np + 80 + h * 32));
                qb1 = __ldg(reinterpret_cast<const uint4*>(np + 96 + h * 32));
            }
            const __half2 dd = *reinterpret_cast<const __half2*>(&chdr.x);
            const float d = __low2float(dd), dmin = __high2float(dd);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                const int grp = h + 2 * half;
                uint32_t s0, mn0, s1, mn1;
                scale_min_k4(2 * grp, chdr.y, chdr.z, chdr.w, s0, mn0);
                scale_min_k4(2 * grp + 1, chdr.y, chdr.z, chdr.w, s1, mn1);
                if (!wait_or_fail(&bars->empty_a[grp], (b & 1) ^ 1, bars, g.status, 114)) {
                    ok = false;
                    break;
                }
                dequant_group_q4k(half ? cb0 : ca0, half ? cb1 : ca1, d * (float)s0, dmin * (float)mn0, d * (float)s1,
                                  dmin * (float)mn1, smem + grp * kSmWBytes, row);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->full_a[grp]);
            }
        }
        // ---- epilogue: all sixteen producer warps, TMEM lane quarter = warp % 4, each group of four warps its own
        // column chunks; a lane is a token, columns are rows ----
        {
            if (wait_or_fail(&bars->accum, 0, bars, g.status, 115)) {
                __syncwarp();
                tc_fence_after();
                const uint32_t q = warp & 3;
                const uint32_t n = n0 + q * 32 + lane;
#pragma unroll 1
                for (int c = (warp - 2) >> 2; c < kSmRows / 32; c += 4) {
                    uint32_t v[32];
                    const uint32_t taddr = tmem + ((q * 32u) << 16) + c * 32;
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
                    if (n < g.N) {
                        float* dst = g.D + (uint64_t)n * g.stride_d + m0 + c * 32;
                        const bool vec = m0 + c * 32 + 32 <= g.M && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
                        if (vec) {  // 32 consecutive rows of one token: 16-byte stores / vector reductions
#pragma unroll
                            for (int jj = 0; jj < 32; jj += 4) {
                                const float4 f = make_float4(__uint_as_float(v[jj]), __uint_as_float(v[jj + 1]),
                                                             __uint_as_float(v[jj + 2]), __uint_as_float(v[jj + 3]));
                                if (gridDim.z == 1)
                                    *reinterpret_cast<float4*>(dst + jj) = f;
                                else
                                    atomicAdd(reinterpret_cast<float4*>(dst + jj), f);
                            }
                        } else {
#pragma unroll
                            for (int jj = 0; jj < 32; ++jj) {
                                if (m0 + c * 32 + jj < g.M) {
                                    if (gridDim.z == 1)
                                        dst[jj] = __uint_as_float(v[jj]);
                                    else
                                        atomicAdd(dst + jj, __uint_as_float(v[jj]));
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kSmRows)
                     : "memory");
    }
}

template <int TYPE, int BN, int NACC>
cudaError_t launch_tile(const uint8_t* A, const void* B, float* D, uint32_t M, uint32_t N, uint32_t K,
                        uint32_t stride_b, uint32_t stride_d, uint32_t* status, cudaStream_t s) {
    EncodeFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap map;
    const cuuint64_t dims[2] = {K, N};
    const cuuint64_t strides[1] = {(cuuint64_t)stride_b * 2};
    const cuuint32_t box[2] = {kBK, BN};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(B), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    // raw weight bytes as a 2-D byte tensor [M][row_bytes]; a box holds one block of 128 rows
    CUtensorMap wmap;
    const cuuint64_t row_bytes = (cuuint64_t)(K >> 8) * Raw<TYPE>::kBlock;
    const cuuint64_t wdims[2] = {row_bytes, M};
    const cuuint64_t wstrides[1] = {row_bytes};
    const cuuint32_t wbox[2] = {Raw<TYPE>::kBox, kBM};
    if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(A), wdims, wstrides, wbox, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    auto kern = gemm_tc_kernel<TYPE, BN, NACC>;
    static std::atomic<uint64_t> attr_done{0};  // per device ordinal
    if (cudaError_t ea = ensure_dynamic_smem(kern, (int)Tile<TYPE, BN>::kSmemBytes, attr_done); ea != cudaSuccess) return ea;
    GemmArgs g{A, D, M, N, K, stride_d, status};
    dim3 grid((M + kBM - 1) / kBM, (N + BN * NACC - 1) / (BN * NACC), 1);
    // Few tiles (short M or few tokens): split K over up to 8 CTAs per tile, at least 4 blocks each, and
    // let the partial tiles add into a zeroed D.
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint32_t tiles = grid.x * grid.y;
    uint32_t splits = tiles ? (uint32_t)sms / tiles : 1;
    splits = splits < 1 ? 1 : (splits > 8 ? 8 : splits);
    while (splits > 1 && (K >> 8) / splits < 4) --splits;
    if (splits > 1) {
        cudaError_t e = cudaMemset2DAsync(D, (size_t)stride_d * 4, 0, (size_t)M * 4, N, s);
        if (e != cudaSuccess) return e;
        grid.z = splits;
    }
    kern<<<grid, kThreads, Tile<TYPE, BN>::kSmemBytes, s>>>(map, wmap, g);
    return cudaGetLastError();
}

cudaError_t launch_small(const uint8_t* A, const void* B, float* D, uint32_t M, uint32_t N, uint32_t K,
                         uint32_t stride_b, uint32_t stride_d, uint32_t* status, cudaStream_t s) {
    EncodeFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    CUtensorMap map;
    const cuuint64_t dims[2] = {K, N};
    const cuuint64_t strides[1] = {(cuuint64_t)stride_b * 2};
    const cuuint32_t box[2] = {kBK, 128};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(B), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    static std::atomic<uint64_t> attr_done{0};  // per device ordinal
    if (cudaError_t ea = ensure_dynamic_smem(gemm_tc_small_kernel, (int)kSmSmemBytes, attr_done); ea != cudaSuccess) return ea;
    GemmArgs g{A, D, M, N, K, stride_d, status};
    dim3 grid((M + kSmRows - 1) / kSmRows, (N + 127) / 128, 1);
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint32_t tiles = grid.x * grid.y;
    uint32_t splits = tiles ? (uint32_t)sms / tiles : 1;
    splits = splits < 1 ? 1 : (splits > 8 ? 8 : splits);
    while (splits > 1 && (K >> 8) / splits < 2) --splits;
    if (splits > 1) {
        cudaError_t e = cudaMemset2DAsync(D, (size_t)stride_d * 4, 0, (size_t)M * 4, N, s);
        if (e != cudaSuccess) return e;
        grid.z = splits;
    }
    gemm_tc_small_kernel<<<grid, kSmThreads, kSmSmemBytes, s>>>(map, g);
    return cudaGetLastError();
}

// The persistent pair kernel. cudaErrorNotSupported: the caller takes another path (nothing launched or written).
template <int TYPE, bool kFetch = TYPE == T_MXFP4>
cudaError_t launch_pair(const uint8_t* A, const void* B, float* D, uint32_t M, uint32_t N, uint32_t K, uint32_t stride_b,
                        uint32_t stride_d, uint32_t* status, uint32_t* flags, uint32_t n_flags, cudaStream_t s) {
    using T = Tile<TYPE, 256>;
    EncodeFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    PairArgs p{};
    p.g = GemmArgs{A, D, M, N, K, stride_d, status};
    p.flags = flags;
    // first byte past the matrix: used where the dequant threads fetch their rows as aligned supersets
    p.a_end = A + (uint64_t)M * (TYPE == T_MXFP4 ? (uint64_t)(K >> 5) * 17u : (uint64_t)(K >> 8) * Raw<TYPE>::kBlock);
    p.n_row_pairs = (M + 2 * kBM - 1) / (2 * kBM);
    p.n_tiles = p.n_row_pairs * ((N + 511) / 512);
    if (!flags || (uint64_t)p.n_tiles * 2 > n_flags) return cudaErrorNotSupported;
    auto kern = gemm_tc_pair_kernel<TYPE, kFetch>;
    static std::atomic<uint64_t> attr_done{0};  // per device ordinal
    if (cudaError_t ea = ensure_dynamic_smem(kern, (int)T::kSmemBytes, attr_done); ea != cudaSuccess) return ea;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = T::kSmemBytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // pairs the device holds at once (every pair of the grid must be resident: pairs wait for each other's tiles)
    static std::atomic<int> max_pairs[64];
    int dev = 0;
    cudaGetDevice(&dev);
    int pairs = dev < 64 ? max_pairs[dev].load(std::memory_order_relaxed) : 0;
    if (pairs == 0) {
        cfg.gridDim = dim3(2, 1, 1);
        if (cudaOccupancyMaxActiveClusters(&pairs, kern, &cfg) != cudaSuccess || pairs < 1) {
            cudaGetLastError();
            return cudaErrorNotSupported;
        }
        if (dev < 64) max_pairs[dev].store(pairs, std::memory_order_relaxed);
    }
    const uint32_t units = p.n_tiles * (TYPE == T_MXFP4 ? (K + 255) >> 8 : K >> 8);
    uint32_t G = units / 4;  // at least four blocks per pair
    G = G < 1 ? 1 : (G > (uint32_t)pairs ? (uint32_t)pairs : G);
    // Nearly as many tiles as pairs: one whole tile per pair (a split tile costs two epilogues and a pass of
    // atomic adds, more than the idle pairs would win)
    if (p.n_tiles <= (uint32_t)pairs && p.n_tiles * 5 >= (uint32_t)pairs * 3) G = p.n_tiles;
    cfg.gridDim = dim3(2 * G, 1, 1);
    // Ranges of a few blocks, shorter than a tile: every pair has one or two partial segments that all end at about
    // the same time, so an ordered hand-over (store, flag, add) would put two epilogues in a row; zero D and let
    // every part add (measured: 5760 x 2880 MXFP4 at 512 tokens 41.9 -> 35.2 us; with ten blocks per pair the
    // flags are ahead again).
    const uint32_t per_pair = units / G;
    p.zeroed = G > 1 && per_pair <= 6 && per_pair < (TYPE == T_MXFP4 ? (K + 255) >> 8 : K >> 8) ? 1u : 0u;
    CUtensorMap map;
    const cuuint64_t dims[2] = {K, N};
    const cuuint64_t strides[1] = {(cuuint64_t)stride_b * 2};
    const cuuint32_t box[2] = {kBK, 256};  // a CTA's 256 tokens: half of either accumulator's operand
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(B), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    CUtensorMap wmap = map;  // not used where the rows have no 16-byte pitch
    if constexpr (!kFetch) {
        const cuuint64_t row_bytes = (cuuint64_t)(K >> 8) * Raw<TYPE>::kBlock;
        const cuuint64_t wdims[2] = {row_bytes, M};
        const cuuint64_t wstrides[1] = {row_bytes};
        const cuuint32_t wbox[2] = {Raw<TYPE>::kBox, kBM};
        if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(A), wdims, wstrides, wbox, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return cudaErrorInvalidValue;
    }
    if (p.zeroed) {
        if (cudaError_t e = cudaMemset2DAsync(D, (size_t)stride_d * 4, 0, (size_t)M * 4, N, s); e != cudaSuccess) return e;
    } else {
        if (cudaError_t e = cudaMemsetAsync(flags, 0, (size_t)p.n_tiles * 2 * sizeof(uint32_t), s); e != cudaSuccess) return e;
    }
    return cudaLaunchKernelEx(&cfg, kern, map, wmap, p);
}

template <int TYPE>
cudaError_t launch_typed(const uint8_t* A, const void* B, float* D, uint32_t M, uint32_t N, uint32_t K,
                         uint32_t stride_b, uint32_t stride_d, uint32_t* status, uint32_t* flags, uint32_t n_flags,
                         cudaStream_t s) {
    if (N <= 128) {
        if constexpr (TYPE == T_Q4_K) return launch_small(A, B, D, M, N, K, stride_b, stride_d, status, s);
        return launch_tile<TYPE, 128, 1>(A, B, D, M, N, K, stride_b, stride_d, status, s);
    }
    if (N <= 256) return launch_tile<TYPE, 256, 1>(A, B, D, M, N, K, stride_b, stride_d, status, s);
    // CTA pairs (half the activation traffic per SM, K streamed over the pairs) unless the half-empty pair of an
    // odd number of row tiles would waste more than a seventh of the work
    const uint32_t row_tiles = (M + kBM - 1) / kBM;
    if (g_pair_mode && ((row_tiles & 1u) == 0 || row_tiles >= 7)) {
        const cudaError_t e = launch_pair<TYPE>(A, B, D, M, N, K, stride_b, stride_d, status, flags, n_flags, s);
        if (e != cudaErrorNotSupported) return e;
    }
    return launch_tile<TYPE, 256, 2>(A, B, D, M, N, K, stride_b, stride_d, status, s);
}

}  // namespace

cudaError_t launch_mul_mm(uint32_t type, const uint8_t* A, const void* B, float* D, uint32_t M, uint32_t N,
                          uint32_t K, uint32_t stride_b, uint32_t stride_d, bool act_bf16, uint32_t* status,
                          uint32_t* tile_flags, uint32_t n_tile_flags, cudaStream_t s, uint64_t* launches) {
    if ((type != T_Q4_K && type != T_Q6_K && type != T_MXFP4) || !act_bf16 || !status) return cudaErrorNotSupported;
    if ((stride_b & 7u) || (reinterpret_cast<uintptr_t>(B) & 15u) || (reinterpret_cast<uintptr_t>(A) & 15u))
        return cudaErrorNotSupported;
    if (type == T_MXFP4) {
        // 512-token tiles on the pair kernel (every weight unpacked once per 512 tokens); fewer tokens, or shapes it
        // leaves, go to the caller's other route (128-token tiles)
        const uint32_t row_tiles = (M + kBM - 1) / kBM;
        if (N <= 256 || (K & 63u) || !g_pair_mode || ((row_tiles & 1u) && row_tiles < 7)) return cudaErrorNotSupported;
        cudaError_t e = launch_pair<T_MXFP4>(A, B, D, M, N, K, stride_b, stride_d, status, tile_flags, n_tile_flags, s);
        if (e == cudaSuccess && launches) ++*launches;
        return e;
    }
    if (K & 255u) return cudaErrorNotSupported;
    // Q6_K rows are 210 bytes per block: the TMA row pitch is a multiple of 16 only for K % 2048 == 0. Other K:
    // the pair kernel with the dequant threads fetching their rows (more than 256 tokens), else the caller's
    // 128-token-tile route.
    if (type == T_Q6_K && (K & 2047u)) {
        const uint32_t row_tiles = (M + kBM - 1) / kBM;
        if (N <= 256 || !g_pair_mode || ((row_tiles & 1u) && row_tiles < 7)) return cudaErrorNotSupported;
        cudaError_t e = launch_pair<T_Q6_K, true>(A, B, D, M, N, K, stride_b, stride_d, status, tile_flags, n_tile_flags, s);
        if (e == cudaSuccess && launches) ++*launches;
        return e;
    }
    if (N < 16) return cudaErrorNotSupported;  // a handful of tokens: the matvec-style kernels are the better fit
    cudaError_t e = type == T_Q4_K
                        ? launch_typed<T_Q4_K>(A, B, D, M, N, K, stride_b, stride_d, status, tile_flags, n_tile_flags, s)
                        : launch_typed<T_Q6_K>(A, B, D, M, N, K, stride_b, stride_d, status, tile_flags, n_tile_flags, s);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
