// MoE prefill: tokens grouped by routed expert, one tensor-core dequant-GEMM tile per (expert, 128 weight
// rows, up to BN of that expert's tokens), so that an expert's weights are read and dequantised once per
// token tile instead of once per (token, slot) pair.
//
//   1. moe_group_kernel     counts the (token, slot) pairs of every expert, lays the experts' pair lists
//                           side by side (no padding) and writes one tile record per BN pairs of an expert
//   2. moe_gather_x_kernel  packs the activation row of every pair, in list order, as bf16 [n_pairs][K]
//   3. moe_gemm_tc_kernel   persistent CTAs walk the (tile, row tile) work items: tcgen05.mma with the
//                           128 weight rows on the TMEM lanes and the tile's pairs on the columns; the
//                           activation box (BN rows from the tile's first pair) comes by TMA and may
//                           run into the next expert's rows, whose columns are never stored
// Raw weight blocks are fetched by the dequant threads themselves with 16-byte cp.async pieces of the
// aligned superset of each row's block (Q6_K blocks are only 2-byte aligned and MXFP4 blocks not aligned
// at all, and their rows have no 16-byte pitch in general, so a tensor map cannot describe them) into a
// ring as deep as shared memory allows (3 to 8 blocks); each copy reports to the slot's mbarrier itself. Types: Q4_K, Q6_K (K % 256 == 0) and MXFP4 (K % 64 == 0; dequantised exactly to bf16).
// Warp roles (23 warps): 0 tensor-memory owner + MMA issuer, 1 TMA loader of the activations, 2 idle,
// 3-18 dequant (set j = 4 warps = group j of every 256-column block = weight stage j), 19-22 epilogue.
// Rings: 4 bf16 weight stages (one per set) each with its activation slot, 4 to 8 raw blocks.
// Two accumulators in tensor memory let the epilogue of one item overlap the MMAs of the next.
// Every mbarrier wait is bounded; a wait that gives up records {1, site}, raises the CTA's flag, and
// every role drains to the common exit where tensor memory is released.
//
// Replaces recordMoeBatchedDispatch's per-pair kernel for prefill batches
// (src/compute/dmmv.zig:746-792; src/shaders/dmmv_q4k_moe_batched.comp:70-164) with the grouping the
// reference's Metal path does (src/shaders/metal/moe_route_pack.metal:13-36).
#include "kernels.h"
#include "tc_common.cuh"

namespace zc {
namespace {

constexpr int kMoeDeqWarp0 = 3, kMoeEpiWarp0 = 19;
constexpr int kMoeThreads = 23 * 32;
// One activation slot (BN x 64 bf16) per weight stage: its TMA load reports to the stage's own barrier, so the
// issuing thread waits once and commits once per stage (each wait and each commit costs it a few hundred
// cycles in this kernel; with a separate activation ring and two waits per stage a layer took 7-20 % longer).
template <int BN>
constexpr int moe_x_slots() { return kAStages; }
constexpr uint32_t kMoeSmemMax = 227u * 1024u;

// The raw-block ring takes what the weight stages and activation slots leave of the 227 KB: its depth is
// what hides the memory latency (one CTA per SM, so blocks in flight per SM = slots - 1).
template <int TYPE, int BN>
struct MoeTile {
    static constexpr uint32_t kRawBytes = kBM * Raw<TYPE>::kBox;
    static constexpr uint32_t kXBytes = BN * kBK * 2;
    static constexpr uint32_t kRawOffset = kAStages * kABytes;
    static constexpr int kXSlots = moe_x_slots<BN>();
    static constexpr uint32_t kAvail = kMoeSmemMax - (512 + 1024) - 1024 - kRawOffset - kXSlots * kXBytes;
    static constexpr int kRawSlots = kAvail / kRawBytes > 8 ? 8 : (int)(kAvail / kRawBytes);
    static constexpr uint32_t kXOffset = (kRawOffset + kRawSlots * kRawBytes + 1023u) & ~1023u;
    static constexpr uint32_t kBarOffset = kXOffset + kXSlots * kXBytes;
    static constexpr uint32_t kSmemBytes = kBarOffset + 512 + 1024;
};

struct MoeBars {
    uint64_t full_a[kAStages];
    uint64_t empty_a[kAStages];
    uint64_t accum_full[2];
    uint64_t accum_empty[2];
    uint64_t full_w[8];   // raw ring: 512 copy-completion arrivals per fill
    uint64_t empty_w[8];  // 16 warp releases per use
    uint32_t tmem_base;
    volatile uint32_t failed;
};

struct MoeGemmArgs {
    const uint8_t* A;
    const uint8_t* a_end;         // one past the last byte of the expert stack
    uint64_t expert_stride;       // bytes
    float* Y;
    const uint32_t* header;       // [0] = number of tiles, [1] = number of listed pairs
    const uint4* tiles;           // {expert, first list slot, pairs in the tile, 0}
    const uint32_t* list;         // pair ids (token * n_used + slot) grouped by expert
    uint32_t M, K, n_used, y_token_stride, row_tiles;
    uint32_t* status;
    uint32_t dense_n;             // > 0: plain GEMM over dense_n tokens (one "expert", identity pair list, no tables)
};

// Tile t: from the table, or (dense) tokens [t * BN, min(dense_n, (t + 1) * BN)) of the only matrix.
template <int BN>
__device__ __forceinline__ uint4 moe_tile(const MoeGemmArgs& g, uint32_t t) {
    if (g.dense_n) return make_uint4(0u, t * BN, min((uint32_t)BN, g.dense_n - t * BN), 0u);
    return __ldg(&g.tiles[t]);
}

template <bool kSleep = true>
__device__ __forceinline__ bool moe_wait(uint64_t* bar, uint32_t parity, MoeBars* bars, uint32_t* status,
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

// Position of the dequant warps in the flat sequence of (work item, 256-column block).
struct BlockCursor {
    uint32_t w;             // work item
    int b;                  // block of the item
    const uint8_t* expert;  // first byte of the item's expert
    uint64_t row_off;       // byte offset of this thread's row inside the expert
};

template <int TYPE, int BN>
__global__ void __launch_bounds__(kMoeThreads, 1)
moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const MoeGemmArgs g) {
    using T = MoeTile<TYPE, BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint8_t* smem_w = smem + T::kRawOffset;
    uint8_t* smem_x = smem + T::kXOffset;
    MoeBars* bars = reinterpret_cast<MoeBars*>(smem + T::kBarOffset);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t n_items = (g.dense_n ? (g.dense_n + BN - 1) / BN : g.header[0]) * g.row_tiles;
    const int n_stages = g.K >> 6;           // 64 columns each
    const int nblk = (n_stages + 3) >> 2;    // 256-column blocks, the last one possibly short (MXFP4)
    constexpr uint32_t kBlock = Raw<TYPE>::kBlock, kBox = Raw<TYPE>::kBox;
    constexpr int kPieces = TYPE == T_MXFP4 ? 10 : (int)kBox / 16;
    const uint64_t row_bytes = TYPE == T_MXFP4 ? (uint64_t)(g.K >> 5) * 17u : (uint64_t)nblk * kBlock;

    if (tid == 0) {
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&bars->full_a[s], 5);  // one arrival per warp of the owning set + the activation box
            mbar_init(&bars->empty_a[s], 1);
        }
        for (int s = 0; s < T::kRawSlots; ++s) {
            mbar_init(&bars->full_w[s], 512);
            mbar_init(&bars->empty_w[s], 16);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars->accum_full[s], 1);
            mbar_init(&bars->accum_empty[s], 4);  // one arrival per epilogue warp
        }
        bars->failed = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&bars->tmem_base)),
                     "r"((uint32_t)(2 * BN))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        if (lane == 0) {  // ---- MMA issuer ----
            constexpr uint32_t idesc = instr_desc<BN>();
            uint32_t gs = 0, i = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++i) {
                const uint32_t ab = i & 1;
                ok = moe_wait<false>(&bars->accum_empty[ab], ((i >> 1) & 1) ^ 1, bars, g.status, 121);
                if (!ok) break;
                tc_fence_after();
                for (int s = 0; s < n_stages; ++s, ++gs) {
                    const int st = gs & 3;
                    const uint32_t ph = (gs >> 2) & 1;
                    ok = moe_wait<false>(&bars->full_a[st], ph, bars, g.status, 122);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t da = smem_desc(smem_u32(smem + st * kABytes));
                    const uint64_t dx = smem_desc(smem_u32(smem_x + st * T::kXBytes));
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        umma_bf16(tmem + ab * BN, da + 2 * k, dx + 2 * k, idesc, (s | k) ? 1u : 0u);
                    umma_commit(&bars->empty_a[st]);
                }
                if (ok) umma_commit(&bars->accum_full[ab]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // ---- TMA loader of the packed activations ----
            uint32_t gs = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
                const uint4 tile = moe_tile<BN>(g, w / g.row_tiles);
                for (int s = 0; s < n_stages; ++s, ++gs) {
                    const int st = gs & 3;
                    ok = moe_wait(&bars->empty_a[st], ((gs >> 2) & 1) ^ 1, bars, g.status, 124);
                    if (!ok) break;
                    mbar_expect_tx(&bars->full_a[st], T::kXBytes);
                    tma_load_2d(smem_x + st * T::kXBytes, &tmap_x, s * kBK, (int)tile.y, &bars->full_a[st]);
                }
            }
        }
    } else if (warp >= kMoeDeqWarp0 && warp < kMoeEpiWarp0) {
        // ---- dequant producers: thread = (row, set j); set j always fills weight stage j. A block that
        // starts at running stage gs hands its group q to set (gs + q) & 3 ----
        const int p = tid - kMoeDeqWarp0 * 32;
        const int row = p & 127, j = p >> 7;
        uint8_t* a_stage = smem + j * kABytes;
        auto locate = [&](uint32_t w, BlockCursor& c) {
            c.w = w;
            c.b = 0;
            if (w < n_items) {
                const uint4 tile = moe_tile<BN>(g, w / g.row_tiles);
                const uint32_t m0 = (w % g.row_tiles) * kBM;
                const uint32_t grow = min(m0 + (uint32_t)row, g.M - 1);  // rows past M are computed and dropped
                c.expert = g.A + (uint64_t)tile.x * g.expert_stride;
                c.row_off = (uint64_t)grow * row_bytes;
            }
        };
        // this thread's pieces (j, j + 4, ...) of the aligned superset of its row's block
        auto fetch = [&](const BlockCursor& c, uint32_t slot_idx) {
            const uint64_t o = c.row_off + (uint64_t)c.b * kBlock;
            const uint8_t* src = c.expert + (o & ~(uint64_t)15);
            uint8_t* dst = smem_w + slot_idx * T::kRawBytes + row * kBox;
#pragma unroll
            for (int pc = 0; pc < kPieces; pc += 4) {
                const int piece = pc + j;
                if (piece < kPieces) {
                    const uint8_t* s = src + piece * 16;
                    const uint32_t n = s + 16 <= g.a_end ? 16u : (s < g.a_end ? (uint32_t)(g.a_end - s) : 0u);
                    cp_async16_zfill(dst + piece * 16, n ? s : g.A, n);
                }
            }
        };
        auto advance = [&](BlockCursor& c) {
            if (c.b + 1 < nblk)
                ++c.b;
            else
                locate(c.w + gridDim.x, c);
        };
        // The raw ring: a slot is filled by all 512 threads (each its pieces) and every copy reports to the
        // slot's mbarrier by itself when it lands (cp.async.mbarrier.arrive.noinc), so no thread has to
        // reach a program point for the others and the four sets drift apart as the MMA order wants.
        // A warp releases a slot once it has read its part; the refill waits for all 16 releases.
        constexpr int kSlots = T::kRawSlots;
        BlockCursor cur, ahead;
        locate(blockIdx.x, cur);
        ahead = cur;
        uint32_t gs = 0, slot_c = 0, use_c = 0, slot_f = 0, use_f = 0;
        bool dead = false;
        auto issue_fetch = [&]() {
            if (ahead.w >= n_items) return;
            if (!dead) dead = !moe_wait(&bars->empty_w[slot_f], (use_f & 1) ^ 1, bars, g.status, 127);
            if (!dead) fetch(ahead, slot_f);
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bars->full_w[slot_f]))
                         : "memory");
            advance(ahead);
            if (++slot_f == (uint32_t)kSlots) {
                slot_f = 0;
                ++use_f;
            }
        };
        for (int d = 0; d < kSlots - 1; ++d) issue_fetch();
        while (cur.w < n_items) {
            const int ns = min(4, n_stages - 4 * cur.b);
            const int q = (j - (int)gs) & 3;  // this set's group of the block, if the block has that many
            const bool mine = q < ns;
            if (mine && !dead) dead = !moe_wait(&bars->full_w[slot_c], use_c & 1, bars, g.status, 128);
            if (mine && !dead)
                dead = !moe_wait(&bars->empty_a[j], (((gs + q) >> 2) & 1) ^ 1, bars, g.status, 125);
            if (mine && !dead) {
                const uint8_t* slot = smem_w + slot_c * T::kRawBytes + row * kBox;
                if constexpr (TYPE == T_Q4_K) {
                    const uint4 chdr = *reinterpret_cast<const uint4*>(slot);
                    const uint4 c0 = *reinterpret_cast<const uint4*>(slot + 16 + q * 32);
                    const uint4 c1 = *reinterpret_cast<const uint4*>(slot + 32 + q * 32);
                    const __half2 dd = *reinterpret_cast<const __half2*>(&chdr.x);
                    const float d = __low2float(dd), dmin = __high2float(dd);
                    uint32_t s0, mn0, s1, mn1;
                    scale_min_k4(2 * q, chdr.y, chdr.z, chdr.w, s0, mn0);
                    scale_min_k4(2 * q + 1, chdr.y, chdr.z, chdr.w, s1, mn1);
                    dequant_group_q4k(c0, c1, d * (float)s0, dmin * (float)mn0, d * (float)s1, dmin * (float)mn1,
                                      a_stage, row);
                } else if constexpr (TYPE == T_Q6_K) {
                    const uint32_t off = (uint32_t)((cur.row_off + (uint64_t)cur.b * kBlock) & 15u);
                    dequant_group_q6k(reinterpret_cast<const uint32_t*>(slot + (off & ~3u)), (off & 2u) * 8u, q,
                                      a_stage, row);
                } else {
                    const uint32_t off = (uint32_t)((cur.row_off + (uint64_t)cur.b * kBlock) & 15u) + 34u * q;
                    dequant_group_mxfp4(reinterpret_cast<const uint32_t*>(slot + (off & ~3u)), (off & 3u) * 8u,
                                        a_stage, row);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->full_a[j]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->empty_w[slot_c]);  // this warp is done with the slot
            advance(cur);
            if (++slot_c == (uint32_t)kSlots) {
                slot_c = 0;
                ++use_c;
            }
            gs += ns;
            issue_fetch();
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (warp >= kMoeEpiWarp0) {
        // ---- epilogue: lane = weight row, column = pair of the tile ----
        const uint32_t q = warp & 3;
        uint32_t i = 0;
        for (uint32_t w = blockIdx.x; w < n_items; w += gridDim.x, ++i) {
            const uint32_t ab = i & 1;
            const uint4 tile = moe_tile<BN>(g, w / g.row_tiles);
            const uint32_t m = (w % g.row_tiles) * kBM + q * 32 + lane;
            if (!moe_wait(&bars->accum_full[ab], (i >> 1) & 1, bars, g.status, 126)) break;
            __syncwarp();
            tc_fence_after();
#pragma unroll 1
            for (uint32_t c = 0; c * 32 < tile.z; ++c) {
                uint32_t v[32];
                const uint32_t taddr = tmem + ((q * 32u) << 16) + ab * BN + c * 32;
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
                // pair of column c*32 + lane; its output row starts at Y + token * y_token_stride + slot * M
                const uint32_t idx = c * 32 + lane;
                const uint32_t pair = idx >= tile.z ? 0u : (g.dense_n ? tile.y + idx : __ldg(&g.list[tile.y + idx]));
                const uint32_t tok = pair / g.n_used, slot = pair - tok * g.n_used;
#pragma unroll
                for (int jj = 0; jj < 32; ++jj) {
                    const uint32_t t_j = __shfl_sync(0xFFFFFFFFu, tok, jj);
                    const uint32_t s_j = __shfl_sync(0xFFFFFFFFu, slot, jj);
                    if (c * 32 + jj < tile.z && m < g.M)
                        g.Y[(uint64_t)t_j * g.y_token_stride + (uint64_t)s_j * g.M + m] = __uint_as_float(v[jj]);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(2 * BN))
                     : "memory");
    }
}

// ---- grouping ------------------------------------------------------------------------------------------
// One CTA. Shared: cnt[n_experts], seg[n_experts] (first list slot, then the running cursor), tstart[n_experts].
__global__ void __launch_bounds__(1024, 1)
moe_group_kernel(const uint32_t* __restrict__ routing, uint32_t n_pairs, uint32_t n_experts, uint32_t bn,
                 uint32_t* __restrict__ header, uint4* __restrict__ tiles, uint32_t* __restrict__ list,
                 uint32_t* __restrict__ status) {
    extern __shared__ uint32_t sh[];
    uint32_t* cnt = sh;
    uint32_t* seg = sh + n_experts;
    uint32_t* tstart = sh + 2 * n_experts;
    const uint32_t tid = threadIdx.x, nt = blockDim.x;
    for (uint32_t e = tid; e < n_experts; e += nt) cnt[e] = 0;
    __syncthreads();
    for (uint32_t p = tid; p < n_pairs; p += nt) {
        const uint32_t e = routing[p];
        if (e < n_experts) {
            atomicAdd(&cnt[e], 1u);
        } else if (status && e != 0xFFFFFFFFu) {  // not an expert (and not the "no expert here" mark): left out and reported
            status[0] = 2u;
            status[1] = e;
        }
    }
    __syncthreads();
    if (tid < 32) {  // exclusive scan of the pair and tile counts: a chunk of experts per lane
        const uint32_t per = (n_experts + 31) / 32;
        const uint32_t e0 = min(tid * per, n_experts), e1 = min(e0 + per, n_experts);
        uint32_t sp = 0, st = 0;
        for (uint32_t e = e0; e < e1; ++e) {
            sp += cnt[e];
            st += (cnt[e] + bn - 1) / bn;
        }
        uint32_t ip = sp, it = st;
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t a = __shfl_up_sync(0xFFFFFFFFu, ip, o), b = __shfl_up_sync(0xFFFFFFFFu, it, o);
            if ((int)tid >= o) {
                ip += a;
                it += b;
            }
        }
        if (tid == 31) {
            header[0] = it;
            header[1] = ip;
        }
        uint32_t bp = ip - sp, bt = it - st;
        for (uint32_t e = e0; e < e1; ++e) {
            seg[e] = bp;
            tstart[e] = bt;
            bp += cnt[e];
            bt += (cnt[e] + bn - 1) / bn;
        }
    }
    __syncthreads();
    for (uint32_t e = tid; e < n_experts; e += nt) {
        const uint32_t c = cnt[e];
        for (uint32_t i = 0; i * bn < c; ++i)
            tiles[tstart[e] + i] = make_uint4(e, seg[e] + i * bn, min(bn, c - i * bn), 0u);
    }
    __syncthreads();
    for (uint32_t p = tid; p < n_pairs; p += nt) {
        const uint32_t e = routing[p];
        if (e < n_experts) list[atomicAdd(&seg[e], 1u)] = p;
    }
}

// One warp per listed pair: its token's activation row as bf16.
__global__ void __launch_bounds__(256)
moe_gather_x_kernel(const float* __restrict__ X, const uint32_t* __restrict__ header,
                    const uint32_t* __restrict__ list, __nv_bfloat16* __restrict__ Xp, uint32_t K, uint32_t n_used,
                    uint32_t x_token_stride) {
    const uint32_t slot = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (slot >= header[1]) return;
    const uint32_t pair = list[slot];
    const float* src = X + (uint64_t)(pair / n_used) * x_token_stride;
    uint4* dst = reinterpret_cast<uint4*>(Xp + (uint64_t)slot * K);
    for (uint32_t c = lane; c < K / 8; c += 32) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(src) + 2 * c);
        const float4 b = __ldg(reinterpret_cast<const float4*>(src) + 2 * c + 1);
        uint4 o;
        o.x = bf2_bits(__floats2bfloat162_rn(a.x, a.y));
        o.y = bf2_bits(__floats2bfloat162_rn(a.z, a.w));
        o.z = bf2_bits(__floats2bfloat162_rn(b.x, b.y));
        o.w = bf2_bits(__floats2bfloat162_rn(b.z, b.w));
        dst[c] = o;
    }
}

constexpr uint32_t kMoeMaxExperts = 4096;

struct WsLayout {
    uint64_t header, tiles, list, xp, total;
    uint32_t max_tiles;
};
WsLayout ws_layout(uint64_t n_pairs, uint32_t K, uint32_t n_experts, uint32_t bn) {
    WsLayout l;
    l.max_tiles = (uint32_t)(n_pairs / bn + n_experts);
    l.header = 0;
    l.tiles = 256;
    l.list = l.tiles + (uint64_t)l.max_tiles * 16;
    l.xp = (l.list + n_pairs * 4 + 255) & ~(uint64_t)255;
    l.total = l.xp + n_pairs * K * 2;
    return l;
}

template <int TYPE, int BN>
cudaError_t launch_gemm(const CUtensorMap& map, const MoeGemmArgs& g, uint32_t max_items, cudaStream_t s) {
    auto kern = moe_gemm_tc_kernel<TYPE, BN>;
    static std::atomic<uint64_t> attr_done{0};  // per device ordinal
    if (cudaError_t ea = ensure_dynamic_smem(kern, (int)MoeTile<TYPE, BN>::kSmemBytes, attr_done); ea != cudaSuccess) return ea;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint32_t grid = max_items < (uint32_t)sms ? max_items : (uint32_t)sms;
    kern<<<grid, kMoeThreads, MoeTile<TYPE, BN>::kSmemBytes, s>>>(map, g);
    return cudaGetLastError();
}

// Tokens per tile: 32 when experts see few pairs on average (the activation box then stays small), else 128.
uint32_t pick_bn(uint64_t n_pairs, uint32_t n_experts) { return n_pairs <= (uint64_t)n_experts * 48 ? 32u : 128u; }

}  // namespace

uint64_t moe_grouped_workspace_bytes(uint64_t n_pairs, uint32_t K, uint32_t n_experts) {
    return ws_layout(n_pairs, K, n_experts, 32).total;  // the smaller tile needs the longer tile table
}

bool moe_grouped_eligible(uint32_t type, const uint8_t* A, uint32_t K, uint64_t expert_stride, uint32_t n_experts,
                          uint64_t n_pairs, const float* X, uint32_t x_token_stride, uint64_t ws_size) {
    if (type != T_Q4_K && type != T_Q6_K && type != T_MXFP4) return false;
    if ((type == T_MXFP4 ? (K & 63u) : (K & 255u)) || K < 64 || n_experts > kMoeMaxExperts || n_pairs > 0x7FFFFFFFull)
        return false;
    if ((reinterpret_cast<uintptr_t>(A) & 15u) || (expert_stride & 15u)) return false;
    if ((reinterpret_cast<uintptr_t>(X) & 15u) || (x_token_stride & 3u)) return false;
    return ws_size >= moe_grouped_workspace_bytes(n_pairs, K, n_experts);
}

cudaError_t launch_moe_grouped(uint32_t type, const uint8_t* A, uint64_t a_bytes, const float* X, float* Y,
                               const uint32_t* routing, uint32_t M, uint32_t K, uint64_t expert_stride,
                               uint32_t n_experts, uint32_t n_used, uint32_t n_tokens, uint32_t x_token_stride,
                               uint32_t y_token_stride, void* ws, uint32_t* status, cudaStream_t s,
                               uint64_t* launches, const uint8_t* A2, uint64_t a2_bytes, float* Y2) {
    EncodeFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    const uint64_t n_pairs = (uint64_t)n_tokens * n_used;
    const uint32_t bn = pick_bn(n_pairs, n_experts);
    const WsLayout l = ws_layout(n_pairs, K, n_experts, bn);
    uint8_t* base = static_cast<uint8_t*>(ws);
    uint32_t* header = reinterpret_cast<uint32_t*>(base + l.header);
    uint4* tiles = reinterpret_cast<uint4*>(base + l.tiles);
    uint32_t* list = reinterpret_cast<uint32_t*>(base + l.list);
    __nv_bfloat16* xp = reinterpret_cast<__nv_bfloat16*>(base + l.xp);

    moe_group_kernel<<<1, 1024, (size_t)n_experts * 12, s>>>(routing, (uint32_t)n_pairs, n_experts, bn, header, tiles,
                                                            list, status);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    moe_gather_x_kernel<<<(uint32_t)((n_pairs + 7) / 8), 256, 0, s>>>(X, header, list, xp, K, n_used, x_token_stride);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;

    CUtensorMap map;
    const cuuint64_t dims[2] = {K, n_pairs};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {kBK, bn};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xp, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    MoeGemmArgs g{A, A + a_bytes, expert_stride, Y, header, tiles, list, M, K, n_used, y_token_stride,
                  (M + kBM - 1) / kBM, status, 0u};
    const uint64_t max_items64 = (uint64_t)l.max_tiles * g.row_tiles;
    const uint32_t max_items = max_items64 > 0xFFFFFFFFull ? 0xFFFFFFFFu : (uint32_t)max_items64;
    // one grouping and one packed activation buffer serve both matrices of a pair (gate and up)
    for (int pass = 0; pass < (A2 ? 2 : 1); ++pass) {
        if (pass == 1) {
            g.A = A2;
            g.a_end = A2 + a2_bytes;
            g.Y = Y2;
        }
        if (type == T_Q4_K)
            e = bn == 32 ? launch_gemm<T_Q4_K, 32>(map, g, max_items, s)
                         : launch_gemm<T_Q4_K, 128>(map, g, max_items, s);
        else if (type == T_MXFP4)
            e = bn == 32 ? launch_gemm<T_MXFP4, 32>(map, g, max_items, s)
                         : launch_gemm<T_MXFP4, 128>(map, g, max_items, s);
        else
            e = bn == 32 ? launch_gemm<T_Q6_K, 32>(map, g, max_items, s)
                         : launch_gemm<T_Q6_K, 128>(map, g, max_items, s);
        if (e != cudaSuccess) return e;
    }
    if (launches) *launches += A2 ? 4 : 3;
    return e;
}

// Plain prefill GEMM D[n][m] = sum_k W[m][k] X[n][k] through the same tile kernel (one matrix, token tiles in
// order, no grouping tables): serves the weight layouts a tensor map cannot describe, i.e. MXFP4 (K % 64 == 0)
// and Q6_K with a row pitch that is not a multiple of 16 bytes. X is bf16 [N][stride_b].
bool mul_mm_cp_async_eligible(uint32_t type, const uint8_t* A, const void* B, uint32_t N, uint32_t K,
                              uint32_t stride_b) {
    if (type != T_MXFP4 && type != T_Q6_K && type != T_Q4_K) return false;
    if ((type == T_MXFP4 ? (K & 63u) : (K & 255u)) || K < 64 || N < 16) return false;
    return !(reinterpret_cast<uintptr_t>(A) & 15u) && !(reinterpret_cast<uintptr_t>(B) & 15u) && !(stride_b & 7u);
}

cudaError_t launch_mul_mm_cp_async(uint32_t type, const uint8_t* A, uint64_t a_bytes, const void* B, float* D,
                                   uint32_t M, uint32_t N, uint32_t K, uint32_t stride_b, uint32_t stride_d,
                                   uint32_t* status, cudaStream_t s, uint64_t* launches) {
    EncodeFn enc = encode_fn();
    if (!enc) return cudaErrorNotSupported;
    const uint32_t bn = N <= 32 ? 32u : 128u;
    CUtensorMap map;
    const cuuint64_t dims[2] = {K, N};
    const cuuint64_t strides[1] = {(cuuint64_t)stride_b * 2};
    const cuuint32_t box[2] = {kBK, bn};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(B), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    MoeGemmArgs g{A, A + a_bytes, 0, D, nullptr, nullptr, nullptr, M, K, 1u, stride_d, (M + kBM - 1) / kBM, status, N};
    const uint64_t items64 = (uint64_t)((N + bn - 1) / bn) * g.row_tiles;
    const uint32_t items = items64 > 0xFFFFFFFFull ? 0xFFFFFFFFu : (uint32_t)items64;
    cudaError_t e;
    if (type == T_Q4_K)
        e = bn == 32 ? launch_gemm<T_Q4_K, 32>(map, g, items, s) : launch_gemm<T_Q4_K, 128>(map, g, items, s);
    else if (type == T_MXFP4)
        e = bn == 32 ? launch_gemm<T_MXFP4, 32>(map, g, items, s) : launch_gemm<T_MXFP4, 128>(map, g, items, s);
    else
        e = bn == 32 ? launch_gemm<T_Q6_K, 32>(map, g, items, s) : launch_gemm<T_Q6_K, 128>(map, g, items, s);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
