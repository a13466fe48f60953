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
//   P_s = sum_{i in s} (v_i - 32) * X_i = D_s - 32 * SX_s,   D_s = sum_i v_i * X_i
// v_i = 6-bit quant 0..63 fed to the tensor core as u8, X_i = round(x_i * 2^f) the block of x in
// 21-bit fixed point split into three 7-bit digits (s8), SX_s = sum_i X_i. D_s, SX_s and P_s are
// exact integers; the only rounding before the f32 scaling is that of x to 21 bits.
//
// Blocks are only 2-byte aligned (210 = 13*16 + 2), so a unit is copied as the 16-byte aligned
// superset of each row's block and read back with aligned 32-bit loads + a funnel shift whose
// amount is the same for the whole warp. Rows must start 16-byte aligned (K a multiple of 2048).
//
// Lane (g = lane/4, t = lane%4) owns, for rows g and g+8, the 32 ql bytes 64h + 32c .. (h = t/2,
// c = t%2) and the 32 qh bytes of half h: low nibbles are elements 128h + 32c + l, high nibbles
// 128h + 64 + 32c + l, i.e. four 16-weight sub-blocks. B is block-diagonal as in the Q4_K kernel.
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
constexpr int kZeroUnits = 72;
constexpr int kFracBits = 20;
constexpr int kPrepBlocks = 6;
constexpr size_t kTwoPerSm = 113 * 1024;

struct Smem6 {
    uint4* xf;       // x digits in B-operand order: unit ((blk*8 + s*4 + i)*2 + p)*4 + t
    uint4* zeros;
    int* sx;         // per 16-element sub-block sum of X (exact)
    float* xs;       // per super-block 2^-f
    uint8_t* ring;   // [kWarps][kDepth] stages of 16 row slots
    float* spartial;
    volatile uint32_t* sflags;
};

__host__ __device__ inline size_t smem_bytes6(uint32_t K, int kWarps) {
    size_t n = (size_t)K * 4 + (size_t)kZeroUnits * 16;
    n += (size_t)(K / 16) * 4 + (size_t)(K / 256) * 4;
    n = (n + 127) & ~size_t(127);
    n += (size_t)kWarps * kRing6;
    n += (size_t)kWarps * 32 * 4 + (size_t)kWarps * 4 + 16;
    return n + 128;
}

__device__ inline Smem6 carve6(uint8_t* base, uint32_t K, int kWarps) {
    Smem6 s;
    uintptr_t p = (reinterpret_cast<uintptr_t>(base) + 127) & ~uintptr_t(127);
    s.xf = reinterpret_cast<uint4*>(p);
    p += (size_t)K * 4;
    s.zeros = reinterpret_cast<uint4*>(p);
    p += (size_t)kZeroUnits * 16;
    s.sx = reinterpret_cast<int*>(p);
    p += (size_t)(K / 16) * 4;
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
// lane = i*8 + s*4 + t handles the 8 consecutive elements 128(t/2) + 64s + 32(t%2) + 8i .. +7
__device__ __forceinline__ uint32_t x_elem6(int lane) {
    const int i = lane >> 3, sh = (lane >> 2) & 1, t = lane & 3;
    return 128 * (t >> 1) + 64 * sh + 32 * (t & 1) + 8 * i;
}
// K: length of the (concatenated) activation. bpe > 0 (MoE down projection): the activation is n_slots
// vectors of bpe * 256 elements, x + s * x_stride, each scaled by the slot's routing weight wts[s].
template <int kWarps>
__device__ __forceinline__ void load_x6(XRegs6& r, const float* __restrict__ x, uint32_t K, uint32_t bpe,
                                        uint32_t x_stride, const uint32_t* __restrict__ wts, int warp, int lane) {
#pragma unroll
    for (int b = 0; b < kPrepBlocks; ++b) {
        const uint32_t blk = warp + b * kWarps;
        if (blk < (K >> 8)) {
            const uint32_t slot = bpe ? blk / bpe : 0u, lb = bpe ? blk - slot * bpe : blk;
            const float* xp = x + (size_t)slot * x_stride + (size_t)lb * 256 + x_elem6(lane);
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
template <int kWarps>
__device__ __forceinline__ void prep_x6(const Smem6& s, const XRegs6& r, uint32_t K, int warp, int lane) {
    const int i = lane >> 3, sh = (lane >> 2) & 1, t = lane & 3;
#pragma unroll
    for (int b = 0; b < kPrepBlocks; ++b) {
        const uint32_t blk = warp + b * kWarps;
        if (blk >= (K >> 8)) break;
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
        uint32_t d0[2] = {0, 0}, d1[2] = {0, 0}, d2[2] = {0, 0};
        int sum = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int X = __float2int_rn(v[e] * scale);
            sum += X;
            d0[e >> 2] |= (uint32_t)((X >> 14) & 0xFF) << (8 * (e & 3));
            d1[e >> 2] |= (uint32_t)((X >> 7) & 0x7F) << (8 * (e & 3));
            d2[e >> 2] |= (uint32_t)(X & 0x7F) << (8 * (e & 3));
        }
        const uint32_t u = (blk * 8 + sh * 4 + i) * 2;
        s.xf[(u + 0) * 4 + t] = make_uint4(d0[0], d0[1], d2[0], d2[1]);
        s.xf[(u + 1) * 4 + t] = make_uint4(d1[0], d1[1], 0u, 0u);
        // 16-element sub-block sums: lanes i and i^1 hold the two halves
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 8);
        if ((i & 1) == 0) s.sx[blk * 16 + (x_elem6(lane) >> 4)] = sum;
        if (lane == 0) s.xs[blk] = __uint_as_float((E + 1u - kFracBits) << 23);
    }
}

__device__ __forceinline__ uint32_t lds_u32s(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}

// N consecutive 32-bit words starting `sh` bits into the aligned word at shared address saddr (sh = 0 or 16)
template <int N>
__device__ __forceinline__ void lds_words(uint32_t saddr, uint32_t sh, uint32_t (&w)[N]) {
    uint32_t prev = lds_u32s(saddr);
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const uint32_t next = lds_u32s(saddr + 4 * (i + 1));
        w[i] = __funnelshift_r(prev, next, sh);
        prev = next;
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
    pdl_launch_dependents();
    const uint32_t bpe = a.K >> 8;                        // blocks per row of one matrix
    const uint32_t bpr = kMoe ? bpe * a.nseg : bpe;       // blocks per (concatenated) row = units per tile
    const Smem6 s = carve6(smem_raw, bpr * 256, kWarps);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3, h = t >> 1, c = t & 1;
    const uint64_t row_bytes = (uint64_t)bpe * 210;
    // matrix that holds block `b` of the concatenated row, and the block's index inside it
    auto matrix_of = [&](uint32_t b, uint32_t& lb) -> const uint8_t* {
        if constexpr (kMoe) {
            const uint32_t slot = b / bpe;
            lb = b - slot * bpe;
            return a.A[0] + (uint64_t)checked_expert(__ldg(a.routing + slot), a.n_experts_max, a.status) * a.expert_stride;
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
    auto request = [&](uint32_t slot) {
        uint8_t* dst = ring + slot * kSlot6;
        const uint32_t row0 = p_tile * 16;
        if constexpr (kRowsAligned) {
            const uint32_t al = (p_blk * 210u) & ~15u;  // aligned start of the block's superset within the row
#pragma unroll
            for (int i = 0; i < kPiecesLane6; ++i) {
                const uint32_t r = piece[i] & 0xFFu, col = piece[i] >> 8;
                if (al + col * 16 < (uint32_t)row_bytes) {  // rows are 16-byte aligned: a piece never crosses the row end
                    const uint32_t row = min(row0 + r, a.M - 1);
                    cp_async16(dst + r * kRow6 + col * 16, a.A[0] + (uint64_t)row * row_bytes + al + col * 16);
                }
            }
        } else {
            uint32_t lb;
            const uint8_t* mat = matrix_of(p_blk, lb);
#pragma unroll
            for (int i = 0; i < kPiecesLane6; ++i) {
                const uint32_t r = piece[i] & 0xFFu, col = piece[i] >> 8;
                const uint32_t row = min(row0 + r, a.M - 1);
                const uint8_t* start = mat + (uint64_t)row * row_bytes + lb * 210u;
                const uint32_t o = (uint32_t)(reinterpret_cast<uintptr_t>(start) & 15u);
                if (col * 16 < o + 210u) {  // the piece holds bytes of the block
                    const uint8_t* src = start - o + col * 16;
                    uint8_t* d = dst + r * kRow6 + col * 16;
                    if (src + 16 <= a_end) {
                        cp_async16(d, src);
                    } else {  // the very end of the tensor: copy only the bytes that exist
                        for (const uint8_t* q = src; q < a_end; ++q) d[q - src] = __ldg(q);
                    }
                }
            }
        }
        if (++p_blk == bpr) { p_blk = 0; ++p_tile; }
    };
    if (n) request(0);
    cp_async_commit();
    pdl_wait();
    XRegs6 xr;
    load_x6<kWarps>(xr, a.x, bpr * 256, kMoe ? bpe : 0u, kMoe ? a.x_slot_stride : 0u,
                    kMoe ? a.routing + a.nseg : nullptr, warp, lane);
#pragma unroll
    for (int i = 1; i < kDepth; ++i) {
        if ((uint32_t)i < n) request(i);
        cp_async_commit();
    }

    if (tid < kZeroUnits) s.zeros[tid] = make_uint4(0u, 0u, 0u, 0u);
    if (tid < kWarps) s.sflags[tid] = 0u;
    prep_x6<kWarps>(s, xr, bpr * 256, warp, lane);
    __syncthreads();

    uint32_t tile = u0 / bpr, blk = u0 % bpr;
    float acc[2] = {0.f, 0.f};
    const bool b_live = (g >> 1) == t;
    const uint32_t xu_live = smem_u32(s.xf + (g & 1) * 4 + t);
    const uint32_t xu_dead = smem_u32(s.zeros + (g >> 1) + 1);
    const uint32_t ring_s = smem_u32(ring), xs_s = smem_u32(s.xs), sx_s = smem_u32(s.sx);
    const uint32_t shl = 4 - 2 * c, shr = 2 * c;  // qh bit pairs: low nibbles use bits 2c.., high nibbles 4+2c..
    constexpr uint32_t kNib = 0x0F0F0F0Fu, kTop = 0x30303030u;

    for (uint32_t it = 0; it < n; ++it) {
        const uint32_t slot = it % kDepth;
        cp_async_wait<kDepth - 1>();
        __syncwarp();
        // byte offset of the block inside each row's aligned superset, and the funnel shift it implies
        uint32_t oA, oB;
        if constexpr (kRowsAligned) {
            oA = oB = (blk * 210u) & 15u;
        } else {
            const uint32_t rA = min(tile * 16 + g, a.M - 1), rB = min(tile * 16 + g + 8, a.M - 1);
            uint32_t lb;
            const uint8_t* mat = matrix_of(blk, lb);
            oA = (uint32_t)(reinterpret_cast<uintptr_t>(mat + (uint64_t)rA * row_bytes + lb * 210u) & 15u);
            oB = (uint32_t)(reinterpret_cast<uintptr_t>(mat + (uint64_t)rB * row_bytes + lb * 210u) & 15u);
        }
        const uint32_t fsA = (oA & 3u) * 8u, fsB = (oB & 3u) * 8u;
        const uint32_t sb = ring_s + slot * kSlot6;
        const uint32_t xu = b_live ? xu_live + blk * 1024u : xu_dead;  // 64 units of 16 bytes per super-block
        // both rows share the B operand; accumulators: [row-pair quad] per sub-block (lo k=0,1; hi k=0,1)
        int d01[4][4], d2[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q)
#pragma unroll
            for (int e = 0; e < 4; ++e) d01[q][e] = d2[q][e] = 0;
        const uint32_t wA = sb + g * kRow6 + (oA & ~3u), wB = sb + (g + 8) * kRow6 + (oB & ~3u);  // byte addresses; word offsets below x 4
        uint32_t qlA[8], qhA[8], qlB[8], qhB[8];
        lds_words<8>(wA + 4 * (16 * h + 8 * c), fsA, qlA);
        lds_words<8>(wA + 4 * (32 + 8 * h), fsA, qhA);
        lds_words<8>(wB + 4 * (16 * h + 8 * c), fsB, qlB);
        lds_words<8>(wB + 4 * (32 + 8 * h), fsB, qhB);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 bl = lds_v4(xu + i * 128), bh = lds_v4(xu + (4 + i) * 128);
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t la = qlA[2 * i + e], ha = qhA[2 * i + e], lb = qlB[2 * i + e], hb = qhB[2 * i + e];
                lo[2 * e] = (la & kNib) | ((ha << shl) & kTop);
                lo[2 * e + 1] = (lb & kNib) | ((hb << shl) & kTop);
                hi[2 * e] = ((la >> 4) & kNib) | ((ha >> shr) & kTop);
                hi[2 * e + 1] = ((lb >> 4) & kNib) | ((hb >> shr) & kTop);
            }
            // words 2i, 2i+1 = elements l = 8i .. 8i+7: sub-block half k = i/2
            mma_u8s8(d01[i >> 1], lo[0], lo[1], lo[2], lo[3], bl.x, bl.y);
            mma_u8s8(d2[i >> 1], lo[0], lo[1], lo[2], lo[3], bl.z, bl.w);
            mma_u8s8(d01[2 + (i >> 1)], hi[0], hi[1], hi[2], hi[3], bh.x, bh.y);
            mma_u8s8(d2[2 + (i >> 1)], hi[0], hi[1], hi[2], hi[3], bh.z, bh.w);
        }
        // scales: the 8 int8 of half h; this lane's four are bytes 2c, 2c+1 (low) and 4+2c, 5+2c (high)
        uint32_t scA[2], scB[2], dA[1], dB[1];
        lds_words<2>(wA + 4 * (48 + 2 * h), fsA, scA);
        lds_words<2>(wB + 4 * (48 + 2 * h), fsB, scB);
        lds_words<1>(wA + 4 * 52, fsA, dA);
        lds_words<1>(wB + 4 * 52, fsB, dB);
        // every lane has read the stage: refill it
        __syncwarp();
        if (it + kDepth < n) request(slot);
        cp_async_commit();

        const uint32_t sx = sx_s + 4 * (blk * 16 + 8 * h + 2 * c);  // sub-blocks 8h+2c+k (low), 8h+4+2c+k (high)
        const int sx0 = (int)lds_u32s(sx), sx1 = (int)lds_u32s(sx + 4), sx2 = (int)lds_u32s(sx + 16), sx3 = (int)lds_u32s(sx + 20);
        const int sxs[4] = {sx0, sx1, sx2, sx3};
        float sumA = 0.f, sumB = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int PA = d01[q][0] * 16384 + d01[q][1] * 128 + d2[q][0] - 32 * sxs[q];
            const int PB = d01[q][2] * 16384 + d01[q][3] * 128 + d2[q][2] - 32 * sxs[q];
            const uint32_t wa = scA[q >> 1] >> (16 * c + 8 * (q & 1)), wb = scB[q >> 1] >> (16 * c + 8 * (q & 1));
            sumA += (float)(int8_t)(wa & 0xFFu) * (float)PA;
            sumB += (float)(int8_t)(wb & 0xFFu) * (float)PB;
        }
        const float xs = lds_f1(xs_s + blk * 4);
        acc[0] += h2f(dA[0]) * xs * sumA;
        acc[1] += h2f(dB[0]) * xs * sumB;

        const uint32_t T = tile;
        bool tile_done = false;
        if (++blk == bpr) { blk = 0; ++tile; tile_done = true; }
        if (tile_done || it + 1 == n) {
            float v[1][2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float w = acc[r];
                w += __shfl_xor_sync(0xFFFFFFFFu, w, 1);
                w += __shfl_xor_sync(0xFFFFFFFFu, w, 2);
                v[0][r] = w;
                acc[r] = 0.f;
            }
            finish_tile<1, EPI, kWarps>(a, s.spartial, s.sflags, v, T, bpr, u0, u1, U, G, me, warp, lane);
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
    if (!a.scratch_partial || !a.scratch_flags || !a.status) return false;
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
    if (!a.scratch_partial || !a.scratch_flags || !a.status) return false;
    if ((reinterpret_cast<uintptr_t>(a.A) & 15u) || (a.expert_stride & 15u) || (a.K & 255u)) return false;
    if ((a.x_expert_stride & 3u) || (reinterpret_cast<uintptr_t>(a.x) & 15u)) return false;
    const uint32_t bpr = (a.K >> 8) * a.n_used;
    if (smem_bytes6(bpr * 256, 16) > 227 * 1024 || bpr > (uint32_t)(kPrepBlocks * 8)) return false;
    const uint64_t U = (uint64_t)((a.M + 15) / 16) * bpr;
    if ((uint64_t)a.M * bpr * 210u < 4 * kStreamMinBytes) return false;  // small expert sets: latency-bound either way
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
    wa.gflags = a.scratch_flags;
    wa.status = a.status;
    wa.spin_limit = a.spin_limit;
    wa.nseg = a.n_used;
    wa.routing = a.routing;
    wa.n_experts_max = a.n_experts_max;
    wa.expert_stride = a.expert_stride;
    wa.x_slot_stride = a.x_expert_stride;
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
    wa.gflags = a.scratch_flags;
    wa.status = a.status;
    wa.spin_limit = a.spin_limit;
    wa.nseg = 0;
    cudaError_t e = mode == MODE_PLAIN ? launch_cfg6<EPI_PLAIN>(wa, a.a_end, st, a.sm_count)
                                       : launch_cfg6<EPI_SIGMOID_ACC>(wa, a.a_end, st, a.sm_count);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
