// Prefill dequant-GEMM on the 5th-generation tensor cores: D[n][m] = sum_k W[m][k] * X[n][k].
//
//   W  quantised GGUF rows (Q4_K), read in place and dequantised to bf16 by producer warps straight
//      into the shared-memory layout tcgen05.mma consumes (K-major, 128-byte swizzle)
//   X  bf16 activations [N][stride_b], fetched by TMA (cp.async.bulk.tensor, 128-byte swizzle)
//   D  f32 [N][stride_d]; accumulators live in tensor memory and are read back with tcgen05.ld
//
// One CTA computes a 128-row x BN-token tile. Warp roles (10 warps):
//   warp 0      allocates tensor memory; lane 0 issues tcgen05.mma and the commits
//   warp 1      lane 0 issues the TMA loads of X
//   warps 2-5   dequantise the even 64-column groups (one thread per row), then run the epilogue
//   warps 6-9   dequantise the odd 64-column groups
// Four shared-memory stages of 64 columns; every wait on an mbarrier is bounded and a wait that
// gives up records {1, site} in the status words, raises a CTA-wide flag and lets every role fall
// through to the common exit, where tensor memory is released.
//
// Replaces the reference's mul_mm_q4k.comp / gemm_q4k.metal tile kernels
// (src/compute/dmmv.zig:1045 recordMulMmQ4K).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "kernels.h"
#include "stream_common.cuh"

namespace zc {
namespace {

constexpr int kBM = 128;      // weight rows per tile (= TMEM lanes)
constexpr int kBK = 64;       // columns per stage: 128 bytes of bf16, one swizzle row
constexpr int kStages = 4;
constexpr int kThreads = 320;
constexpr uint32_t kABytes = kBM * kBK * 2;  // 16 KB

template <int BN>
struct Tile {
    static constexpr uint32_t kBBytes = BN * kBK * 2;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kBarOffset = kStages * kStageBytes;
    static constexpr uint32_t kSmemBytes = kBarOffset + 256 + 1024;  // barriers + alignment slack
};

// Barrier block that follows the stages.
struct Bars {
    uint64_t full_a[kStages];
    uint64_t full_b[kStages];
    uint64_t empty[kStages];
    uint64_t accum;
    uint32_t tmem_base;
    volatile uint32_t failed;
};

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]^T, bf16 x bf16 -> f32, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    const uint32_t lo = ((saddr >> 4) & 0x3FFFu) | (1u << 16);         // start address, leading offset (unused) = 1
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);         // stride offset, version 1, SWIZZLE_128B
    return ((uint64_t)hi << 32) | lo;
}

// Instruction descriptor: f32 accumulator, bf16 A and B, both K-major, M = 128, N = BN.
template <int BN>
__host__ __device__ constexpr uint32_t instr_desc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

__device__ __forceinline__ bool wait_or_fail(uint64_t* bar, uint32_t parity, Bars* bars, uint32_t* status,
                                             uint32_t site) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && bars->failed) return false;
    }
    bars->failed = 1;
    if (status) {
        status[0] = 1;
        status[1] = site;
    }
    return false;
}

__device__ __forceinline__ uint32_t bf2_bits(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __nv_bfloat162 bits_bf2(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }

// Four weights (the low nibbles of bytes 0..3 of `nib`, already masked to 0x0F0F0F0F) -> two bf16x2
// words: (128 + q) built by byte permutation (exact in bf16), minus 128, times d*sc, minus dmin*m.
__device__ __forceinline__ void deq4(uint32_t nib, __nv_bfloat162 dsc, __nv_bfloat162 ndm, uint32_t& o0,
                                     uint32_t& o1) {
    const __nv_bfloat162 k128 = bits_bf2(0x43004300u);
    const uint32_t p0 = __byte_perm(nib, 0x43434343u, 0x4140);
    const uint32_t p1 = __byte_perm(nib, 0x43434343u, 0x4342);
    o0 = bf2_bits(__hfma2(__hsub2(bits_bf2(p0), k128), dsc, ndm));
    o1 = bf2_bits(__hfma2(__hsub2(bits_bf2(p1), k128), dsc, ndm));
}

// One 64-column group of a Q4_K row: 32 bytes of nibbles -> 8 chunks of 8 bf16 written to the
// swizzled row `row` of the stage at `a_stage`.
__device__ __forceinline__ void dequant_group_q4k(const uint4& q0, const uint4& q1, float d_sc_lo, float dm_lo,
                                                  float d_sc_hi, float dm_hi, uint8_t* a_stage, int row) {
    const __nv_bfloat162 s_lo = __float2bfloat162_rn(d_sc_lo), m_lo = __float2bfloat162_rn(-dm_lo);
    const __nv_bfloat162 s_hi = __float2bfloat162_rn(d_sc_hi), m_hi = __float2bfloat162_rn(-dm_hi);
    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    uint8_t* rowp = a_stage + row * 128;
    const int sw = row & 7;
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // chunk c: bytes 8c..8c+7 -> low nibbles = columns 8c.., high = 32+8c..
        uint4 lo, hi;
        deq4(w[2 * c] & 0x0F0F0F0Fu, s_lo, m_lo, lo.x, lo.y);
        deq4(w[2 * c + 1] & 0x0F0F0F0Fu, s_lo, m_lo, lo.z, lo.w);
        deq4((w[2 * c] >> 4) & 0x0F0F0F0Fu, s_hi, m_hi, hi.x, hi.y);
        deq4((w[2 * c + 1] >> 4) & 0x0F0F0F0Fu, s_hi, m_hi, hi.z, hi.w);
        *reinterpret_cast<uint4*>(rowp + ((c ^ sw) << 4)) = lo;
        *reinterpret_cast<uint4*>(rowp + (((c + 4) ^ sw) << 4)) = hi;
    }
}

struct GemmArgs {
    const uint8_t* A;
    float* D;
    uint32_t M, N, K;
    uint32_t stride_d;
    uint32_t* status;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_q4k_tc_kernel(const __grid_constant__ CUtensorMap tmap_b, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // swizzle atoms: 1024-byte aligned
    Bars* bars = reinterpret_cast<Bars*>(smem + Tile<BN>::kBarOffset);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t m0 = blockIdx.x * kBM, n0 = blockIdx.y * BN;
    const int n_it = g.K / kBK;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&bars->full_a[s], 4);  // one arrival per producer warp of the owning set
            mbar_init(&bars->full_b[s], 1);
            mbar_init(&bars->empty[s], 1);
        }
        mbar_init(&bars->accum, 1);
        bars->failed = 0;
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(&bars->tmem_base)),
                     "r"((uint32_t)BN)
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
            bool ok = true;
            for (int it = 0; it < n_it && ok; ++it) {
                const int s = it % kStages;
                const uint32_t ph = (it / kStages) & 1;
                ok = wait_or_fail(&bars->full_a[s], ph, bars, g.status, 101) &&
                     wait_or_fail(&bars->full_b[s], ph, bars, g.status, 102);
                if (!ok) break;
                tc_fence_after();
                const uint64_t da = smem_desc(smem_u32(smem + s * Tile<BN>::kStageBytes));
                const uint64_t db = smem_desc(smem_u32(smem + s * Tile<BN>::kStageBytes + kABytes));
#pragma unroll
                for (int k = 0; k < kBK / 16; ++k)  // 16 columns = 32 bytes per instruction
                    umma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, (it | k) ? 1u : 0u);
                umma_commit(&bars->empty[s]);
            }
            umma_commit(&bars->accum);
        }
    } else if (warp == 1) {
        if (lane == 0) {  // ---- TMA loader of X ----
            for (int it = 0; it < n_it; ++it) {
                const int s = it % kStages;
                const uint32_t ph = ((it / kStages) & 1) ^ 1;
                if (!wait_or_fail(&bars->empty[s], ph, bars, g.status, 103)) break;
                mbar_expect_tx(&bars->full_b[s], Tile<BN>::kBBytes);
                tma_load_2d(smem + s * Tile<BN>::kStageBytes + kABytes, &tmap_b, it * kBK, (int)n0, &bars->full_b[s]);
            }
        }
    } else {
        // ---- dequant producers: thread = one row, set h owns the 64-column groups with (it & 1) == h ----
        const int p = tid - 64;
        const int row = p & 127, h = p >> 7;
        const uint32_t grow = min(m0 + (uint32_t)row, g.M - 1);  // rows past M are computed and dropped
        const uint32_t nblk = g.K >> 8;
        const uint8_t* rp = g.A + (uint64_t)grow * nblk * 144u;
        // registers one block ahead: header (d, dmin, 12 scale bytes) and this set's two groups
        uint4 hdr = __ldg(reinterpret_cast<const uint4*>(rp));
        uint4 qa0 = __ldg(reinterpret_cast<const uint4*>(rp + 16 + h * 32));
        uint4 qa1 = __ldg(reinterpret_cast<const uint4*>(rp + 32 + h * 32));
        uint4 qb0 = __ldg(reinterpret_cast<const uint4*>(rp + 80 + h * 32));
        uint4 qb1 = __ldg(reinterpret_cast<const uint4*>(rp + 96 + h * 32));
        bool ok = true;
        for (uint32_t b = 0; b < nblk && ok; ++b) {
            const uint4 chdr = hdr, ca0 = qa0, ca1 = qa1, cb0 = qb0, cb1 = qb1;
            if (b + 1 < nblk) {
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
            for (int half = 0; half < 2; ++half) {  // groups h and h + 2 of the block
                const int grp = h + 2 * half;
                const int it = (int)b * 4 + grp;
                const int s = it % kStages;
                const uint32_t ph = ((it / kStages) & 1) ^ 1;
                uint32_t s0, mn0, s1, mn1;
                scale_min_k4(2 * grp, chdr.y, chdr.z, chdr.w, s0, mn0);
                scale_min_k4(2 * grp + 1, chdr.y, chdr.z, chdr.w, s1, mn1);
                if (!wait_or_fail(&bars->empty[s], ph, bars, g.status, 104)) {
                    ok = false;
                    break;
                }
                dequant_group_q4k(half ? cb0 : ca0, half ? cb1 : ca1, d * (float)s0, dmin * (float)mn0,
                                  d * (float)s1, dmin * (float)mn1, smem + s * Tile<BN>::kStageBytes, row);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->full_a[s]);
            }
        }
        // ---- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----
        if (warp < 6) {
            if (wait_or_fail(&bars->accum, 0, bars, g.status, 105)) {
                __syncwarp();
                tc_fence_after();
                const uint32_t q = warp & 3;
                const uint32_t m = m0 + q * 32 + lane;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
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
                        for (int j = 0; j < 32; ++j) {
                            const uint32_t n = n0 + c * 32 + j;
                            if (n < g.N) g.D[(uint64_t)n * g.stride_d + m] = __uint_as_float(v[j]);
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)BN) : "memory");
    }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

template <int BN>
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
    auto kern = gemm_q4k_tc_kernel<BN>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)Tile<BN>::kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    GemmArgs g{A, D, M, N, K, stride_d, status};
    const dim3 grid((M + kBM - 1) / kBM, (N + BN - 1) / BN);
    kern<<<grid, kThreads, Tile<BN>::kSmemBytes, s>>>(map, g);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_mul_mm(uint32_t type, const uint8_t* A, const void* B, float* D, uint32_t M, uint32_t N,
                          uint32_t K, uint32_t stride_b, uint32_t stride_d, bool act_bf16, uint32_t* status,
                          cudaStream_t s, uint64_t* launches) {
    if (type != T_Q4_K || !act_bf16 || !status) return cudaErrorNotSupported;
    if ((K & 255u) || (stride_b & 7u) || (reinterpret_cast<uintptr_t>(B) & 15u) ||
        (reinterpret_cast<uintptr_t>(A) & 15u))
        return cudaErrorNotSupported;
    if (N < 16) return cudaErrorNotSupported;  // a handful of tokens: the matvec-style kernels are the better fit
    cudaError_t e = N <= 128 ? launch_tile<128>(A, B, D, M, N, K, stride_b, stride_d, status, s)
                             : launch_tile<256>(A, B, D, M, N, K, stride_b, stride_d, status, s);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
