// Building blocks of the streaming decode matvec: mbarrier + bulk-copy (TMA 1-D)
// pipeline primitives with bounded waits, the f16 tensor-core MMA used as a
// dot-product engine, and the split-K work partition with its fix-up protocol.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace zc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait with an iteration limit. Returns false when the limit is hit: the caller
// records an error status and leaves its loop instead of spinning forever.
constexpr uint32_t kWaitLimit = 1u << 22;  // each failed try_wait already suspends for a while
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Bulk asynchronous copy global -> this CTA's shared memory, completion counted
// on an mbarrier. Both addresses 16-byte aligned, size a multiple of 16. No
// multicast: every CTA fetches its own bytes.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col). Used as a dot-product engine:
// the 16 A rows are 16 weight rows, columns 0/1 of B hold the two f16 terms of x.
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t h2_bcast(float v) {
    const __half2 h = __float2half2_rn(v);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// (a & mask) | orv in one LOP3
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(orv));
    return d;
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// ---- split-K partition ---------------------------------------------------------------
// Work units are (16-row tile, k-chunk) pairs in tile-major order; CTA c of G owns the
// contiguous unit range [c*U/G, (c+1)*U/G). With G <= U every CTA owns at least one unit.
__device__ __forceinline__ uint64_t part_begin(uint64_t c, uint64_t U, uint64_t G) { return c * U / G; }
// The CTA that owns unit u.
__device__ __forceinline__ uint32_t part_owner(uint64_t u, uint64_t U, uint64_t G) {
    return (uint32_t)(((u + 1) * G + U - 1) / U - 1);
}

}  // namespace zc
