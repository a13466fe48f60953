// Shared device helpers of the streaming kernels: mbarrier primitives with bounded waits (used by the
// tensor-core GEMM pipeline) and the split-K work partition of the streaming matvecs.
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

// one poll that never suspends the thread: for a thread that serves several rings
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Iteration limit of every mbarrier wait: a waiter that reaches it records an error status and leaves
// its loop instead of spinning forever (each failed try_wait already suspends for a while).
constexpr uint32_t kWaitLimit = 1u << 22;

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// ---- split-K partition ---------------------------------------------------------------
// Work units are (16-row tile, k-chunk) pairs in tile-major order; worker (warp) c of G owns the
// contiguous unit range [c*U/G, (c+1)*U/G). With G <= U every worker owns at least one unit.
__device__ __forceinline__ uint64_t part_begin(uint64_t c, uint64_t U, uint64_t G) { return c * U / G; }
// The worker that owns unit u.
__device__ __forceinline__ uint32_t part_owner(uint64_t u, uint64_t U, uint64_t G) {
    return (uint32_t)(((u + 1) * G + U - 1) / U - 1);
}

}  // namespace zc
