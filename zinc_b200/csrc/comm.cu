// One-shot all-reduce of small f32 vectors across the GPUs of one node, over NVLink peer memory.
//
// The tensor-parallel decode step sums a hidden-state vector (16 KB) across ranks twice per layer.
// At that size a collective is pure latency, so it is a single kernel: every rank stores its
// vector into a slot of every peer's receive buffer (plain peer stores), publishes a flag,
// waits (bounded) for the flags of all ranks in its own buffer, and adds the slots in rank
// order, so all ranks compute bit-identical sums. No multicast, no second kernel.
//
// Receive buffer of one rank (cudaMalloc, exported with cudaIpcGetMemHandle, zeroed):
//   data  [2 parities][kCommMaxRanks][kCommSlotBytes]   slot r of parity p <- rank r's vector
//   gather [2 parities][kCommGatherBytes]                all-gather: rank r's slice at r * n floats
//   flags [2 parities][kCommMaxRanks] u32                epoch of the vector in that slot (one set per collective kind)
//   epoch words                                          collectives of each kind this rank has completed
// All ranks issue the same sequence of all-reduces, so the epochs agree. Reduction e uses
// parity e & 1; a rank can be at most one reduction ahead of a peer (it cannot finish e+1 before
// the peer has contributed to it, i.e. finished e), so two parities are enough to keep a slot
// from being overwritten while it is still being read.
//
// The reference is single-GPU; this has no counterpart there.
#include "kernels.h"

namespace zc {
namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Programmatic dependent launch: the kernel may be scheduled while its predecessor drains and lets its
// successor (a streaming matvec, which prefetches weights before it needs the reduced vector) start early;
// nothing is read or written before griddepcontrol.wait has seen every earlier kernel complete.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__global__ void __launch_bounds__(kThreads) allreduce_oneshot_kernel(const CommArgs c, float* buf, uint32_t n) {
    __shared__ uint32_t failed;
    const int tid = threadIdx.x;
    if (tid == 0) failed = 0;
    pdl_enter();
    uint8_t* local = c.peers[c.rank];
    uint32_t* epoch_word = reinterpret_cast<uint32_t*>(local + kCommEpochOffset);
    const uint32_t epoch = *epoch_word + 1;
    const uint32_t parity = epoch & 1u;
    const uint32_t n4 = n >> 2;
    const float4* in = reinterpret_cast<const float4*>(buf);
    // 1. my vector into slot [parity][rank] of every rank's buffer (mine included)
    const size_t slot_off = ((size_t)parity * kCommMaxRanks + c.rank) * kCommSlotBytes;
    for (uint32_t i = tid; i < n4; i += kThreads) {
        const float4 v = in[i];
        for (uint32_t r = 0; r < c.world; ++r)
            reinterpret_cast<float4*>(c.peers[r] + slot_off)[i] = v;
    }
    __threadfence_system();
    __syncthreads();
    // 2. publish, 3. wait for everyone's flag in my own buffer
    if (tid < (int)c.world) {
        uint32_t* remote = reinterpret_cast<uint32_t*>(c.peers[tid] + kCommFlagOffset) + parity * kCommMaxRanks + c.rank;
        st_release_sys(remote, epoch);
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(local + kCommFlagOffset) + parity * kCommMaxRanks + tid;
        uint32_t spins = 0;
        while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
            if (++spins >= c.spin_limit) {
                failed = 1;
                if (c.status) {
                    c.status[0] = 1;
                    c.status[1] = 200u + tid;
                }
                break;
            }
        }
    }
    __syncthreads();
    // A wait gave up: a slot may hold a stale vector, so nothing is summed and the epoch does not advance.
    // The status words carry {1, site}; the host marks the communicator unusable (zc_submit_and_wait).
    if (failed) return;
    // 4. sum the slots in rank order (identical on every rank)
    const uint8_t* slots = local + (size_t)parity * kCommMaxRanks * kCommSlotBytes;
    float4* out = reinterpret_cast<float4*>(buf);
    for (uint32_t i = tid; i < n4; i += kThreads) {
        float4 acc = __ldcg(reinterpret_cast<const float4*>(slots) + i);
        for (uint32_t r = 1; r < c.world; ++r) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(slots + (size_t)r * kCommSlotBytes) + i);
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        out[i] = acc;
    }
    if (tid == 0) *epoch_word = epoch;
}

// All-gather with the same protocol, several CTAs wide (all co-resident: the grid is far smaller than
// the SM count and the kernel neither starts early nor lets its successor start early). Each CTA
// pushes its share of the local slice to every rank; the last CTA to finish pushing publishes the
// flags; every CTA then waits for all ranks' flags and copies its share of the gathered vector out.
constexpr int kGatherCtas = 16;

__global__ void __launch_bounds__(kThreads) allgather_oneshot_kernel(const CommArgs c, const float* src, float* dst,
                                                                     uint32_t n) {
    __shared__ uint32_t s_last, s_failed;
    const int tid = threadIdx.x;
    uint8_t* local = c.peers[c.rank];
    uint32_t* words = reinterpret_cast<uint32_t*>(local + kCommEpochOffset);
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(words + 1) + 1;  // stable until every CTA has left
    const uint32_t parity = epoch & 1u;
    const size_t region = kCommGatherOffset + (size_t)parity * kCommGatherBytes;
    const uint32_t n4 = n >> 2;
    // 1. push my slice
    const float4* in = reinterpret_cast<const float4*>(src);
    for (uint32_t i = blockIdx.x * kThreads + tid; i < n4; i += gridDim.x * kThreads) {
        const float4 v = in[i];
        for (uint32_t r = 0; r < c.world; ++r)
            reinterpret_cast<float4*>(c.peers[r] + region + (size_t)c.rank * n * 4)[i] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (tid == 0) {
        s_failed = 0;
        s_last = atomicAdd(words + 2, 1u) == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (s_last) {  // every CTA's stores are fenced: publish
        if (tid == 0) words[2] = 0;
        if (tid < (int)c.world)
            st_release_sys(reinterpret_cast<uint32_t*>(c.peers[tid] + kCommGatherFlagOffset) + parity * kCommMaxRanks + c.rank,
                           epoch);
    }
    // 2. wait for all ranks
    if (tid < (int)c.world) {
        const uint32_t* mine =
            reinterpret_cast<const uint32_t*>(local + kCommGatherFlagOffset) + parity * kCommMaxRanks + tid;
        uint32_t spins = 0;
        while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
            if (++spins >= c.spin_limit) {
                s_failed = 1;
                if (c.status) {
                    c.status[0] = 1;
                    c.status[1] = 300u + tid;
                }
                break;
            }
        }
    }
    __syncthreads();
    // 3. copy the gathered vector out (not after a wait that gave up: a slice may be stale; the status words
    // carry {1, site} and the host marks the communicator unusable)
    if (!s_failed) {
        const float4* all = reinterpret_cast<const float4*>(local + region);
        float4* out = reinterpret_cast<float4*>(dst);
        const uint32_t total4 = n4 * c.world;
        for (uint32_t i = blockIdx.x * kThreads + tid; i < total4; i += gridDim.x * kThreads) out[i] = __ldcg(all + i);
    }
    __syncthreads();
    if (tid == 0 && atomicAdd(words + 3, 1u) == gridDim.x - 1) {  // last CTA to leave: next epoch
        words[3] = 0;
        words[1] = epoch;
    }
}

__device__ __forceinline__ uint2 ld_volatile_pair(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// The consumer half of the fused exchange as a kernel of its own, for the call sites where the next launch on
// the stream cannot carry it (same loop as consume_pushed in the streaming kernels).
__global__ void __launch_bounds__(256) consume_kernel(const ConsumeArgs c) {
    pdl_enter();
    for (uint32_t i = threadIdx.x * gridDim.x + blockIdx.x; i < c.n; i += blockDim.x * gridDim.x) {
        float s = c.acc ? c.dst[i] : 0.f;
        for (uint32_t r = 0; r < c.world; ++r) {
            uint2* p = c.slots + (size_t)r * kPushMaxFloats + i;
            uint2 q = ld_volatile_pair(p);
            uint32_t spins = 0;
            while (q.y == 0u) {
                if (++spins > c.spin_limit) {
                    c.status[0] = 1;
                    c.status[1] = 400u + r;
                    break;
                }
                q = ld_volatile_pair(p);
            }
            s += __uint_as_float(q.x);
            *p = make_uint2(0u, 0u);
        }
        c.dst[i] = s;
    }
}

}  // namespace

cudaError_t launch_consume(const ConsumeArgs& c, cudaStream_t s, uint64_t* launches) {
    if (c.n == 0) return cudaSuccess;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((c.n + 255) / 256, 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, consume_kernel, c);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

cudaError_t launch_allgather_oneshot(const CommArgs& c, const float* src, float* dst, uint32_t n, cudaStream_t s,
                                     uint64_t* launches) {
    allgather_oneshot_kernel<<<kGatherCtas, kThreads, 0, s>>>(c, src, dst, n);
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

cudaError_t launch_allreduce_oneshot(const CommArgs& c, float* buf, uint32_t n, cudaStream_t s, uint64_t* launches) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, allreduce_oneshot_kernel, c, buf, n);
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
