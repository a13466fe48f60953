// Shared skeleton of the warp-autonomous streaming matvec kernels: launch arguments, the
// asynchronous-copy and int8 tensor-core primitives, the fused epilogues and the ordered
// hand-off of split-K partial sums between workers.
#pragma once

#include "common.cuh"
#include "stream_common.cuh"

namespace zc {
namespace {

// Programmatic dependent launch: let the next kernel of the stream start its prologue while this
// one runs, and wait for the previous kernel's results before touching anything it may have
// written. Both are no-ops for kernels launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

struct WarpArgs {
    const uint8_t* A[2];
    const float* x;
    float* y;
    const float* gate;
    uint32_t M, K, acc_mode;
    uint2* gpartial;     // [workers][32] partial sums published across CTAs as {f32 bits, 1}; {0, 0} = empty,
                         // the reader puts that back. A 64-bit store is one transaction: no flag, no fence.
    uint32_t* status;    // [0] error code, [1] site
    // Grouped launch (several matrices that share x and K, e.g. Q, K and V): segment i covers the
    // 16-row tiles [seg_end[i-1], seg_end[i]). Its pointers and row bound are pre-shifted by the
    // segment's first tile, so that the kernel can index them with the global tile / row number.
    uint32_t nseg;       // 0: single matrix (A[0], y, M)
    uint32_t seg_end[3];
    const uint8_t* segA[3];
    float* segY[3];
    uint32_t segM[3];
    // MoE launch (expert slots chosen by a routing buffer on the device): slot s covers the tiles
    // [s * tiles_per_expert, (s+1) * tiles_per_expert) of the matrices A[i] + routing[s] * expert_stride and
    // writes rows [s * M, (s+1) * M) of y (stream 0) and y2 (stream 1). x is shared by all slots.
    const uint32_t* routing;
    uint64_t expert_stride;
    uint32_t n_experts_max = 0xFFFFFFFFu;  // ids at or beyond it are reported through the status words
    uint32_t tiles_per_expert;
    float* y2;
    uint32_t spin_limit = 1u << 26;  // polls after which a split-K wait gives up (status {1, site})
    uint32_t x_slot_stride;  // MoE down projection: elements between the slots' activation vectors
    PushArgs push;           // EPI_PLAIN: rows go to every rank's receive buffer instead of y
    ConsumeArgs consume;     // pending reduction completed by this launch's threads after the dependency wait
    uint32_t act = 0;        // EPI_PAIR only: 0 write both streams, 1 y = silu(gate) * up, 2 the GPT-OSS form
    const uint8_t* A_sh[2] = {nullptr, nullptr};  // MoE: matrices of the slot whose id is kSharedExpert
    const uint8_t* A_sh_end[2] = {nullptr, nullptr};  // first byte past the buffers that hold them
    // MoE per-expert biases [n_experts][M]: EPI_PAIR adds the slot's expert's rows of bias[0] / bias[1] to the
    // gate / up row; EPI_ACC adds sum_s w_s bias[0][e_s][row]
    const float* bias[2] = {nullptr, nullptr};
    uint32_t late = 0;       // release the dependents after the dependency wait, and read the routing after it
};

// Start of a streaming kernel: release the next kernel of the stream at once, unless this launch was told that
// its predecessor did the same while the routing buffer was still being written. Then the dependency wait comes
// first, so that whatever starts behind this kernel finds every older kernel complete.
__device__ __forceinline__ void pdl_prologue(const WarpArgs& a) {
    if (a.late) pdl_wait();
    pdl_launch_dependents();
}
// The same in two steps, for kernels with set-up work that touches nothing another kernel writes: pdl_begin at
// the start, pdl_late before the first read of the routing buffer (or of anything else a predecessor writes).
__device__ __forceinline__ void pdl_begin(const WarpArgs& a) {
    if (!a.late) pdl_launch_dependents();
}
__device__ __forceinline__ void pdl_late(const WarpArgs& a) {
    if (a.late) {
        pdl_wait();
        pdl_launch_dependents();
    }
}

// The activation a fused gate + up launch applies (src/shaders/swiglu.comp:25-33, swiglu_oai.comp:24-34).
__device__ __forceinline__ float gate_up_act(uint32_t act, float gate, float up) {
    if (act == 2) {
        const float g = fminf(gate, 7.0f);
        const float u = fmaxf(-7.0f, fminf(up, 7.0f));
        return (g / (1.0f + expf(1.702f * (-g)))) * (u + 1.0f);
    }
    return (gate / (1.0f + expf(-gate))) * up;
}


__device__ __forceinline__ uint4 lds128(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// Loads through the shared window (32-bit addresses from smem_u32): the pointers of the carved shared
// memory go through integer arithmetic, after which the compiler can no longer prove the address space
// and would fall back to generic loads.
__device__ __forceinline__ uint4 lds_v4(uint32_t saddr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
    return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t saddr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(saddr));
    return v;
}
__device__ __forceinline__ float lds_f1(uint32_t saddr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(saddr));
    return v;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// D(16x8,s32) += A(16x32,s8,row) * B(32x8,s8,col)
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same with unsigned A (quants that are stored with an offset, e.g. Q6_K's 0..63)
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint2 ld_volatile_u2(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// The consumer half of the fused exchange, spread over the grid: element i belongs to thread i / n_ctas of CTA
// i % n_ctas. Waits (bounded) for the tagged value of every rank, adds them in rank order and clears the tags.
__device__ __forceinline__ void consume_pushed(const ConsumeArgs& c, uint32_t cta, uint32_t n_ctas, uint32_t tid,
                                               uint32_t n_threads) {
    for (uint32_t i = tid * n_ctas + cta; i < c.n; i += n_threads * n_ctas) {
        float s = c.acc ? c.dst[i] : 0.f;
        for (uint32_t r = 0; r < c.world; ++r) {
            uint2* p = c.slots + (size_t)r * kPushMaxFloats + i;
            uint2 q = ld_volatile_u2(p);
            uint32_t spins = 0;
            while (q.y == 0u) {
                if (++spins > c.spin_limit) {
                    c.status[0] = 1;
                    c.status[1] = 400u + r;
                    break;
                }
                q = ld_volatile_u2(p);
            }
            s += __uint_as_float(q.x);
            *p = make_uint2(0u, 0u);
        }
        c.dst[i] = s;
    }
}

enum { EPI_PLAIN = 0, EPI_GATE_UP = 1, EPI_SIGMOID_ACC = 2, EPI_PAIR = 3, EPI_ACC = 4 };

// Where the rows of one tile go: the launch's own outputs, or those of the segment / expert slot the tile
// belongs to, moved back by the segment's first row so that the global row number indexes them.
struct RowOut {
    float* y;
    float* y2;
    uint32_t M;       // row bound in that indexing
    const float* b0;  // EPI_PAIR: the slot's expert's gate / up bias rows (null: none); EPI_ACC: the bias table
    const float* b1;
};
__device__ __forceinline__ RowOut row_out(const WarpArgs& a) { return RowOut{a.y, a.y2, a.M, a.bias[0], a.bias[1]}; }

// Does this launch add to y (and so needs its old value)?
template <int EPI>
__device__ __forceinline__ bool epi_accumulates(const WarpArgs& a) {
    if constexpr (EPI == EPI_ACC || EPI == EPI_SIGMOID_ACC) return true;
    if constexpr (EPI == EPI_PLAIN) return a.acc_mode != 0 && a.push.world == 0;
    return false;
}

// yold: the value of y[row] before this launch, for the accumulating forms (read by the caller ahead of time,
// so that the round trip overlaps the wait for the other workers' partial sums; one warp owns a row's result)
template <int NS, int EPI>
__device__ __forceinline__ void write_row(const WarpArgs& a, const RowOut& o, uint32_t row, const float (&v)[NS],
                                          float yold) {
    if (row >= o.M) return;
    if constexpr (EPI == EPI_GATE_UP) {
        o.y[row] = (v[0] / (1.0f + expf(-v[0]))) * v[1];
    } else if constexpr (EPI == EPI_ACC) {  // y += result, whatever acc_mode says
        float b = 0.f;
        if (o.b0) {  // MoE down projection: the selected experts' biases, weighted like their products
            for (uint32_t s = 0; s < a.nseg; ++s) {
                const uint32_t e = __ldg(a.routing + s);
                if (e < a.n_experts_max)
                    b = fmaf(__uint_as_float(__ldg(a.routing + a.nseg + s)), __ldg(o.b0 + (size_t)e * a.M + row), b);
            }
        }
        o.y[row] = yold + (v[0] + b);
    } else if constexpr (EPI == EPI_PAIR) {  // two streams (MoE gate and up rows): both outputs, or their activation
        const float vg = o.b0 ? v[0] + __ldg(o.b0 + row) : v[0];
        const float vu = o.b1 ? v[NS - 1] + __ldg(o.b1 + row) : v[NS - 1];
        if (a.act) {
            o.y[row] = gate_up_act(a.act, vg, vu);
        } else {
            o.y[row] = vg;
            o.y2[row] = vu;
        }
    } else if constexpr (EPI == EPI_SIGMOID_ACC) {
        o.y[row] = yold + (1.0f / (1.0f + expf(-__ldg(a.gate)))) * v[0];
    } else {
        if (a.push.world) {
            const uint2 pv = make_uint2(__float_as_uint(v[0]), 1u);
            for (uint32_t r = 0; r < a.push.world; ++r) a.push.peers[r][row] = pv;
        } else {
            o.y[row] = a.acc_mode ? yold + v[0] : v[0];
        }
    }
}



// Ends a tile for this warp. v[i][r]: sums of stream i for rows g (r = 0) and g+8 (r = 1), already
// reduced over the four lanes of a row.
template <int NS, int EPI, int kWarps>
__device__ __forceinline__ void finish_tile(const WarpArgs& a, const RowOut& o, float* spartial, volatile uint32_t* sflags, float (&v)[NS][2], uint32_t T,
                                            uint32_t upt_all, uint32_t u0, uint32_t u1, uint32_t U, uint32_t G,
                                            uint32_t me, int warp, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const uint32_t first = T * upt_all, last = first + upt_all - 1;
    if (u0 > first) {
        // not the first contributor: publish the partial sums for the worker that owns `first`
        const uint32_t fin = part_owner(first, U, G);
        if (fin / kWarps == blockIdx.x) {  // same CTA: shared memory and a flag
            float* dst = spartial + warp * 32;
            if (t == 0) {
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                    dst[i * 16 + g] = v[i][0];
                    dst[i * 16 + g + 8] = v[i][1];
                }
                __threadfence_block();
            }
            __syncwarp();
            if (lane == 0) sflags[warp] = 1u;
        } else if (t == 0) {  // another CTA: value and tag travel together
            uint2* dst = a.gpartial + (size_t)me * 32;
#pragma unroll
            for (int i = 0; i < NS; ++i) {
                dst[i * 16 + g] = make_uint2(__float_as_uint(v[i][0]), 1u);
                dst[i * 16 + g + 8] = make_uint2(__float_as_uint(v[i][1]), 1u);
            }
        }
        return;
    }
    // the old values of the rows this warp completes, requested before any waiting
    float yold0 = 0.f, yold1 = 0.f;
    if (t == 0 && epi_accumulates<EPI>(a)) {
        if (T * 16 + g < o.M) yold0 = o.y[T * 16 + g];
        if (T * 16 + g + 8 < o.M) yold1 = o.y[T * 16 + g + 8];
    }
    if (last >= u1) {
        // first contributor of a tile that continues in later workers. They published early (the
        // tile is the first thing they work on). Lane t of each row adds parts t, t+4, ... (the order is
        // fixed by lane index, not by timing): parts from this CTA after their flag is up, parts from
        // other CTAs by polling the tagged values themselves, every wait bounded.
        const uint32_t cl = part_owner(last, U, G);
        float w[NS][2];
#pragma unroll
        for (int i = 0; i < NS; ++i) w[i][0] = w[i][1] = 0.f;
        bool gave_up = false;
        // kGroup parts of this lane at a time: the first read of every value a group needs from other CTAs is
        // issued before any of them is waited for (a tile with many parts would otherwise pay one round trip
        // through L2 per part and row)
        constexpr int kGroup = NS == 1 ? 6 : 2;
        for (uint32_t c0 = me + 1 + t; c0 <= cl; c0 += 4 * kGroup) {
            uint2 q[kGroup][NS][2];
#pragma unroll
            for (int p = 0; p < kGroup; ++p) {
                const uint32_t c = c0 + 4 * p;
                if (c <= cl && c / kWarps != blockIdx.x) {
                    const uint2* src = a.gpartial + (size_t)c * 32;
#pragma unroll
                    for (int i = 0; i < NS; ++i) {
                        q[p][i][0] = ld_volatile_u2(src + i * 16 + g);
                        q[p][i][1] = ld_volatile_u2(src + i * 16 + g + 8);
                    }
                }
            }
#pragma unroll
            for (int p = 0; p < kGroup; ++p) {
                const uint32_t c = c0 + 4 * p;
                if (c > cl) break;
                if (c / kWarps == blockIdx.x) {
                    volatile uint32_t* flag = sflags + (c % kWarps);
                    uint32_t spins = 0;
                    while (*flag == 0u) {
                        if (++spins > a.spin_limit) { gave_up = true; break; }
                    }
                    __threadfence_block();
                    const float* src = spartial + (c % kWarps) * 32;
#pragma unroll
                    for (int i = 0; i < NS; ++i) {
                        w[i][0] += *reinterpret_cast<const volatile float*>(src + i * 16 + g);
                        w[i][1] += *reinterpret_cast<const volatile float*>(src + i * 16 + g + 8);
                    }
                } else {
                    uint2* src = a.gpartial + (size_t)c * 32;
#pragma unroll
                    for (int i = 0; i < NS; ++i) {
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            uint2* ptr = src + i * 16 + g + 8 * r;
                            uint2 v2 = q[p][i][r];
                            uint32_t spins = 0;
                            while (v2.y == 0u) {
                                if (++spins > a.spin_limit) { gave_up = true; break; }
                                v2 = ld_volatile_u2(ptr);
                            }
                            w[i][r] += __uint_as_float(v2.x);
                            *ptr = make_uint2(0u, 0u);  // empty again for the next launch
                        }
                    }
                }
            }
        }
        if (gave_up) { a.status[0] = 1; a.status[1] = 3; }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < NS; ++i) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float q = w[i][r];
                q += __shfl_xor_sync(0xFFFFFFFFu, q, 1);
                q += __shfl_xor_sync(0xFFFFFFFFu, q, 2);
                v[i][r] += q;
            }
        }
    }
    if (t == 0) {
        float r0[NS], r1[NS];
#pragma unroll
        for (int i = 0; i < NS; ++i) { r0[i] = v[i][0]; r1[i] = v[i][1]; }
        write_row<NS, EPI>(a, o, T * 16 + g, r0, yold0);
        write_row<NS, EPI>(a, o, T * 16 + g + 8, r1, yold1);
    }
}

// Launch with programmatic stream serialization: the kernel may begin while its predecessor
// in the stream is still running and synchronises on it with pdl_wait().
template <typename Kern>
inline cudaError_t launch_pdl(Kern kern, uint32_t grid, uint32_t block, size_t smem, cudaStream_t st,
                              const WarpArgs& a) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, a);
}

}  // namespace
}  // namespace zc
