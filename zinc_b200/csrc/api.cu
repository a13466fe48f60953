// C ABI of the library: context, argument validation, dispatch to the kernels.
// Nothing here computes on the CPU; a call either enqueues CUDA work on the
// context's stream or returns an error status.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

#include "../../include/zinc_cuda.h"
#include "common.cuh"
#include "kernels.h"

namespace zc {
cudaError_t launch_mul_mm_simple(uint32_t type, const uint8_t* A, const void* B, float* D, uint32_t M, uint32_t N,
                                 uint32_t K, uint32_t stride_b, uint32_t stride_d, bool act_bf16, cudaStream_t s,
                                 uint64_t* launches);
}

struct zc_ctx {
    int device = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;
    uint64_t launches = 0;
    uint32_t* status_host = nullptr;  // pinned, mapped: deferred device-side status words
    uint32_t* status_dev = nullptr;
    uint2* scratch_partial = nullptr;  // split-K partial sums of the streaming matvecs, tagged (zero between launches)
    uint2* router_tagged = nullptr;      // 1024 tagged logits of the fused router + selection kernel (zero between launches)
    uint64_t router_mark = 0;            // value of `launches` right after that kernel's last launch (0: never)
    float* merge_scratch = nullptr;      // kMergeScratchFloats f32: a merged attention vector on its way to a matvec
    uint32_t* gemm_flags = nullptr;      // kGemmTileFlags words: tiles of a prefill GEMM that are summed through memory
    int sm_count = 0;
    // tensor-parallel peer exchange (zc_comm_*)
    zc::CommArgs comm;
    uint8_t* comm_local = nullptr;
    bool comm_open[zc::kCommMaxRanks] = {false};
    bool comm_broken = false;          // a wait for a peer gave up: epochs no longer agree across ranks
    zc::ConsumeArgs pending;           // pushed vectors not yet reduced (n != 0): the next call completes it
    uint32_t push_parity = 0;          // receive-buffer half the next push uses
    uint32_t wait_limit = 0;           // 0: every kernel family's default; else polls per device-side wait
    // caller-owned scratch for the grouped MoE prefill path (zc_set_workspace)
    void* workspace = nullptr;
    uint64_t workspace_size = 0;
    char err[512] = {0};
};

namespace {

using namespace zc;

constexpr uint32_t kMergeScratchFloats = 16384;
constexpr size_t kRouterTaggedBytes = 1024 * sizeof(uint2);
constexpr uint32_t kGemmTileFlags = 32768;  // two per 256 x 512 tile of a prefill GEMM split over CTA pairs
constexpr size_t kScratchBytes =
    kStreamPartialBytes + kRouterTaggedBytes + kMergeScratchFloats * sizeof(float) + kGemmTileFlags * sizeof(uint32_t);

int32_t fail(zc_ctx* ctx, int32_t code, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

int32_t cuda_fail(zc_ctx* ctx, cudaError_t e, const char* what) {
    if (e == cudaErrorNotSupported) return fail(ctx, ZC_ERR_UNSUPPORTED_TYPE, "%s: unsupported quant type", what);
    if (e == cudaErrorMemoryAllocation) return fail(ctx, ZC_ERR_OOM, "%s: %s", what, cudaGetErrorString(e));
    return fail(ctx, ZC_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool dmmv_type_ok(uint32_t t) {
    switch (t) {
        case T_Q4_K: case T_MXFP4: case T_Q5_0: case T_Q5_1: case T_Q5_K:
        case T_Q6_K: case T_Q8_0: case T_F16: case T_F32: return true;
        default: return false;
    }
}

inline uint64_t row_bytes_of(uint32_t type, uint32_t K) {
    return (uint64_t)(K / block_size(type)) * bytes_per_block(type);
}

inline bool range_ok(uint64_t offset, uint64_t need, uint64_t size) {
    return offset <= size && need <= size - offset;
}

inline bool aligned(const void* p, uint64_t off, uint64_t a) {
    return ((reinterpret_cast<uintptr_t>(p) + off) % a) == 0;
}

// Entry of a call that may carry a pending reduction of pushed vectors in its own kernel.
#define ZC_ENTER_CARRY(ctx)                                                        \
    do {                                                                           \
        if (!(ctx)) return ZC_ERR_INVALID_ARG;                                     \
        cudaError_t e_ = cudaSetDevice((ctx)->device);                             \
        if (e_ != cudaSuccess) return cuda_fail((ctx), e_, "cudaSetDevice");       \
    } while (0)
// Entry of every other call: a pending reduction is completed by a small kernel first, so that whatever
// the call does comes after it in stream order.
#define ZC_ENTER(ctx)                                                              \
    do {                                                                           \
        ZC_ENTER_CARRY(ctx);                                                       \
        const int32_t f_ = flush_pending(ctx);                                     \
        if (f_ != ZC_OK) return f_;                                                \
    } while (0)

int32_t flush_pending(zc_ctx* ctx) {
    if (ctx->pending.n == 0) return ZC_OK;
    const zc::ConsumeArgs c = ctx->pending;
    ctx->pending = zc::ConsumeArgs();
    const cudaError_t e = zc::launch_consume(c, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, "completing a pushed reduction");
}

// Hands a pending reduction to the launch described by `a` (which completes it in its own kernel, or in a small
// kernel in front of it), unless that launch reads or writes the vector being reduced.
inline int32_t take_pending(zc_ctx* ctx, DmmvArgs& a) {
    if (ctx->pending.n == 0) return ZC_OK;
    const uintptr_t lo = reinterpret_cast<uintptr_t>(ctx->pending.dst), hi = lo + (uintptr_t)ctx->pending.n * 4;
    auto overlaps = [&](const void* p, uint64_t bytes) {
        const uintptr_t q = reinterpret_cast<uintptr_t>(p);
        return p != nullptr && q < hi && lo < q + bytes;
    };
    if (overlaps(a.x, (uint64_t)a.K * 4) || overlaps(a.y, (uint64_t)a.M * 4)) return flush_pending(ctx);
    a.consume = ctx->pending;
    ctx->pending = zc::ConsumeArgs();
    return ZC_OK;
}

// Common checks of one matvec-shaped call.
int32_t check_mat(zc_ctx* ctx, const char* fn, uint32_t type, const void* A, uint64_t a_size, uint64_t a_offset,
                  uint64_t a_bytes, uint32_t M, uint32_t K) {
    if (!dmmv_type_ok(type)) return fail(ctx, ZC_ERR_UNSUPPORTED_TYPE, "%s: unsupported quant type %u", fn, type);
    if (!A) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: null weight pointer", fn);
    if (M == 0 || K == 0) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: M and K must be non-zero", fn);
    if (K % block_size(type) != 0)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: K=%u is not a multiple of the block size %u", fn, K, block_size(type));
    if (!range_ok(a_offset, a_bytes, a_size))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: weights need %llu bytes at offset %llu, buffer has %llu", fn,
                    (unsigned long long)a_bytes, (unsigned long long)a_offset, (unsigned long long)a_size);
    const uint64_t al = (type == T_F32) ? 4 : (type == T_F16 || type == T_Q6_K || type == T_Q8_0 || type == T_Q5_0) ? 2
                        : (type == T_MXFP4) ? 1 : 4;
    if (!aligned(A, a_offset, al))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: weight address must be %llu-byte aligned", fn, (unsigned long long)al);
    return ZC_OK;
}

int32_t check_vec(zc_ctx* ctx, const char* fn, const char* name, const void* p, uint64_t size, uint64_t offset,
                  uint64_t need, uint64_t align) {
    if (!p) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: null %s pointer", fn, name);
    if (!range_ok(offset, need, size))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: %s needs %llu bytes at offset %llu, buffer has %llu", fn, name,
                    (unsigned long long)need, (unsigned long long)offset, (unsigned long long)size);
    if (!aligned(p, offset, align))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: %s address must be %llu-byte aligned", fn, name,
                    (unsigned long long)align);
    return ZC_OK;
}

#define ZC_TRY(expr)                   \
    do {                               \
        const int32_t rc_ = (expr);    \
        if (rc_ != ZC_OK) return rc_;  \
    } while (0)

inline const uint8_t* u8(const void* p, uint64_t off) { return static_cast<const uint8_t*>(p) + off; }
inline const float* f32p(const void* p, uint64_t off) {
    return reinterpret_cast<const float*>(static_cast<const uint8_t*>(p) + off);
}
inline float* f32m(void* p, uint64_t off) { return reinterpret_cast<float*>(static_cast<uint8_t*>(p) + off); }

inline void attach_scratch(zc_ctx* ctx, DmmvArgs& a) {
    a.scratch_partial = ctx->scratch_partial;
    a.status = ctx->status_dev;
    if (ctx->wait_limit) a.spin_limit = ctx->wait_limit;
    a.sm_count = ctx->sm_count;
    // nothing was launched since the fused router + selection kernel, which lets its successor start early:
    // that successor must order itself behind it before it trusts the routing buffer
    a.late = ctx->router_mark != 0 && ctx->router_mark == ctx->launches;
}

// Experts a stacked weight buffer holds: ids read from a device-side routing buffer must stay below it.
inline uint32_t experts_in_buffer(uint64_t a_size, uint64_t expert_bytes, uint64_t expert_stride) {
    if (a_size < expert_bytes || expert_stride == 0) return 0;
    const uint64_t n = (a_size - expert_bytes) / expert_stride + 1;
    return n > 0xFFFFFFFFull ? 0xFFFFFFFFu : (uint32_t)n;
}

int32_t comm_usable(zc_ctx* ctx, const char* fn) {
    if (!ctx->comm_local) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: no communicator (zc_comm_init / zc_comm_connect)", fn);
    if (ctx->comm_broken)
        return fail(ctx, ZC_ERR_TIMEOUT, "%s: an earlier exchange gave up waiting for a peer; destroy the communicator "
                    "and set it up again on every rank", fn);
    for (uint32_t r = 0; r < ctx->comm.world; ++r)
        if (!ctx->comm.peers[r]) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: rank %u is not connected", fn, r);
    ctx->comm.spin_limit = ctx->wait_limit ? ctx->wait_limit : (1u << 24);
    return ZC_OK;
}

}  // namespace

extern "C" {

int32_t zc_set_wait_limit(zc_ctx* ctx, uint32_t polls) {
    if (!ctx) return ZC_ERR_INVALID_ARG;
    ctx->wait_limit = polls;
    return ZC_OK;
}

int32_t zc_init(int32_t device, zc_ctx** out_ctx) {
    if (!out_ctx) return ZC_ERR_INVALID_ARG;
    *out_ctx = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0 || device < 0 || device >= n) return ZC_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return ZC_ERR_CUDA;
    if (prop.major != 10) return ZC_ERR_NOT_LOADED;  // kernels are built for sm_100a only
    if (cudaSetDevice(device) != cudaSuccess) return ZC_ERR_CUDA;
    zc_ctx* ctx = new (std::nothrow) zc_ctx();
    if (!ctx) return ZC_ERR_OOM;
    ctx->device = device;
    if (cudaStreamCreateWithFlags(&ctx->own_stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return ZC_ERR_CUDA;
    }
    ctx->stream = ctx->own_stream;
    if (cudaHostAlloc(reinterpret_cast<void**>(&ctx->status_host), 256, cudaHostAllocMapped) != cudaSuccess ||
        cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->status_dev), ctx->status_host, 0) != cudaSuccess) {
        cudaStreamDestroy(ctx->own_stream);
        delete ctx;
        return ZC_ERR_OOM;
    }
    memset(ctx->status_host, 0, 256);
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaMalloc(reinterpret_cast<void**>(&ctx->scratch_partial), kScratchBytes) != cudaSuccess ||
        cudaMemset(ctx->scratch_partial, 0, kScratchBytes) != cudaSuccess) {
        if (ctx->scratch_partial) cudaFree(ctx->scratch_partial);
        cudaFreeHost(ctx->status_host);
        cudaStreamDestroy(ctx->own_stream);
        delete ctx;
        return ZC_ERR_OOM;
    }
    ctx->router_tagged = reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(ctx->scratch_partial) + kStreamPartialBytes);
    ctx->merge_scratch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ctx->scratch_partial) + kStreamPartialBytes +
                                                  kRouterTaggedBytes);
    ctx->gemm_flags = reinterpret_cast<uint32_t*>(ctx->merge_scratch + kMergeScratchFloats);
    *out_ctx = ctx;
    return ZC_OK;
}

int32_t zc_destroy(zc_ctx* ctx) {
    if (!ctx) return ZC_ERR_INVALID_ARG;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    zc_comm_destroy(ctx);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    if (ctx->scratch_partial) cudaFree(ctx->scratch_partial);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return ZC_OK;
}

int32_t zc_comm_init(zc_ctx* ctx, uint32_t rank, uint32_t world, uint8_t* out_handle) {
    ZC_ENTER(ctx);
    const char* fn = "zc_comm_init";
    if (world < 2 || world > kCommMaxRanks || rank >= world || !out_handle)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: need 2 <= world <= %u, rank < world and a 64-byte handle buffer", fn,
                    kCommMaxRanks);
    if (ctx->comm_local) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: already initialised", fn);
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&ctx->comm_local), kCommBufBytes);
    if (e != cudaSuccess) return cuda_fail(ctx, e, fn);
    e = cudaMemset(ctx->comm_local, 0, kCommBufBytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ctx->comm_local);
    if (e != cudaSuccess) {
        cudaFree(ctx->comm_local);
        ctx->comm_local = nullptr;
        return cuda_fail(ctx, e, fn);
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(out_handle, &h, 64);
    ctx->comm = CommArgs();
    ctx->comm.rank = rank;
    ctx->comm.world = world;
    ctx->comm.status = ctx->status_dev;
    ctx->comm.peers[rank] = ctx->comm_local;
    return ZC_OK;
}

int32_t zc_comm_connect(zc_ctx* ctx, const uint8_t* all_handles) {
    ZC_ENTER(ctx);
    const char* fn = "zc_comm_connect";
    if (!ctx->comm_local || !all_handles) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: call zc_comm_init first", fn);
    for (uint32_t r = 0; r < ctx->comm.world; ++r) {
        if (r == ctx->comm.rank || ctx->comm_open[r] || ctx->comm.peers[r]) continue;  // self, open, or lent locally
        cudaIpcMemHandle_t h;
        memcpy(&h, all_handles + (size_t)r * 64, 64);
        void* p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return cuda_fail(ctx, e, fn);
        ctx->comm.peers[r] = static_cast<uint8_t*>(p);
        ctx->comm_open[r] = true;
    }
    return ZC_OK;
}

int32_t zc_allreduce_sum_f32(zc_ctx* ctx, void* buf, uint64_t buf_size, uint64_t offset, uint32_t n) {
    ZC_ENTER(ctx);
    const char* fn = "zc_allreduce_sum_f32";
    ZC_TRY(comm_usable(ctx, fn));
    if (n == 0 || (n & 3u) || (uint64_t)n * 4 > kCommSlotBytes)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: n=%u must be a non-zero multiple of 4, at most %llu", fn, n,
                    (unsigned long long)(kCommSlotBytes / 4));
    ZC_TRY(check_vec(ctx, fn, "buf", buf, buf_size, offset, (uint64_t)n * 4, 16));
    const cudaError_t e = launch_allreduce_oneshot(ctx->comm, f32m(buf, offset), n, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_allgather_f32(zc_ctx* ctx, const void* src, uint64_t src_size, uint64_t src_offset, void* dst,
                         uint64_t dst_size, uint64_t dst_offset, uint32_t n) {
    ZC_ENTER(ctx);
    const char* fn = "zc_allgather_f32";
    ZC_TRY(comm_usable(ctx, fn));
    if (n == 0 || (n & 3u) || (uint64_t)n * 4 * ctx->comm.world > kCommGatherBytes)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: n=%u must be a non-zero multiple of 4 with world * n <= %llu", fn, n,
                    (unsigned long long)(kCommGatherBytes / 4));
    ZC_TRY(check_vec(ctx, fn, "src", src, src_size, src_offset, (uint64_t)n * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "dst", dst, dst_size, dst_offset, (uint64_t)n * 4 * ctx->comm.world, 16));
    const cudaError_t e = launch_allgather_oneshot(ctx->comm, f32p(src, src_offset), f32m(dst, dst_offset), n,
                                                   ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_comm_destroy(zc_ctx* ctx) {
    ZC_ENTER(ctx);
    if (!ctx->comm_local) return ZC_OK;
    cudaStreamSynchronize(ctx->stream);
    for (uint32_t r = 0; r < kCommMaxRanks; ++r)
        if (ctx->comm_open[r]) {
            cudaIpcCloseMemHandle(ctx->comm.peers[r]);
            ctx->comm_open[r] = false;
        }
    cudaFree(ctx->comm_local);
    ctx->comm_local = nullptr;
    ctx->comm = CommArgs();
    ctx->comm_broken = false;
    ctx->push_parity = 0;
    return ZC_OK;
}

int32_t zc_comm_connect_local(zc_ctx* ctx, uint32_t rank, void* receive_buffer, uint64_t size) {
    ZC_ENTER(ctx);
    const char* fn = "zc_comm_connect_local";
    if (!ctx->comm_local) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: call zc_comm_init first", fn);
    if (rank >= ctx->comm.world || rank == ctx->comm.rank || ctx->comm_open[rank])
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: rank %u is this rank, out of range or already connected", fn, rank);
    if (!receive_buffer || size < kCommBufBytes || (reinterpret_cast<uintptr_t>(receive_buffer) & 255u))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: need a 256-byte aligned device buffer of at least %llu bytes", fn,
                    (unsigned long long)kCommBufBytes);
    ctx->comm.peers[rank] = static_cast<uint8_t*>(receive_buffer);  // borrowed: never closed or freed here
    return ZC_OK;
}

uint64_t zc_comm_buffer_bytes(void) { return kCommBufBytes; }

int32_t zc_set_stream(zc_ctx* ctx, void* cuda_stream) {
    if (!ctx) return ZC_ERR_INVALID_ARG;
    ctx->stream = static_cast<cudaStream_t>(cuda_stream);  // NULL is CUDA's default stream
    return ZC_OK;
}

int32_t zc_use_own_stream(zc_ctx* ctx) {
    if (!ctx) return ZC_ERR_INVALID_ARG;
    ctx->stream = ctx->own_stream;
    return ZC_OK;
}

void* zc_get_stream(zc_ctx* ctx) { return ctx ? static_cast<void*>(ctx->stream) : nullptr; }

const char* zc_last_error(zc_ctx* ctx) { return ctx ? ctx->err : "null context"; }

const char* zc_status_string(int32_t s) {
    switch (s) {
        case ZC_OK: return "ok";
        case ZC_ERR_UNSUPPORTED_TYPE: return "unsupported quant type";
        case ZC_ERR_NOT_LOADED: return "kernel not loaded (device is not sm_100)";
        case ZC_ERR_INVALID_ARG: return "invalid argument";
        case ZC_ERR_OOM: return "out of memory";
        case ZC_ERR_CUDA: return "CUDA error";
        case ZC_ERR_TIMEOUT: return "device-side wait timed out";
        default: return "unknown status";
    }
}

uint64_t zc_launch_count(zc_ctx* ctx) { return ctx ? ctx->launches : 0; }

int32_t zc_alloc(zc_ctx* ctx, uint64_t bytes, void** out_dptr) {
    ZC_ENTER(ctx);
    if (!out_dptr || bytes == 0) return fail(ctx, ZC_ERR_INVALID_ARG, "zc_alloc: bad arguments");
    cudaError_t e = cudaMalloc(out_dptr, bytes);
    if (e != cudaSuccess) {
        *out_dptr = nullptr;
        return cuda_fail(ctx, e, "zc_alloc");
    }
    return ZC_OK;
}

int32_t zc_free(zc_ctx* ctx, void* dptr) {
    ZC_ENTER(ctx);
    if (!dptr) return ZC_OK;
    cudaError_t e = cudaFree(dptr);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, "zc_free");
}

int32_t zc_upload(zc_ctx* ctx, void* dst, uint64_t dst_offset, const void* host_src, uint64_t bytes) {
    ZC_ENTER(ctx);
    if (!dst || (!host_src && bytes)) return fail(ctx, ZC_ERR_INVALID_ARG, "zc_upload: null pointer");
    if (bytes == 0) return ZC_OK;
    cudaError_t e = cudaMemcpyAsync(static_cast<uint8_t*>(dst) + dst_offset, host_src, bytes, cudaMemcpyHostToDevice,
                                    ctx->stream);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, "zc_upload");
}

int32_t zc_download(zc_ctx* ctx, void* host_dst, const void* src, uint64_t src_offset, uint64_t bytes) {
    ZC_ENTER(ctx);
    if (!src || (!host_dst && bytes)) return fail(ctx, ZC_ERR_INVALID_ARG, "zc_download: null pointer");
    if (bytes == 0) return ZC_OK;
    cudaError_t e = cudaMemcpyAsync(host_dst, static_cast<const uint8_t*>(src) + src_offset, bytes,
                                    cudaMemcpyDeviceToHost, ctx->stream);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, "zc_download");
}

int32_t zc_memset(zc_ctx* ctx, void* dst, uint64_t dst_offset, int32_t byte_value, uint64_t bytes) {
    ZC_ENTER(ctx);
    if (!dst) return fail(ctx, ZC_ERR_INVALID_ARG, "zc_memset: null pointer");
    if (bytes == 0) return ZC_OK;
    cudaError_t e = cudaMemsetAsync(static_cast<uint8_t*>(dst) + dst_offset, byte_value, bytes, ctx->stream);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, "zc_memset");
}

int32_t zc_barrier(zc_ctx* ctx) { return ctx ? ZC_OK : ZC_ERR_INVALID_ARG; }

int32_t zc_submit_and_wait(zc_ctx* ctx) {
    ZC_ENTER(ctx);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "zc_submit_and_wait");
    if (ctx->status_host[0] != 0) {
        const uint32_t code = ctx->status_host[0], where = ctx->status_host[1];
        ctx->status_host[0] = 0;
        ctx->status_host[1] = 0;
        if (code == 2)
            return fail(ctx, ZC_ERR_INVALID_ARG,
                        "a routing buffer named expert %u, which the weight buffer does not hold; the results of that "
                        "call are invalid", where);
        // A wait gave up. Tagged partial sums may be left behind and would be taken for fresh ones by the next
        // streaming matvec: clear them. A peer exchange that gave up leaves the ranks' epochs out
        // of step: the communicator refuses further collectives until it is destroyed and set up again.
        cudaMemsetAsync(ctx->scratch_partial, 0, kStreamPartialBytes + kRouterTaggedBytes, ctx->stream);
        cudaStreamSynchronize(ctx->stream);
        if (where >= 200 && ctx->comm_local) ctx->comm_broken = true;
        return fail(ctx, ZC_ERR_TIMEOUT, "device-side wait gave up (code %u, site %u)", code, where);
    }
    return ZC_OK;
}

// ---- pre-recorded op sequences ------------------------------------------------------------
int32_t zc_begin_record(zc_ctx* ctx) {
    ZC_ENTER(ctx);
    cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, "zc_begin_record");
}

int32_t zc_end_record(zc_ctx* ctx, void** out_recording) {
    ZC_ENTER(ctx);
    if (!out_recording) return fail(ctx, ZC_ERR_INVALID_ARG, "zc_end_record: null output");
    *out_recording = nullptr;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "zc_end_record");
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "zc_end_record (instantiate)");
    *out_recording = exec;
    return ZC_OK;
}

int32_t zc_replay(zc_ctx* ctx, void* recording) {
    ZC_ENTER(ctx);
    if (!recording) return fail(ctx, ZC_ERR_INVALID_ARG, "zc_replay: null recording");
    cudaError_t e = cudaGraphLaunch(static_cast<cudaGraphExec_t>(recording), ctx->stream);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, "zc_replay");
}

int32_t zc_free_recording(zc_ctx* ctx, void* recording) {
    ZC_ENTER(ctx);
    if (!recording) return ZC_OK;
    cudaError_t e = cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(recording));
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, "zc_free_recording");
}

uint32_t zc_block_size(uint32_t type) { return block_size(type); }
uint32_t zc_bytes_per_block(uint32_t type) { return bytes_per_block(type); }
uint64_t zc_tensor_size_bytes(uint32_t type, uint64_t n) {
    const uint64_t bs = block_size(type), bpb = bytes_per_block(type);
    return ((n + bs - 1) / bs) * bpb;
}
uint64_t zc_expert_slice_bytes(uint32_t type, uint32_t rows, uint32_t cols) {
    const uint64_t bs = block_size(type), bpb = bytes_per_block(type);
    if (bpb == 0) return (uint64_t)rows * cols * 4;
    return (uint64_t)rows * (cols / bs) * bpb;
}
int32_t zc_dmmv_supported(uint32_t type) { return dmmv_type_ok(type) ? 1 : 0; }
int32_t zc_moe_dmmv_supported(uint32_t type) { return dmmv_type_ok(type) ? 1 : 0; }

int32_t zc_dmmv(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* x, uint64_t x_size, void* y,
                uint64_t y_size, uint32_t M, uint32_t K, uint64_t a_offset, uint64_t x_offset, uint64_t y_offset,
                uint32_t acc_mode) {
    ZC_ENTER_CARRY(ctx);
    ZC_TRY(check_mat(ctx, "zc_dmmv", type, A, a_size, a_offset, (uint64_t)M * row_bytes_of(type, K), M, K));
    ZC_TRY(check_vec(ctx, "zc_dmmv", "x", x, x_size, x_offset, (uint64_t)K * 4, 16));
    ZC_TRY(check_vec(ctx, "zc_dmmv", "y", y, y_size, y_offset, (uint64_t)M * 4, 4));
    DmmvArgs a;
    a.A = u8(A, a_offset);
    a.x = f32p(x, x_offset);
    a.y = f32m(y, y_offset);
    a.M = M;
    a.K = K;
    a.acc_mode = acc_mode;
    a.a_end = u8(A, a_size);
    attach_scratch(ctx, a);
    cudaError_t e;
    const bool router = type == T_F32 && M <= 2048 && (K & 3u) == 0 && acc_mode == 0 && aligned(A, a_offset, 16);
    if (router) ZC_TRY(flush_pending(ctx));
    else ZC_TRY(take_pending(ctx, a));
    if (router)
        // few f32 rows (a router): one CTA per row instead of one warp per row
        e = launch_rms_norm_dmmv_f32(a.x, nullptr, reinterpret_cast<const float*>(a.A), nullptr, a.y, M, K, 0.f,
                                     ctx->stream, &ctx->launches);
    else
        e = launch_dmmv(type, MODE_PLAIN, a, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, "zc_dmmv");
}

int32_t zc_dmmv_o_proj_merge(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* partial,
                             uint64_t partial_size, void* y, uint64_t y_size, const void* sinks, uint64_t sinks_size,
                             uint32_t M, uint32_t K, uint64_t a_offset, uint64_t y_offset, uint32_t acc_mode,
                             uint32_t n_heads, uint32_t n_i_chunks, uint32_t sink_offset, uint32_t head_dim) {
    ZC_ENTER(ctx);
    const char* fn = "zc_dmmv_o_proj_merge";
    if (!dmmv_type_ok(type)) return fail(ctx, ZC_ERR_UNSUPPORTED_TYPE, "%s: unsupported quant type %u", fn, type);
    if (n_heads == 0 || head_dim == 0 || n_i_chunks == 0 || n_i_chunks > 16 || (uint64_t)n_heads * head_dim != K)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: need K = n_heads * head_dim and 1 <= n_i_chunks <= 16", fn);
    if (K > kMergeScratchFloats && !(type == T_Q4_K))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: K beyond %u", fn, kMergeScratchFloats);
    ZC_TRY(check_mat(ctx, fn, type, A, a_size, a_offset, (uint64_t)M * row_bytes_of(type, K), M, K));
    const uint64_t pfloats = (uint64_t)n_heads * n_i_chunks * head_dim + (uint64_t)n_heads * n_i_chunks * 2;
    ZC_TRY(check_vec(ctx, fn, "partial", partial, partial_size, 0, pfloats * 4, 8));
    ZC_TRY(check_vec(ctx, fn, "y", y, y_size, y_offset, (uint64_t)M * 4, 4));
    if (sinks) ZC_TRY(check_vec(ctx, fn, "sinks", sinks, sinks_size, 0, ((uint64_t)sink_offset + n_heads) * 4, 4));
    DmmvArgs a;
    a.A = u8(A, a_offset);
    a.y = f32m(y, y_offset);
    a.M = M;
    a.K = K;
    a.acc_mode = acc_mode;
    a.a_end = u8(A, a_size);
    a.merge.partial = f32p(partial, 0);
    a.merge.sinks = sinks ? f32p(sinks, 0) : nullptr;
    a.merge.n_heads = n_heads;
    a.merge.n_chunks = n_i_chunks;
    a.merge.head_dim = head_dim;
    a.merge.sink_offset = sink_offset;
    attach_scratch(ctx, a);
    const uint64_t wbytes = (uint64_t)M * row_bytes_of(type, K);
    cudaError_t e;
    if (wbytes >= kStreamMinBytes && warp_dmmv_eligible(type, MODE_PLAIN, a)) {
        // the streaming kernel merges the partials while it loads its activation
        e = launch_warp_dmmv(type, MODE_PLAIN, a, ctx->stream, &ctx->launches);
    } else {
        if (K > kMergeScratchFloats) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: K beyond %u", fn, kMergeScratchFloats);
        e = launch_attn_merge(a.merge, ctx->merge_scratch, ctx->stream, &ctx->launches);
        if (e == cudaSuccess) {
            a.merge = MergeArgs();
            a.x = ctx->merge_scratch;
            a.late = false;
            e = launch_dmmv(type, MODE_PLAIN, a, ctx->stream, &ctx->launches);
        }
    }
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_dmmv_push(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* x, uint64_t x_size,
                     void* dst, uint64_t dst_size, uint32_t M, uint32_t K, uint64_t a_offset, uint64_t x_offset,
                     uint64_t dst_offset, uint32_t acc_mode) {
    ZC_ENTER_CARRY(ctx);
    const char* fn = "zc_dmmv_push";
    ZC_TRY(comm_usable(ctx, fn));
    ZC_TRY(check_mat(ctx, fn, type, A, a_size, a_offset, (uint64_t)M * row_bytes_of(type, K), M, K));
    ZC_TRY(check_vec(ctx, fn, "x", x, x_size, x_offset, (uint64_t)K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "dst", dst, dst_size, dst_offset, (uint64_t)M * 4, 4));
    if (M > kPushMaxFloats)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: M=%u is beyond the %u rows the fused exchange carries", fn, M,
                    kPushMaxFloats);
    DmmvArgs a;
    a.A = u8(A, a_offset);
    a.x = f32p(x, x_offset);
    a.y = f32m(dst, dst_offset);
    a.M = M;
    a.K = K;
    a.a_end = u8(A, a_size);
    attach_scratch(ctx, a);
    ZC_TRY(take_pending(ctx, a));  // an earlier push into another vector rides along; into this one: completed first
    const uint32_t parity = ctx->push_parity;
    ctx->push_parity ^= 1u;
    a.push.world = ctx->comm.world;
    for (uint32_t r = 0; r < ctx->comm.world; ++r)
        a.push.peers[r] = reinterpret_cast<uint2*>(ctx->comm.peers[r] + kCommPushOffset + parity * kCommPushParityBytes) +
                          (size_t)ctx->comm.rank * kPushMaxFloats;
    const cudaError_t e = launch_dmmv(type, MODE_PLAIN, a, ctx->stream, &ctx->launches);
    if (e != cudaSuccess) return cuda_fail(ctx, e, fn);
    ctx->pending.slots = reinterpret_cast<uint2*>(ctx->comm_local + kCommPushOffset + parity * kCommPushParityBytes);
    ctx->pending.dst = f32m(dst, dst_offset);
    ctx->pending.n = M;
    ctx->pending.world = ctx->comm.world;
    ctx->pending.acc = acc_mode ? 1u : 0u;
    ctx->pending.spin_limit = ctx->wait_limit ? ctx->wait_limit : (1u << 24);
    ctx->pending.status = ctx->status_dev;
    return ZC_OK;
}

int32_t zc_rms_norm_dmmv_f32(zc_ctx* ctx, const void* hidden, uint64_t hidden_size, const void* norm_weights,
                             uint64_t norm_size, const void* router_weights, uint64_t router_size, void* norm_out,
                             uint64_t norm_out_size, void* logits, uint64_t logits_size, uint32_t M, uint32_t K,
                             float eps) {
    ZC_ENTER(ctx);
    const char* fn = "zc_rms_norm_dmmv_f32";
    if (M == 0 || K == 0 || (K & 3u))  // the reference's dispatch gate: K % 4 == 0 (vec4 reads)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: M and K must be non-zero and K a multiple of 4", fn);
    ZC_TRY(check_vec(ctx, fn, "hidden", hidden, hidden_size, 0, (uint64_t)K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "norm_weights", norm_weights, norm_size, 0, (uint64_t)K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "router_weights", router_weights, router_size, 0, (uint64_t)M * K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "logits", logits, logits_size, 0, (uint64_t)M * 4, 4));
    if (norm_out) {
        ZC_TRY(check_vec(ctx, fn, "norm_out", norm_out, norm_out_size, 0, (uint64_t)K * 4, 16));
        if (norm_out == hidden)  // other CTAs still read hidden while CTA 0 writes the normalised vector
            return fail(ctx, ZC_ERR_INVALID_ARG, "%s: norm_out must not alias hidden", fn);
    }
    const cudaError_t e = launch_rms_norm_dmmv_f32(f32p(hidden, 0), f32p(norm_weights, 0), f32p(router_weights, 0),
                                                   norm_out ? f32m(norm_out, 0) : nullptr, f32m(logits, 0), M, K, eps,
                                                   ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_rms_norm_dmmv_alpha_beta(zc_ctx* ctx, const void* hidden, uint64_t hidden_size, const void* norm_weights,
                                    uint64_t norm_size, const void* alpha_weights, uint64_t alpha_size,
                                    const void* beta_weights, uint64_t beta_size, void* norm_out,
                                    uint64_t norm_out_size, void* alpha_out, uint64_t alpha_out_size, void* beta_out,
                                    uint64_t beta_out_size, uint32_t M, uint32_t K, float eps) {
    ZC_ENTER(ctx);
    const char* fn = "zc_rms_norm_dmmv_alpha_beta";
    if (M == 0 || K == 0 || (K & 3u))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: M and K must be non-zero and K a multiple of 4", fn);
    ZC_TRY(check_vec(ctx, fn, "hidden", hidden, hidden_size, 0, (uint64_t)K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "norm_weights", norm_weights, norm_size, 0, (uint64_t)K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "alpha_weights", alpha_weights, alpha_size, 0, (uint64_t)M * K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "beta_weights", beta_weights, beta_size, 0, (uint64_t)M * K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "alpha_out", alpha_out, alpha_out_size, 0, (uint64_t)M * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "beta_out", beta_out, beta_out_size, 0, (uint64_t)M * 4, 4));
    if (norm_out) {
        ZC_TRY(check_vec(ctx, fn, "norm_out", norm_out, norm_out_size, 0, (uint64_t)K * 4, 16));
        if (norm_out == hidden) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: norm_out must not alias hidden", fn);
    }
    const cudaError_t e = launch_rms_norm_dmmv_f32(f32p(hidden, 0), f32p(norm_weights, 0), f32p(alpha_weights, 0),
                                                   norm_out ? f32m(norm_out, 0) : nullptr, f32m(alpha_out, 0), M, K, eps,
                                                   ctx->stream, &ctx->launches, f32p(beta_weights, 0), f32m(beta_out, 0));
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_dmmv_multi(zc_ctx* ctx, uint32_t type, uint32_t n, const void* const* A, const uint64_t* a_size,
                      const uint64_t* a_offset, const void* x, uint64_t x_size, uint64_t x_offset, void* const* y,
                      const uint64_t* y_size, const uint64_t* y_offset, const uint32_t* M, uint32_t K,
                      uint32_t acc_mode) {
    ZC_ENTER_CARRY(ctx);
    const char* fn = "zc_dmmv_multi";
    if (n == 0 || n > 3) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: n must be 1, 2 or 3", fn);
    if (!A || !a_size || !a_offset || !y || !y_size || !y_offset || !M)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: null argument array", fn);
    ZC_TRY(check_vec(ctx, fn, "x", x, x_size, x_offset, (uint64_t)K * 4, 16));
    const uint8_t* Ap[3];
    float* yp[3];
    for (uint32_t i = 0; i < n; ++i) {
        ZC_TRY(check_mat(ctx, fn, type, A[i], a_size[i], a_offset[i], (uint64_t)M[i] * row_bytes_of(type, K), M[i], K));
        ZC_TRY(check_vec(ctx, fn, "y", y[i], y_size[i], y_offset[i], (uint64_t)M[i] * 4, 4));
        Ap[i] = u8(A[i], a_offset[i]);
        yp[i] = f32m(y[i], y_offset[i]);
    }
    DmmvArgs a;
    a.x = f32p(x, x_offset);
    a.K = K;
    a.acc_mode = acc_mode;
    attach_scratch(ctx, a);
    a.M = 0;  // no single output vector: only x can collide with a pending reduction
    ZC_TRY(take_pending(ctx, a));
    for (uint32_t i = 0; i < n; ++i) {  // an output that is the vector being reduced: complete the reduction first
        const uintptr_t lo = reinterpret_cast<uintptr_t>(a.consume.dst), hi = lo + (uintptr_t)a.consume.n * 4;
        const uintptr_t q = reinterpret_cast<uintptr_t>(yp[i]);
        if (a.consume.n && q < hi && lo < q + (uintptr_t)M[i] * 4) {
            ctx->pending = a.consume;
            a.consume = ConsumeArgs();
            ZC_TRY(flush_pending(ctx));
        }
    }
    cudaError_t e = cudaSuccess;
    if (warp_dmmv_multi_eligible(type, n, Ap, M, K, a)) {
        e = launch_warp_dmmv_multi(n, Ap, yp, M, a, ctx->stream, &ctx->launches);
    } else {
        for (uint32_t i = 0; i < n && e == cudaSuccess; ++i) {  // any type, any shape: one launch per matrix
            DmmvArgs ai = a;
            ai.A = Ap[i];
            ai.y = yp[i];
            ai.M = M[i];
            if (i) ai.consume = ConsumeArgs();  // the first launch completes a pending reduction
            e = launch_dmmv(type, MODE_PLAIN, ai, ctx->stream, &ctx->launches);
        }
    }
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_dmmv_fused_gate_up_swiglu(zc_ctx* ctx, uint32_t type, const void* Wg, uint64_t wg_size, const void* Wu,
                                     uint64_t wu_size, const void* x, uint64_t x_size, void* out, uint64_t out_size,
                                     uint32_t M, uint32_t K, uint64_t gate_offset, uint64_t up_offset,
                                     uint64_t x_offset, uint64_t out_offset) {
    ZC_ENTER_CARRY(ctx);
    const char* fn = "zc_dmmv_fused_gate_up_swiglu";
    ZC_TRY(check_mat(ctx, fn, type, Wg, wg_size, gate_offset, (uint64_t)M * row_bytes_of(type, K), M, K));
    ZC_TRY(check_mat(ctx, fn, type, Wu, wu_size, up_offset, (uint64_t)M * row_bytes_of(type, K), M, K));
    ZC_TRY(check_vec(ctx, fn, "x", x, x_size, x_offset, (uint64_t)K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "out", out, out_size, out_offset, (uint64_t)M * 4, 4));
    DmmvArgs a;
    a.A = u8(Wg, gate_offset);
    a.A2 = u8(Wu, up_offset);
    a.x = f32p(x, x_offset);
    a.y = f32m(out, out_offset);
    a.M = M;
    a.K = K;
    attach_scratch(ctx, a);
    ZC_TRY(take_pending(ctx, a));
    cudaError_t e = launch_dmmv(type, MODE_GATE_UP_SWIGLU, a, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_dmmv_sigmoid_acc(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* x,
                            uint64_t x_size, void* y, uint64_t y_size, const void* gate, uint64_t gate_size,
                            uint32_t M, uint32_t K, uint64_t a_offset, uint64_t x_offset, uint64_t y_offset,
                            uint32_t gate_index) {
    ZC_ENTER(ctx);
    const char* fn = "zc_dmmv_sigmoid_acc";
    ZC_TRY(check_mat(ctx, fn, type, A, a_size, a_offset, (uint64_t)M * row_bytes_of(type, K), M, K));
    ZC_TRY(check_vec(ctx, fn, "x", x, x_size, x_offset, (uint64_t)K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "y", y, y_size, y_offset, (uint64_t)M * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "gate", gate, gate_size, (uint64_t)gate_index * 4, 4, 4));
    DmmvArgs a;
    a.A = u8(A, a_offset);
    a.x = f32p(x, x_offset);
    a.y = f32m(y, y_offset);
    a.gate = f32p(gate, (uint64_t)gate_index * 4);
    a.M = M;
    a.K = K;
    attach_scratch(ctx, a);
    cudaError_t e = launch_dmmv(type, MODE_SIGMOID_ACC, a, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_dmmv_batch(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* X, uint64_t x_size,
                      void* Y, uint64_t y_size, uint32_t M, uint32_t K, uint64_t a_offset, uint64_t x_offset,
                      uint64_t y_offset, uint32_t num_cols) {
    ZC_ENTER(ctx);
    const char* fn = "zc_dmmv_batch";
    ZC_TRY(check_mat(ctx, fn, type, A, a_size, a_offset, (uint64_t)M * row_bytes_of(type, K), M, K));
    if (num_cols == 0) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: num_cols must be non-zero", fn);
    ZC_TRY(check_vec(ctx, fn, "X", X, x_size, x_offset, (uint64_t)num_cols * K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "Y", Y, y_size, y_offset, (uint64_t)num_cols * M * 4, 4));
    cudaError_t e;
    // Enough columns to amortise tile dequantisation: tensor-core GEMM
    // (Y[c][M] is D column-major with stride M, X[c][K] is B with stride K).
    if (num_cols >= 16)
        e = launch_mul_mm(type, u8(A, a_offset), f32p(X, x_offset), f32m(Y, y_offset), M, num_cols, K, K, M, false,
                          ctx->status_dev, ctx->gemm_flags, kGemmTileFlags, ctx->stream, &ctx->launches);
    else
        e = cudaErrorNotSupported;
    if (e == cudaErrorNotSupported)
        e = launch_dmmv_batch(type, u8(A, a_offset), f32p(X, x_offset), f32m(Y, y_offset), M, K, num_cols,
                              ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_mul_mm(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* B, uint64_t b_size,
                  void* D, uint64_t d_size, uint32_t M, uint32_t N, uint32_t K, uint32_t stride_b, uint32_t stride_d,
                  uint64_t a_offset, uint64_t b_offset, uint64_t d_offset, uint32_t act_type) {
    ZC_ENTER(ctx);
    const char* fn = "zc_mul_mm";
    if (act_type != ZC_F32 && act_type != ZC_BF16)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: activations must be f32 or bf16", fn);
    if (N == 0) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: N must be non-zero", fn);
    ZC_TRY(check_mat(ctx, fn, type, A, a_size, a_offset, (uint64_t)M * row_bytes_of(type, K), M, K));
    if (stride_b < K || stride_d < M) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: stride smaller than extent", fn);
    const uint64_t esz = act_type == ZC_BF16 ? 2 : 4;
    ZC_TRY(check_vec(ctx, fn, "B", B, b_size, b_offset * esz, ((uint64_t)(N - 1) * stride_b + K) * esz, esz));
    ZC_TRY(check_vec(ctx, fn, "D", D, d_size, d_offset * 4, ((uint64_t)(N - 1) * stride_d + M) * 4, 4));
    const void* Bp = static_cast<const uint8_t*>(B) + b_offset * esz;
    cudaError_t e = launch_mul_mm(type, u8(A, a_offset), Bp, f32m(D, d_offset * 4), M, N, K, stride_b, stride_d,
                                  act_type == ZC_BF16, ctx->status_dev, ctx->gemm_flags, kGemmTileFlags, ctx->stream,
                                  &ctx->launches);
    // layouts a tensor map cannot describe (MXFP4; Q6_K rows without a 16-byte pitch): still tensor cores
    if (e == cudaErrorNotSupported && act_type == ZC_BF16 &&
        mul_mm_cp_async_eligible(type, u8(A, a_offset), Bp, N, K, stride_b))
        e = launch_mul_mm_cp_async(type, u8(A, a_offset), a_size - a_offset, Bp, f32m(D, d_offset * 4), M, N, K,
                                   stride_b, stride_d, ctx->status_dev, ctx->stream, &ctx->launches);
    if (e == cudaErrorNotSupported)
        e = launch_mul_mm_simple(type, u8(A, a_offset), Bp, f32m(D, d_offset * 4), M, N, K, stride_b, stride_d,
                                 act_type == ZC_BF16, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

// Shared checks of the per-slot MoE calls.
static int32_t check_moe(zc_ctx* ctx, const char* fn, uint32_t type, const void* A, uint64_t a_size,
                         const void* x, uint64_t x_size, const void* routing, uint64_t routing_size, uint32_t M,
                         uint32_t K, uint64_t expert_stride, uint32_t n_used, uint32_t x_expert_stride,
                         uint64_t x_offset, uint32_t routing_words) {
    // Expert ids live on the device, so only the first expert's extent can be
    // bounds-checked here; the stride must cover one expert.
    ZC_TRY(check_mat(ctx, fn, type, A, a_size, 0, (uint64_t)M * row_bytes_of(type, K), M, K));
    if (n_used == 0) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: n_used must be non-zero", fn);
    if (expert_stride < (uint64_t)M * row_bytes_of(type, K))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: expert_stride smaller than one expert", fn);
    if (x_expert_stride % 4 != 0)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: x_expert_stride must be a multiple of 4 elements", fn);
    ZC_TRY(check_vec(ctx, fn, "x", x, x_size, x_offset, ((uint64_t)(n_used - 1) * x_expert_stride + K) * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "routing", routing, routing_size, 0, (uint64_t)routing_words * 4, 4));
    return ZC_OK;
}

int32_t zc_moe_dmmv(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* x, uint64_t x_size,
                    void* y, uint64_t y_size, const void* routing, uint64_t routing_size, uint32_t M, uint32_t K,
                    uint64_t expert_stride, uint32_t n_used, uint32_t x_expert_stride, uint64_t x_offset,
                    uint64_t y_offset) {
    ZC_ENTER(ctx);
    const char* fn = "zc_moe_dmmv";
    ZC_TRY(check_moe(ctx, fn, type, A, a_size, x, x_size, routing, routing_size, M, K, expert_stride, n_used,
                     x_expert_stride, x_offset, n_used));
    ZC_TRY(check_vec(ctx, fn, "y", y, y_size, y_offset, (uint64_t)n_used * M * 4, 4));
    DmmvArgs a;
    a.A = u8(A, 0);
    a.x = f32p(x, x_offset);
    a.y = f32m(y, y_offset);
    a.routing = static_cast<const uint32_t*>(routing);
    a.M = M;
    a.K = K;
    a.expert_stride = expert_stride;
    a.n_used = n_used;
    a.x_expert_stride = x_expert_stride;
    a.n_experts_max = experts_in_buffer(a_size, (uint64_t)M * row_bytes_of(type, K), expert_stride);
    a.status = ctx->status_dev;
    cudaError_t e = launch_dmmv(type, MODE_MOE, a, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

// What the extended MoE calls add: the shared expert's matrices (a slot whose id is ZC_SHARED_EXPERT selects them)
// and per-expert f32 bias tables [n_experts][M]. All optional.
struct MoeExtras {
    const void* sh = nullptr;
    uint64_t sh_size = 0;
    const void* sh2 = nullptr;
    uint64_t sh2_size = 0;
    const void* bias = nullptr;
    uint64_t bias_size = 0;
    const void* bias2 = nullptr;
    uint64_t bias2_size = 0;
};

static int32_t moe_gate_up_common(zc_ctx* ctx, const char* fn, uint32_t type, const void* Wg, uint64_t wg_size,
                                  const void* Wu, uint64_t wu_size, const void* x, uint64_t x_size, void* y_gate,
                                  uint64_t yg_size, void* y_up, uint64_t yu_size, const void* routing,
                                  uint64_t routing_size, uint32_t M, uint32_t K, uint64_t expert_stride,
                                  uint32_t n_used, uint32_t x_expert_stride, uint64_t x_offset, uint64_t y_offset,
                                  uint32_t act, const MoeExtras& ex = MoeExtras()) {
    ZC_TRY(check_moe(ctx, fn, type, Wg, wg_size, x, x_size, routing, routing_size, M, K, expert_stride, n_used,
                     x_expert_stride, x_offset, n_used));
    ZC_TRY(check_mat(ctx, fn, type, Wu, wu_size, 0, (uint64_t)M * row_bytes_of(type, K), M, K));
    if ((ex.sh == nullptr) != (ex.sh2 == nullptr))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: the shared expert needs both its gate and its up matrix", fn);
    if (ex.sh) {
        ZC_TRY(check_mat(ctx, fn, type, ex.sh, ex.sh_size, 0, (uint64_t)M * row_bytes_of(type, K), M, K));
        ZC_TRY(check_mat(ctx, fn, type, ex.sh2, ex.sh2_size, 0, (uint64_t)M * row_bytes_of(type, K), M, K));
    }
    const uint32_t n_stack = experts_in_buffer(wg_size < wu_size ? wg_size : wu_size,
                                               (uint64_t)M * row_bytes_of(type, K), expert_stride);
    if ((ex.bias == nullptr) != (ex.bias2 == nullptr))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: gate and up biases come together", fn);
    if (ex.bias) {
        ZC_TRY(check_vec(ctx, fn, "gate_bias", ex.bias, ex.bias_size, 0, (uint64_t)n_stack * M * 4, 4));
        ZC_TRY(check_vec(ctx, fn, "up_bias", ex.bias2, ex.bias2_size, 0, (uint64_t)n_stack * M * 4, 4));
    }
    ZC_TRY(check_vec(ctx, fn, act ? "y" : "y_gate", y_gate, yg_size, y_offset, (uint64_t)n_used * M * 4, 4));
    if (!act) ZC_TRY(check_vec(ctx, fn, "y_up", y_up, yu_size, y_offset, (uint64_t)n_used * M * 4, 4));
    DmmvArgs a;
    a.A = u8(Wg, 0);
    a.A2 = u8(Wu, 0);
    a.x = f32p(x, x_offset);
    a.y = f32m(y_gate, y_offset);
    a.y2 = act ? nullptr : f32m(y_up, y_offset);
    a.act = act;
    a.routing = static_cast<const uint32_t*>(routing);
    a.M = M;
    a.K = K;
    a.expert_stride = expert_stride;
    a.n_used = n_used;
    a.x_expert_stride = x_expert_stride;
    a.a_end = u8(Wg, wg_size);
    a.a2_end = u8(Wu, wu_size);
    a.n_experts_max = n_stack;
    if (ex.sh) {
        a.A_sh = u8(ex.sh, 0);
        a.A2_sh = u8(ex.sh2, 0);
        a.a_sh_end = u8(ex.sh, ex.sh_size);
        a.a2_sh_end = u8(ex.sh2, ex.sh2_size);
    }
    a.bias = static_cast<const float*>(ex.bias);
    a.bias2 = static_cast<const float*>(ex.bias2);
    attach_scratch(ctx, a);
    cudaError_t e;
    if (warp_moe_gate_up_eligible(type, a))
        e = launch_warp_moe_gate_up(a, ctx->stream, &ctx->launches);
    else if (mxfp4_moe_gate_up_eligible(type, a))
        e = launch_mxfp4_moe_gate_up(a, ctx->stream, &ctx->launches);
    else
        e = launch_dmmv(type, MODE_MOE_GATE_UP, a, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_moe_fused_gate_up(zc_ctx* ctx, uint32_t type, const void* Wg, uint64_t wg_size, const void* Wu,
                             uint64_t wu_size, const void* x, uint64_t x_size, void* y_gate, uint64_t yg_size,
                             void* y_up, uint64_t yu_size, const void* routing, uint64_t routing_size, uint32_t M,
                             uint32_t K, uint64_t expert_stride, uint32_t n_used, uint32_t x_expert_stride,
                             uint64_t x_offset, uint64_t y_offset) {
    ZC_ENTER(ctx);
    return moe_gate_up_common(ctx, "zc_moe_fused_gate_up", type, Wg, wg_size, Wu, wu_size, x, x_size, y_gate, yg_size,
                              y_up, yu_size, routing, routing_size, M, K, expert_stride, n_used, x_expert_stride,
                              x_offset, y_offset, 0);
}

int32_t zc_moe_fused_gate_up_act(zc_ctx* ctx, uint32_t type, const void* Wg, uint64_t wg_size, const void* Wu,
                                 uint64_t wu_size, const void* x, uint64_t x_size, void* y, uint64_t y_size,
                                 const void* routing, uint64_t routing_size, uint32_t M, uint32_t K,
                                 uint64_t expert_stride, uint32_t n_used, uint32_t x_expert_stride, uint64_t x_offset,
                                 uint64_t y_offset, uint32_t oai) {
    ZC_ENTER(ctx);
    if (oai > 1) return fail(ctx, ZC_ERR_INVALID_ARG, "zc_moe_fused_gate_up_act: oai must be 0 or 1");
    return moe_gate_up_common(ctx, "zc_moe_fused_gate_up_act", type, Wg, wg_size, Wu, wu_size, x, x_size, y, y_size,
                              nullptr, 0, routing, routing_size, M, K, expert_stride, n_used, x_expert_stride,
                              x_offset, y_offset, 1 + oai);
}

static int32_t moe_down_acc_common(zc_ctx* ctx, const char* fn, uint32_t type, const void* A, uint64_t a_size,
                                   const void* x, uint64_t x_size, void* y, uint64_t y_size, const void* routing,
                                   uint64_t routing_size, uint32_t M, uint32_t K, uint64_t expert_stride,
                                   uint32_t n_used, uint32_t x_expert_stride, uint64_t x_offset, uint64_t y_offset,
                                   const MoeExtras& ex = MoeExtras()) {
    ZC_TRY(check_moe(ctx, fn, type, A, a_size, x, x_size, routing, routing_size, M, K, expert_stride, n_used,
                     x_expert_stride, x_offset, 2 * n_used));
    ZC_TRY(check_vec(ctx, fn, "y", y, y_size, y_offset, (uint64_t)M * 4, 4));
    if (ex.sh) ZC_TRY(check_mat(ctx, fn, type, ex.sh, ex.sh_size, 0, (uint64_t)M * row_bytes_of(type, K), M, K));
    if (ex.bias)
        ZC_TRY(check_vec(ctx, fn, "down_bias", ex.bias, ex.bias_size, 0,
                         (uint64_t)experts_in_buffer(a_size, (uint64_t)M * row_bytes_of(type, K), expert_stride) * M * 4, 4));
    DmmvArgs a;
    if (ex.sh) {
        a.A_sh = u8(ex.sh, 0);
        a.a_sh_end = u8(ex.sh, ex.sh_size);
    }
    a.bias = static_cast<const float*>(ex.bias);
    a.A = u8(A, 0);
    a.x = f32p(x, x_offset);
    a.y = f32m(y, y_offset);
    a.routing = static_cast<const uint32_t*>(routing);
    a.M = M;
    a.K = K;
    a.expert_stride = expert_stride;
    a.n_used = n_used;
    a.x_expert_stride = x_expert_stride;
    a.a_end = u8(A, a_size);
    a.n_experts_max = experts_in_buffer(a_size, (uint64_t)M * row_bytes_of(type, K), expert_stride);
    attach_scratch(ctx, a);
    cudaError_t e;
    if (mxfp4_moe_down_acc_eligible(type, a))
        e = launch_mxfp4_moe_down_acc(a, ctx->stream, &ctx->launches);
    else if (q6k_moe_down_acc_eligible(type, a))
        e = launch_q6k_moe_down_acc(a, ctx->stream, &ctx->launches);
    else
        e = launch_dmmv(type, MODE_MOE_DOWN_ACC, a, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_moe_fused_down_acc(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* x,
                              uint64_t x_size, void* y, uint64_t y_size, const void* routing, uint64_t routing_size,
                              uint32_t M, uint32_t K, uint64_t expert_stride, uint32_t n_used,
                              uint32_t x_expert_stride, uint64_t x_offset, uint64_t y_offset) {
    ZC_ENTER(ctx);
    return moe_down_acc_common(ctx, "zc_moe_fused_down_acc", type, A, a_size, x, x_size, y, y_size, routing,
                               routing_size, M, K, expert_stride, n_used, x_expert_stride, x_offset, y_offset);
}

int32_t zc_moe_gate_up_act_ex(zc_ctx* ctx, uint32_t type, const void* Wg, uint64_t wg_size, const void* Wu,
                              uint64_t wu_size, const void* shared_gate, uint64_t shared_gate_size,
                              const void* shared_up, uint64_t shared_up_size, const void* gate_bias,
                              uint64_t gate_bias_size, const void* up_bias, uint64_t up_bias_size, const void* x,
                              uint64_t x_size, void* y, uint64_t y_size, const void* routing, uint64_t routing_size,
                              uint32_t M, uint32_t K, uint64_t expert_stride, uint32_t n_used, uint64_t x_offset,
                              uint64_t y_offset, uint32_t oai) {
    ZC_ENTER(ctx);
    if (oai > 1) return fail(ctx, ZC_ERR_INVALID_ARG, "zc_moe_gate_up_act_ex: oai must be 0 or 1");
    MoeExtras ex;
    ex.sh = shared_gate;
    ex.sh_size = shared_gate_size;
    ex.sh2 = shared_up;
    ex.sh2_size = shared_up_size;
    ex.bias = gate_bias;
    ex.bias_size = gate_bias_size;
    ex.bias2 = up_bias;
    ex.bias2_size = up_bias_size;
    return moe_gate_up_common(ctx, "zc_moe_gate_up_act_ex", type, Wg, wg_size, Wu, wu_size, x, x_size, y, y_size,
                              nullptr, 0, routing, routing_size, M, K, expert_stride, n_used, 0, x_offset, y_offset,
                              1 + oai, ex);
}

int32_t zc_moe_down_acc_ex(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* shared_down,
                           uint64_t shared_down_size, const void* down_bias, uint64_t down_bias_size, const void* x,
                           uint64_t x_size, void* y, uint64_t y_size, const void* routing, uint64_t routing_size,
                           uint32_t M, uint32_t K, uint64_t expert_stride, uint32_t n_used, uint32_t x_expert_stride,
                           uint64_t x_offset, uint64_t y_offset) {
    ZC_ENTER(ctx);
    MoeExtras ex;
    ex.sh = shared_down;
    ex.sh_size = shared_down_size;
    ex.bias = down_bias;
    ex.bias_size = down_bias_size;
    return moe_down_acc_common(ctx, "zc_moe_down_acc_ex", type, A, a_size, x, x_size, y, y_size, routing,
                               routing_size, M, K, expert_stride, n_used, x_expert_stride, x_offset, y_offset, ex);
}

int32_t zc_moe_router_topk(zc_ctx* ctx, const void* hidden, uint64_t hidden_size, const void* norm_weights,
                           uint64_t norm_size, const void* router_weights, uint64_t router_size, const void* bias,
                           uint64_t bias_size, void* norm_out, uint64_t norm_out_size, void* logits,
                           uint64_t logits_size, void* routing, uint64_t routing_size, void* routing_local,
                           uint64_t routing_local_size, uint32_t n_experts, uint32_t K, uint32_t k, uint32_t rule,
                           float eps, uint32_t shared_slot, uint32_t e_lo, uint32_t e_hi, uint32_t local_shared) {
    ZC_ENTER(ctx);
    const char* fn = "zc_moe_router_topk";
    if (n_experts == 0 || k == 0 || k > n_experts || rule > 1 || shared_slot > 1 || K == 0 || (K & 3u))
        return fail(ctx, ZC_ERR_INVALID_ARG,
                    "%s: need 0 < k <= n_experts, rule in {0,1}, shared_slot in {0,1}, K a non-zero multiple of 4", fn);
    if (n_experts > 1024)
        return fail(ctx, ZC_ERR_INVALID_ARG,
                    "%s: at most 1024 experts (beyond: zc_rms_norm_dmmv_f32 / zc_dmmv, then zc_softmax_topk)", fn);
    if (routing_local && (e_lo > e_hi || e_hi > n_experts))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: need e_lo <= e_hi <= n_experts", fn);
    const uint64_t words = 2ull * (k + shared_slot);
    ZC_TRY(check_vec(ctx, fn, "hidden", hidden, hidden_size, 0, (uint64_t)K * 4, 16));
    if (norm_weights) ZC_TRY(check_vec(ctx, fn, "norm_weights", norm_weights, norm_size, 0, (uint64_t)K * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "router_weights", router_weights, router_size, 0, (uint64_t)n_experts * K * 4, 16));
    if (bias) ZC_TRY(check_vec(ctx, fn, "bias", bias, bias_size, 0, (uint64_t)n_experts * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "logits", logits, logits_size, 0, (uint64_t)n_experts * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "routing", routing, routing_size, 0, words * 4, 4));
    if (routing_local) ZC_TRY(check_vec(ctx, fn, "routing_local", routing_local, routing_local_size, 0, words * 4, 4));
    if (norm_out) {
        if (!norm_weights) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: norm_out without norm_weights", fn);
        ZC_TRY(check_vec(ctx, fn, "norm_out", norm_out, norm_out_size, 0, (uint64_t)K * 4, 16));
        if (norm_out == hidden) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: norm_out must not alias hidden", fn);
    }
    const cudaError_t e = launch_moe_router_topk(
        f32p(hidden, 0), norm_weights ? f32p(norm_weights, 0) : nullptr, f32p(router_weights, 0),
        static_cast<const float*>(bias), norm_out ? f32m(norm_out, 0) : nullptr, f32m(logits, 0),
        static_cast<uint32_t*>(routing), static_cast<uint32_t*>(routing_local), ctx->router_tagged, ctx->status_dev,
        ctx->wait_limit ? ctx->wait_limit : (1u << 26), n_experts, K, k,
        rule, shared_slot, e_lo, e_hi, local_shared, eps, ctx->stream, &ctx->launches);
    if (e != cudaSuccess) return cuda_fail(ctx, e, fn);
    ctx->router_mark = ctx->launches;
    return ZC_OK;
}

static int32_t check_moe_batched(zc_ctx* ctx, const char* fn, uint32_t type, const void* A, uint64_t a_size,
                                 const void* X, uint64_t x_size, void* Y, uint64_t y_size, const void* routing,
                                 uint64_t routing_size, uint32_t M, uint32_t K, uint64_t expert_stride,
                                 uint32_t n_experts, uint32_t n_experts_used, uint32_t n_tokens,
                                 uint32_t x_token_stride, uint32_t y_token_stride) {
    if (n_tokens == 0 || n_experts_used == 0 || n_experts == 0)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: zero token, expert or slot count", fn);
    ZC_TRY(check_mat(ctx, fn, type, A, a_size, 0, (uint64_t)n_experts * expert_stride, M, K));
    if (expert_stride < (uint64_t)M * row_bytes_of(type, K))
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: expert_stride smaller than one expert", fn);
    if (x_token_stride < K || x_token_stride % 4 != 0 || y_token_stride < (uint64_t)n_experts_used * M)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: token stride too small or x stride not a multiple of 4", fn);
    ZC_TRY(check_vec(ctx, fn, "X", X, x_size, 0, ((uint64_t)(n_tokens - 1) * x_token_stride + K) * 4, 16));
    ZC_TRY(check_vec(ctx, fn, "Y", Y, y_size, 0,
                     ((uint64_t)(n_tokens - 1) * y_token_stride + (uint64_t)n_experts_used * M) * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "routing", routing, routing_size, 0, (uint64_t)n_tokens * n_experts_used * 4, 4));
    return ZC_OK;
}

int32_t zc_moe_dmmv_batched(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* X,
                            uint64_t x_size, void* Y, uint64_t y_size, const void* routing, uint64_t routing_size,
                            uint32_t M, uint32_t K, uint64_t expert_stride, uint32_t n_experts,
                            uint32_t n_experts_used, uint32_t n_tokens, uint32_t x_token_stride,
                            uint32_t y_token_stride) {
    ZC_ENTER(ctx);
    const char* fn = "zc_moe_dmmv_batched";
    ZC_TRY(check_moe_batched(ctx, fn, type, A, a_size, X, x_size, Y, y_size, routing, routing_size, M, K, expert_stride,
                             n_experts, n_experts_used, n_tokens, x_token_stride, y_token_stride));
    // With a workspace and a prefill-sized batch: group the pairs by expert and run the tensor-core tiles.
    if (ctx->workspace && n_tokens >= 16 &&
        moe_grouped_eligible(type, u8(A, 0), K, expert_stride, n_experts, (uint64_t)n_tokens * n_experts_used,
                             f32p(X, 0), x_token_stride, ctx->workspace_size)) {
        cudaError_t eg = launch_moe_grouped(type, u8(A, 0), a_size, f32p(X, 0), f32m(Y, 0),
                                            static_cast<const uint32_t*>(routing), M, K, expert_stride, n_experts,
                                            n_experts_used, n_tokens, x_token_stride, y_token_stride, ctx->workspace,
                                            ctx->status_dev, ctx->stream, &ctx->launches);
        return eg == cudaSuccess ? ZC_OK : cuda_fail(ctx, eg, fn);
    }
    cudaError_t e = launch_moe_dmmv_batched(type, u8(A, 0), f32p(X, 0), f32m(Y, 0),
                                            static_cast<const uint32_t*>(routing), M, K, expert_stride,
                                            n_experts_used, n_tokens, x_token_stride, y_token_stride, n_experts,
                                            ctx->status_dev, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_moe_dmmv_batched_pair(zc_ctx* ctx, uint32_t type, const void* Wg, uint64_t wg_size, const void* Wu,
                                 uint64_t wu_size, const void* X, uint64_t x_size, void* Yg, uint64_t yg_size, void* Yu,
                                 uint64_t yu_size, const void* routing, uint64_t routing_size, uint32_t M, uint32_t K,
                                 uint64_t expert_stride, uint32_t n_experts, uint32_t n_experts_used,
                                 uint32_t n_tokens, uint32_t x_token_stride, uint32_t y_token_stride) {
    ZC_ENTER(ctx);
    const char* fn = "zc_moe_dmmv_batched_pair";
    ZC_TRY(check_moe_batched(ctx, fn, type, Wg, wg_size, X, x_size, Yg, yg_size, routing, routing_size, M, K,
                             expert_stride, n_experts, n_experts_used, n_tokens, x_token_stride, y_token_stride));
    ZC_TRY(check_moe_batched(ctx, fn, type, Wu, wu_size, X, x_size, Yu, yu_size, routing, routing_size, M, K,
                             expert_stride, n_experts, n_experts_used, n_tokens, x_token_stride, y_token_stride));
    const bool grouped = ctx->workspace && n_tokens >= 16 && !(reinterpret_cast<uintptr_t>(Wu) & 15u) &&
                         moe_grouped_eligible(type, u8(Wg, 0), K, expert_stride, n_experts,
                                              (uint64_t)n_tokens * n_experts_used, f32p(X, 0), x_token_stride,
                                              ctx->workspace_size);
    if (!grouped) {  // the two single calls run whichever path fits
        ZC_TRY(zc_moe_dmmv_batched(ctx, type, Wg, wg_size, X, x_size, Yg, yg_size, routing, routing_size, M, K,
                                   expert_stride, n_experts, n_experts_used, n_tokens, x_token_stride, y_token_stride));
        return zc_moe_dmmv_batched(ctx, type, Wu, wu_size, X, x_size, Yu, yu_size, routing, routing_size, M, K,
                                   expert_stride, n_experts, n_experts_used, n_tokens, x_token_stride, y_token_stride);
    }
    cudaError_t e = launch_moe_grouped(type, u8(Wg, 0), wg_size, f32p(X, 0), f32m(Yg, 0),
                                       static_cast<const uint32_t*>(routing), M, K, expert_stride, n_experts,
                                       n_experts_used, n_tokens, x_token_stride, y_token_stride, ctx->workspace,
                                       ctx->status_dev, ctx->stream, &ctx->launches, u8(Wu, 0), wu_size, f32m(Yu, 0));
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

uint64_t zc_moe_grouped_workspace_bytes(uint32_t n_tokens, uint32_t n_experts_used, uint32_t K, uint32_t n_experts) {
    return moe_grouped_workspace_bytes((uint64_t)n_tokens * n_experts_used, K, n_experts);
}

uint64_t zc_mul_mm_workspace_bytes(uint32_t type, uint32_t N, uint32_t K) {
    return type == T_MXFP4 ? mul_mm_mx_workspace_bytes(N, K) : 0;
}

int32_t zc_mul_mm_block_scaled(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, const void* B, uint64_t b_size,
                               void* D, uint64_t d_size, uint32_t M, uint32_t N, uint32_t K, uint32_t stride_b,
                               uint32_t stride_d, uint64_t a_offset, uint64_t b_offset, uint64_t d_offset,
                               void* workspace, uint64_t workspace_size) {
    ZC_ENTER(ctx);
    const char* fn = "zc_mul_mm_block_scaled";
    if (type != T_MXFP4) return fail(ctx, ZC_ERR_UNSUPPORTED_TYPE, "%s: MXFP4 weights only", fn);
    if (N < 64 || K < 128) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: needs at least 64 tokens and K >= 128", fn);
    ZC_TRY(check_mat(ctx, fn, type, A, a_size, a_offset, (uint64_t)M * row_bytes_of(type, K), M, K));
    if (stride_b < K || stride_d < M) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: stride smaller than extent", fn);
    ZC_TRY(check_vec(ctx, fn, "B", B, b_size, b_offset * 2, ((uint64_t)(N - 1) * stride_b + K) * 2, 2));
    ZC_TRY(check_vec(ctx, fn, "D", D, d_size, d_offset * 4, ((uint64_t)(N - 1) * stride_d + M) * 4, 4));
    const void* Bp = static_cast<const uint8_t*>(B) + b_offset * 2;
    if (!mul_mm_mx_eligible(type, u8(A, a_offset), Bp, N, K, stride_b, workspace, workspace_size))
        return fail(ctx, ZC_ERR_INVALID_ARG,
                    "%s: needs 16-byte aligned A and B, stride_b a multiple of 8 and a 256-byte aligned workspace of "
                    "zc_mul_mm_workspace_bytes(type, N, K) bytes", fn);
    const cudaError_t e = launch_mul_mm_mx(u8(A, a_offset), a_size - a_offset, Bp, f32m(D, d_offset * 4), M, N, K, stride_b,
                                           stride_d, workspace, ctx->status_dev, ctx->sm_count, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_set_workspace(zc_ctx* ctx, void* workspace, uint64_t size) {
    ZC_ENTER(ctx);
    if ((workspace == nullptr) != (size == 0) || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return fail(ctx, ZC_ERR_INVALID_ARG, "zc_set_workspace: need a 256-byte aligned pointer with its size, or NULL and 0");
    ctx->workspace = workspace;
    ctx->workspace_size = size;
    return ZC_OK;
}

int32_t zc_softmax_topk(zc_ctx* ctx, const void* logits, uint64_t logits_size, const void* bias, void* out,
                        uint64_t out_size, uint32_t n_experts, uint32_t k, uint32_t rule, uint32_t n_tokens,
                        uint32_t logits_stride, uint32_t out_stride) {
    ZC_ENTER(ctx);
    const char* fn = "zc_softmax_topk";
    if (n_experts == 0 || k == 0 || k > n_experts || n_tokens == 0 || rule > 1)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: need 0 < k <= n_experts, n_tokens > 0, rule in {0,1}", fn);
    if (logits_stride < n_experts || out_stride < 2 * k)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: stride smaller than row", fn);
    if ((uint64_t)n_experts * 4 > 200 * 1024) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: n_experts too large", fn);
    ZC_TRY(check_vec(ctx, fn, "logits", logits, logits_size, 0,
                     ((uint64_t)(n_tokens - 1) * logits_stride + n_experts) * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "out", out, out_size, 0, ((uint64_t)(n_tokens - 1) * out_stride + 2 * k) * 4, 4));
    cudaError_t e = launch_softmax_topk(static_cast<const float*>(logits), static_cast<const float*>(bias),
                                        static_cast<uint32_t*>(out), n_experts, k, rule, n_tokens, logits_stride,
                                        out_stride, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_moe_weighted_acc(zc_ctx* ctx, void* a, uint64_t a_size, const void* b, uint64_t b_size,
                            const void* routing, uint64_t routing_size, uint32_t n, uint32_t n_used,
                            uint32_t src_stride) {
    ZC_ENTER(ctx);
    const char* fn = "zc_moe_weighted_acc";
    if (n == 0 || n_used == 0) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: n and n_used must be non-zero", fn);
    ZC_TRY(check_vec(ctx, fn, "a", a, a_size, 0, (uint64_t)n * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "b", b, b_size, 0, ((uint64_t)(n_used - 1) * src_stride + n) * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "routing", routing, routing_size, 0, (uint64_t)2 * n_used * 4, 4));
    cudaError_t e = launch_moe_weighted_acc(static_cast<float*>(a), static_cast<const float*>(b),
                                            static_cast<const uint32_t*>(routing), n, n_used, src_stride,
                                            ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

static int32_t swiglu_common(zc_ctx* ctx, const void* gate, const void* up, void* y, uint32_t n, bool oai) {
    ZC_ENTER(ctx);
    if (!gate || !up || !y || n == 0) return fail(ctx, ZC_ERR_INVALID_ARG, "zc_swiglu: bad arguments");
    cudaError_t e = launch_swiglu(static_cast<const float*>(gate), static_cast<const float*>(up),
                                  static_cast<float*>(y), n, oai, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, "zc_swiglu");
}
int32_t zc_swiglu(zc_ctx* ctx, const void* gate, const void* up, void* y, uint32_t n) {
    return swiglu_common(ctx, gate, up, y, n, false);
}
int32_t zc_swiglu_oai(zc_ctx* ctx, const void* gate, const void* up, void* y, uint32_t n) {
    return swiglu_common(ctx, gate, up, y, n, true);
}

int32_t zc_bias_add(zc_ctx* ctx, void* out, uint64_t out_size, const void* bias, uint64_t bias_size, uint32_t n,
                    uint32_t src_offset) {
    ZC_ENTER(ctx);
    const char* fn = "zc_bias_add";
    if (n == 0) return fail(ctx, ZC_ERR_INVALID_ARG, "%s: n must be non-zero", fn);
    ZC_TRY(check_vec(ctx, fn, "out", out, out_size, 0, (uint64_t)n * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "bias", bias, bias_size, (uint64_t)src_offset * 4, (uint64_t)n * 4, 4));
    cudaError_t e = launch_bias_add(static_cast<float*>(out), static_cast<const float*>(bias), n, src_offset,
                                    ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_moe_bias_act(zc_ctx* ctx, const void* gate, uint64_t gate_size, const void* up, uint64_t up_size,
                        const void* gate_bias, uint64_t gate_bias_size, const void* up_bias, uint64_t up_bias_size,
                        const void* routing, uint64_t routing_size, void* y, uint64_t y_size, uint32_t M,
                        uint32_t n_used, uint32_t n_experts, uint32_t oai) {
    ZC_ENTER(ctx);
    const char* fn = "zc_moe_bias_act";
    if (M == 0 || n_used == 0 || n_experts == 0 || oai > 1)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: M, n_used and n_experts must be non-zero, oai 0 or 1", fn);
    const uint64_t act_bytes = (uint64_t)n_used * M * 4, bias_bytes = (uint64_t)n_experts * M * 4;
    ZC_TRY(check_vec(ctx, fn, "gate", gate, gate_size, 0, act_bytes, 4));
    ZC_TRY(check_vec(ctx, fn, "up", up, up_size, 0, act_bytes, 4));
    ZC_TRY(check_vec(ctx, fn, "y", y, y_size, 0, act_bytes, 4));
    if (gate_bias) ZC_TRY(check_vec(ctx, fn, "gate_bias", gate_bias, gate_bias_size, 0, bias_bytes, 4));
    if (up_bias) ZC_TRY(check_vec(ctx, fn, "up_bias", up_bias, up_bias_size, 0, bias_bytes, 4));
    ZC_TRY(check_vec(ctx, fn, "routing", routing, routing_size, 0, (uint64_t)n_used * 4, 4));
    cudaError_t e = launch_moe_bias_act(static_cast<const float*>(gate), static_cast<const float*>(up),
                                        static_cast<const float*>(gate_bias), static_cast<const float*>(up_bias),
                                        static_cast<const uint32_t*>(routing), static_cast<float*>(y), M, n_used,
                                        n_experts, oai != 0, ctx->status_dev, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_moe_weighted_bias_acc(zc_ctx* ctx, void* a, uint64_t a_size, const void* bias, uint64_t bias_size,
                                 const void* routing, uint64_t routing_size, uint32_t n, uint32_t n_used,
                                 uint32_t n_experts) {
    ZC_ENTER(ctx);
    const char* fn = "zc_moe_weighted_bias_acc";
    if (n == 0 || n_used == 0 || n_experts == 0)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: n, n_used and n_experts must be non-zero", fn);
    ZC_TRY(check_vec(ctx, fn, "a", a, a_size, 0, (uint64_t)n * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "bias", bias, bias_size, 0, (uint64_t)n_experts * n * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "routing", routing, routing_size, 0, (uint64_t)2 * n_used * 4, 4));
    cudaError_t e = launch_moe_weighted_bias_acc(static_cast<float*>(a), static_cast<const float*>(bias),
                                                 static_cast<const uint32_t*>(routing), n, n_used, n_experts,
                                                 ctx->status_dev, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_moe_ep_filter(zc_ctx* ctx, const void* routing, uint64_t routing_size, void* out, uint64_t out_size,
                         uint32_t k, uint32_t n_tokens, uint32_t routing_stride, uint32_t out_stride,
                         uint32_t expert_lo, uint32_t expert_hi) {
    ZC_ENTER(ctx);
    const char* fn = "zc_moe_ep_filter";
    if (k == 0 || n_tokens == 0 || routing_stride < k || out_stride < k || expert_lo >= expert_hi)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: zero count, stride < k or empty expert range", fn);
    const uint32_t per = out_stride < 2 * k ? k : 2 * k;  // ids alone, or ids and weights
    if (routing_stride < per)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: routing rows hold no weights to copy", fn);
    ZC_TRY(check_vec(ctx, fn, "routing", routing, routing_size, 0, ((uint64_t)(n_tokens - 1) * routing_stride + per) * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "out", out, out_size, 0, ((uint64_t)(n_tokens - 1) * out_stride + per) * 4, 4));
    const cudaError_t e = launch_moe_ep_filter(static_cast<const uint32_t*>(routing), static_cast<uint32_t*>(out), k,
                                               n_tokens, routing_stride, out_stride, expert_lo, expert_hi, ctx->stream,
                                               &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_count_experts(zc_ctx* ctx, const void* routing, uint64_t routing_size, void* counts,
                         uint64_t counts_size, uint32_t n_tokens, uint32_t n_layers, uint32_t layer,
                         uint32_t n_experts_used, uint32_t n_experts, uint64_t d_offset_bytes) {
    ZC_ENTER(ctx);
    const char* fn = "zc_count_experts";
    if (n_tokens == 0 || n_experts == 0 || n_experts_used == 0 || n_layers == 0 || layer >= n_layers)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: zero count or layer out of range", fn);
    const uint32_t slot = 2 * n_experts_used;
    ZC_TRY(check_vec(ctx, fn, "counts", counts, counts_size, d_offset_bytes, (uint64_t)n_experts * 4, 4));
    const uint64_t need = ((uint64_t)(n_tokens - 1) * slot * n_layers + (uint64_t)layer * slot + n_experts_used) * 4;
    ZC_TRY(check_vec(ctx, fn, "routing", routing, routing_size, 0, need, 4));
    cudaError_t e = launch_count_experts(
        static_cast<const uint32_t*>(routing),
        reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(counts) + d_offset_bytes), n_experts, n_experts_used,
        n_tokens, 1, slot * n_layers, layer * slot, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_moe_route_pack(zc_ctx* ctx, const void* routing, uint64_t routing_size, void* counts,
                          uint64_t counts_size, void* ids, uint64_t ids_size, uint32_t n_tokens, uint32_t n_experts,
                          uint32_t k, uint32_t routing_stride, uint32_t ids_stride) {
    ZC_ENTER(ctx);
    const char* fn = "zc_moe_route_pack";
    if (n_tokens == 0 || n_experts == 0 || k == 0 || routing_stride < k)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: zero count or routing_stride < k", fn);
    if ((uint64_t)ids_stride < (uint64_t)n_tokens)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: ids_stride must hold one route per token", fn);
    ZC_TRY(check_vec(ctx, fn, "routing", routing, routing_size, 0,
                     ((uint64_t)(n_tokens - 1) * routing_stride + k) * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "counts", counts, counts_size, 0, (uint64_t)n_experts * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "ids", ids, ids_size, 0, (uint64_t)n_experts * ids_stride * 4, 4));
    cudaError_t e = launch_moe_route_pack(static_cast<const uint32_t*>(routing), static_cast<uint32_t*>(counts),
                                          static_cast<uint32_t*>(ids), n_tokens, n_experts, k, routing_stride,
                                          ids_stride, ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_moe_route_scatter(zc_ctx* ctx, const void* routing, uint64_t routing_size, const void* src,
                             uint64_t src_size, void* dst, uint64_t dst_size, uint32_t n_tokens,
                             uint32_t hidden_dim, uint32_t k, uint32_t routing_stride) {
    ZC_ENTER(ctx);
    const char* fn = "zc_moe_route_scatter";
    if (n_tokens == 0 || hidden_dim == 0 || k == 0 || routing_stride < 2 * k)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: zero count or routing_stride < 2k", fn);
    ZC_TRY(check_vec(ctx, fn, "routing", routing, routing_size, 0,
                     ((uint64_t)(n_tokens - 1) * routing_stride + 2 * k) * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "src", src, src_size, 0, (uint64_t)n_tokens * k * hidden_dim * 4, 4));
    ZC_TRY(check_vec(ctx, fn, "dst", dst, dst_size, 0, (uint64_t)n_tokens * hidden_dim * 4, 4));
    cudaError_t e = launch_moe_route_scatter(static_cast<const uint32_t*>(routing), static_cast<const float*>(src),
                                             static_cast<float*>(dst), n_tokens, hidden_dim, k, routing_stride,
                                             ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

int32_t zc_dequant_rows(zc_ctx* ctx, uint32_t type, const void* A, uint64_t a_size, void* out, uint64_t out_size,
                        uint64_t first_row, uint32_t n_rows, uint32_t K, uint64_t a_offset) {
    ZC_ENTER(ctx);
    const char* fn = "zc_dequant_rows";
    if (!dmmv_type_ok(type)) return fail(ctx, ZC_ERR_UNSUPPORTED_TYPE, "%s: unsupported quant type %u", fn, type);
    if (n_rows == 0 || K == 0 || K % block_size(type) != 0)
        return fail(ctx, ZC_ERR_INVALID_ARG, "%s: n_rows and K must be non-zero, K a multiple of the block size", fn);
    ZC_TRY(check_vec(ctx, fn, "A", A, a_size, a_offset, (first_row + n_rows) * row_bytes_of(type, K), 1));
    ZC_TRY(check_vec(ctx, fn, "out", out, out_size, 0, (uint64_t)n_rows * K * 4, 4));
    cudaError_t e = launch_dequant_rows(type, u8(A, a_offset), static_cast<float*>(out), first_row, n_rows, K,
                                        ctx->stream, &ctx->launches);
    return e == cudaSuccess ? ZC_OK : cuda_fail(ctx, e, fn);
}

}  // extern "C"
