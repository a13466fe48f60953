// zc_dmmv_q4k_static_scratch: the streaming Q4_K matvec with its split-K scratch in a
// file-scope __device__ array instead of memory a context allocated.
//
// Why: the streaming matvec hands partial row sums between warps of different CTAs through a
// small global scratch (each sum stored together with a tag word). Every other entry point takes that
// scratch from a context, and creating a context allocates (device scratch, pinned status
// words, a stream). A host that has already given all device memory to its own arena (weights
// and KV cache sized to fill HBM), or that runs where an allocation would synchronise the
// device (inside its decode loop), cannot afford that. This entry point needs no context and
// calls no allocating routine: the scratch is part of the loaded module.
//
// The array is shared by every call on the same device. Consequences:
//  * the array must be all zero when a launch starts. A __device__ array is zero when the module
//    is loaded on a device, and each launch leaves it zero (the reader of a tagged sum clears it),
//    so the set-up writes nothing. A launch that gave up on a bounded wait (status word set) may
//    leave tagged sums behind; the next call sees the non-zero status word only if the caller
//    checks it, so a caller that finds status_words[0] != 0 must stop using this entry point on
//    that device.
//  * two calls whose kernels can overlap (different streams, or threads without ordering)
//    race on the array and give wrong results. Calls on one stream are ordered and safe.
//
// Set-up happens inside the first call on each device: cudaGetSymbolAddress and one attribute
// query (no device work). Make the first call on a device before starting any stream capture on it.
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/zinc_cuda.h"
#include "common.cuh"
#include "kernels.h"

namespace {

using namespace zc;

// Scratch capacity: kStreamMaxWorkers (4096) worker warps, each 32 partial sums as {f32 bits, tag}
// pairs: 4096 * 32 * 8 = 1048576 bytes.
constexpr size_t kStaticScratchBytes = kStreamPartialBytes;
constexpr uint32_t kStaticMaxK = 12288;  // 48 blocks of 256: what the per-warp staging holds
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct DeviceState {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
    int sm_count = 0;
};

DeviceState g_dev[kMaxDevices];
std::mutex g_dev_mutex;

int32_t sfail(char* buf, uint64_t cap, int32_t code, const char* fmt, ...) {
    if (buf && cap) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, (size_t)cap, fmt, ap);
        va_end(ap);
    }
    return code;
}

// Once per device, with that device current.
cudaError_t setup_device(int device, DeviceState** out) {
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceState& st = g_dev[device];
    if (!st.ready) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return e;
        int sms = 0;
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return e;
        st.scratch = static_cast<unsigned char*>(ptr);
        st.sm_count = sms;
        st.ready = true;
    }
    *out = &st;
    return cudaSuccess;
}

inline bool fits(uint64_t offset, uint64_t need, uint64_t size) { return offset <= size && need <= size - offset; }

}  // namespace

extern "C" int32_t zc_dmmv_q4k_static_scratch(void* cuda_stream, const void* A, uint64_t a_size, const void* x,
                                              uint64_t x_size, void* y, uint64_t y_size, uint32_t M, uint32_t K,
                                              uint64_t a_offset, uint64_t x_offset, uint64_t y_offset,
                                              uint32_t acc_mode, uint32_t* status_words, char* err_buf,
                                              uint64_t err_cap) {
    const char* fn = "zc_dmmv_q4k_static_scratch";
    if (err_buf && err_cap) err_buf[0] = 0;
    if (!A || !x || !y) return sfail(err_buf, err_cap, ZC_ERR_INVALID_ARG, "%s: null buffer pointer", fn);
    if (!status_words || (reinterpret_cast<uintptr_t>(status_words) & 3u))
        return sfail(err_buf, err_cap, ZC_ERR_INVALID_ARG,
                     "%s: status_words must point to two zeroed, device-visible u32 words", fn);
    if (M == 0 || K == 0 || (K & 255u))
        return sfail(err_buf, err_cap, ZC_ERR_INVALID_ARG, "%s: M must be non-zero and K a non-zero multiple of 256 (K=%u)",
                     fn, K);
    if (K > kStaticMaxK)
        return sfail(err_buf, err_cap, ZC_ERR_INVALID_ARG,
                     "%s: K=%u is beyond this entry point's maximum of %u; use zc_dmmv", fn, K, kStaticMaxK);
    const uint64_t row_bytes = (uint64_t)(K >> 8) * 144u;
    if (!fits(a_offset, (uint64_t)M * row_bytes, a_size) || !fits(x_offset, (uint64_t)K * 4, x_size) ||
        !fits(y_offset, (uint64_t)M * 4, y_size))
        return sfail(err_buf, err_cap, ZC_ERR_INVALID_ARG, "%s: offset + extent exceeds a buffer's size", fn);
    if ((reinterpret_cast<uintptr_t>(A) + a_offset) & 15u)
        return sfail(err_buf, err_cap, ZC_ERR_INVALID_ARG, "%s: weights must be 16-byte aligned", fn);
    if (((reinterpret_cast<uintptr_t>(x) + x_offset) & 15u) || ((reinterpret_cast<uintptr_t>(y) + y_offset) & 3u))
        return sfail(err_buf, err_cap, ZC_ERR_INVALID_ARG, "%s: x must be 16-byte and y 4-byte aligned", fn);

    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return sfail(err_buf, err_cap, ZC_ERR_CUDA, "%s: cudaGetDevice: %s", fn, cudaGetErrorString(e));
    if (device < 0 || device >= kMaxDevices)
        return sfail(err_buf, err_cap, ZC_ERR_INVALID_ARG, "%s: device index %d is beyond the %d supported", fn, device,
                     kMaxDevices);
    DeviceState* st = nullptr;
    e = setup_device(device, &st);
    if (e != cudaSuccess)
        return sfail(err_buf, err_cap, ZC_ERR_CUDA, "%s: set-up of the static scratch: %s", fn, cudaGetErrorString(e));

    DmmvArgs a;
    a.A = static_cast<const uint8_t*>(A) + a_offset;
    a.x = reinterpret_cast<const float*>(static_cast<const uint8_t*>(x) + x_offset);
    a.y = reinterpret_cast<float*>(static_cast<uint8_t*>(y) + y_offset);
    a.M = M;
    a.K = K;
    a.acc_mode = acc_mode;
    a.scratch_partial = reinterpret_cast<uint2*>(st->scratch);
    a.status = status_words;
    a.sm_count = st->sm_count;
    if (!warp_dmmv_eligible(T_Q4_K, MODE_PLAIN, a))
        return sfail(err_buf, err_cap, ZC_ERR_INVALID_ARG,
                     "%s: M=%u K=%u is too small for the streaming kernel (needs at least 16 row-tile x k-segment "
                     "units); use zc_dmmv",
                     fn, M, K);
    e = launch_warp_dmmv(T_Q4_K, MODE_PLAIN, a, static_cast<cudaStream_t>(cuda_stream), nullptr);
    if (e != cudaSuccess) return sfail(err_buf, err_cap, ZC_ERR_CUDA, "%s: launch: %s", fn, cudaGetErrorString(e));
    return ZC_OK;
}
