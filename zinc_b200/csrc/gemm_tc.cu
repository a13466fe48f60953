// Tensor-core dequant-GEMM entry (tcgen05 path). Placeholder body: reports
// "not supported" so callers take the CUDA-core GEMM.
#include "kernels.h"

namespace zc {

cudaError_t launch_mul_mm(uint32_t, const uint8_t*, const void*, float*, uint32_t, uint32_t, uint32_t, uint32_t,
                          uint32_t, bool, cudaStream_t, uint64_t*) {
    return cudaErrorNotSupported;
}

}  // namespace zc
