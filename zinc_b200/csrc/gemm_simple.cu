// CUDA-core dequant-GEMM for shapes and types the tensor-core kernel does not
// take (small or ragged problems, 32-element block types, unaligned operands).
// D[col][row] = sum_k A[row][k] * B[col][k], A quantized row-major, B and D
// column-major with element strides (src/compute/dmmv.zig:139-155 in the
// reference project). Weights are dequantised exactly; accumulation is f32.
#include "dequant.cuh"
#include "kernels.h"

namespace zc {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <uint32_t TYPE, bool BF16>
__global__ void __launch_bounds__(256) gemm_simple_kernel(const uint8_t* __restrict__ A, const void* __restrict__ B,
                                                          float* __restrict__ D, uint32_t M, uint32_t N, uint32_t K,
                                                          uint32_t stride_b, uint32_t stride_d) {
    __shared__ float sA[TK][TM + 1];
    __shared__ float sB[TK][TN + 1];
    const uint64_t row_bytes = (uint64_t)(K / block_size(TYPE)) * bytes_per_block(TYPE);
    const uint32_t m0 = blockIdx.x * TM, n0 = blockIdx.y * TN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4] = {};
    for (uint32_t k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + 256 * i;  // 0..1023
            const int kk = e & 15, rr = e >> 4;
            const uint32_t row = m0 + rr, col = n0 + rr, k = k0 + kk;
            float av = 0.f, bv = 0.f;
            if (k < K) {
                if (row < M) av = dequant_elem<TYPE>(A + (uint64_t)row * row_bytes, k);
                if (col < N) {
                    if (BF16)
                        bv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(B)[(size_t)col * stride_b + k]);
                    else
                        bv = reinterpret_cast<const float*>(B)[(size_t)col * stride_b + k];
                }
            }
            sA[kk][rr] = av;
            sB[kk][rr] = bv;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = sA[kk][tx + 16 * i];
                b[i] = sB[kk][ty + 16 * i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t col = n0 + ty + 16 * j;
        if (col >= N) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t row = m0 + tx + 16 * i;
            if (row < M) D[(size_t)col * stride_d + row] = acc[i][j];
        }
    }
}

template <uint32_t TYPE>
cudaError_t launch_t(const uint8_t* A, const void* B, float* D, uint32_t M, uint32_t N, uint32_t K,
                     uint32_t stride_b, uint32_t stride_d, bool bf16, cudaStream_t s) {
    dim3 grid((M + TM - 1) / TM, (N + TN - 1) / TN);
    if (bf16) gemm_simple_kernel<TYPE, true><<<grid, 256, 0, s>>>(A, B, D, M, N, K, stride_b, stride_d);
    else gemm_simple_kernel<TYPE, false><<<grid, 256, 0, s>>>(A, B, D, M, N, K, stride_b, stride_d);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_mul_mm_simple(uint32_t type, const uint8_t* A, const void* B, float* D, uint32_t M, uint32_t N,
                                 uint32_t K, uint32_t stride_b, uint32_t stride_d, bool act_bf16, cudaStream_t s,
                                 uint64_t* launches) {
    cudaError_t e;
    switch (type) {
        case T_Q4_K: e = launch_t<T_Q4_K>(A, B, D, M, N, K, stride_b, stride_d, act_bf16, s); break;
        case T_Q5_K: e = launch_t<T_Q5_K>(A, B, D, M, N, K, stride_b, stride_d, act_bf16, s); break;
        case T_Q6_K: e = launch_t<T_Q6_K>(A, B, D, M, N, K, stride_b, stride_d, act_bf16, s); break;
        case T_Q8_0: e = launch_t<T_Q8_0>(A, B, D, M, N, K, stride_b, stride_d, act_bf16, s); break;
        case T_MXFP4: e = launch_t<T_MXFP4>(A, B, D, M, N, K, stride_b, stride_d, act_bf16, s); break;
        case T_Q5_0: e = launch_t<T_Q5_0>(A, B, D, M, N, K, stride_b, stride_d, act_bf16, s); break;
        case T_Q5_1: e = launch_t<T_Q5_1>(A, B, D, M, N, K, stride_b, stride_d, act_bf16, s); break;
        case T_F16: e = launch_t<T_F16>(A, B, D, M, N, K, stride_b, stride_d, act_bf16, s); break;
        case T_F32: e = launch_t<T_F32>(A, B, D, M, N, K, stride_b, stride_d, act_bf16, s); break;
        default: return cudaErrorNotSupported;
    }
    if (e == cudaSuccess && launches) ++*launches;
    return e;
}

}  // namespace zc
