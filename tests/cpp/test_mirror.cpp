// Exercises the C++ host mirror (include/zinc_dmmv.hpp). Without a CUDA device it checks the layout
// helpers and that init reports the failure; with a device it also checks the error cases the
// reference's dispatch layer returns (src/compute/dmmv.zig:722, 767, 822) and one tiny matvec on
// zero weights. Prints "ok <mode>" and exits 0 on success.
#include <cstdio>
#include <cstring>
#include <vector>

#include "zinc_dmmv.hpp"

#define EXPECT(cond)                                                          \
    do {                                                                      \
        if (!(cond)) {                                                        \
            std::fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                         \
        }                                                                     \
    } while (0)

int main() {
    using namespace zinc;
    // block geometry (src/model/gguf.zig:71-123) and expertSliceBytes (src/compute/forward.zig:650-656)
    EXPECT(zc_block_size(ZC_Q4_K) == 256 && zc_bytes_per_block(ZC_Q4_K) == 144);
    EXPECT(zc_block_size(ZC_Q6_K) == 256 && zc_bytes_per_block(ZC_Q6_K) == 210);
    EXPECT(zc_block_size(ZC_MXFP4) == 32 && zc_bytes_per_block(ZC_MXFP4) == 17);
    EXPECT(zc_tensor_size_bytes(ZC_Q4_K, 4096ull * 4096ull) == 9437184ull);
    EXPECT(zc_expert_slice_bytes(ZC_MXFP4, 2880, 2880) == 4406400ull);
    EXPECT(DmmvDispatch::pipelineForType(GGMLType::q5_k));
    EXPECT(!DmmvDispatch::pipelineForType(GGMLType::bf16));
    // workspace of the grouped MoE prefill path: tile table + pair list + packed bf16 activations
    EXPECT(DmmvDispatch::moeGroupedWorkspaceBytes(512, 8, 2048, 256) >= 4096ull * 2048ull * 2ull);

    DmmvDispatch dd;
    const Error e = DmmvDispatch::init(0, dd);
    if (e != Error::None) {  // no usable device: the mirror must report it, not fall back
        EXPECT(e == Error::CudaFailure || e == Error::PipelineNotLoaded);
        std::puts("ok no-device");
        return 0;
    }
    const uint32_t M = 32, K = 512;
    const uint64_t wbytes = (uint64_t)M * (K / 256) * 144;
    Buffer A{nullptr, wbytes}, x{nullptr, K * 4}, y{nullptr, M * 4};
    EXPECT(zc_alloc(dd.context(), A.size, &A.ptr) == ZC_OK);
    EXPECT(zc_alloc(dd.context(), x.size, &x.ptr) == ZC_OK);
    EXPECT(zc_alloc(dd.context(), y.size, &y.ptr) == ZC_OK);
    EXPECT(zc_memset(dd.context(), A.ptr, 0, 0, A.size) == ZC_OK);
    EXPECT(zc_memset(dd.context(), x.ptr, 0, 0, x.size) == ZC_OK);
    EXPECT(zc_memset(dd.context(), y.ptr, 0, 0xFF, y.size) == ZC_OK);
    EXPECT(dd.setWorkspace(Buffer{A.ptr, 0}) == Error::InvalidArgument);  // pointer without a size
    EXPECT(dd.setWorkspace(Buffer{}) == Error::None);
    EXPECT(dd.recordDispatch(GGMLType::bf16, A, x, y, M, K, 0, 0, 0) == Error::UnsupportedQuantType);
    EXPECT(dd.recordDispatch(GGMLType::q4_k, A, x, y, M, 300, 0, 0, 0) == Error::InvalidArgument);
    EXPECT(dd.recordDispatch(GGMLType::q4_k, A, x, y, M, K, 16, 0, 0) == Error::InvalidArgument);  // runs past A
    EXPECT(dd.recordDispatch(GGMLType::q4_k, A, x, y, DmmvPushConstants{M, K, 0, 0, 0, 0}) == Error::None);
    EXPECT(dd.submitAndWait() == Error::None);
    std::vector<float> host(M, 1.0f);
    EXPECT(zc_download(dd.context(), host.data(), y.ptr, 0, y.size) == ZC_OK);
    for (float v : host) EXPECT(v == 0.0f);  // zero weights: d = dmin = 0
    zc_free(dd.context(), A.ptr);
    zc_free(dd.context(), x.ptr);
    zc_free(dd.context(), y.ptr);
    std::puts("ok device");
    return 0;
}
