// Parses the GGUF file given as argv[1] with include/zinc_gguf.hpp and prints what it found, one item
// per line, for the Python test to compare with what it wrote. With "--device" it also uploads every
// tensor (row shard 1 of 2 for 2-D tensors with an even row count) and checks the bytes read back.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iterator>
#include <vector>

#include "zinc_gguf.hpp"

int main(int argc, char** argv) {
    using namespace zinc;
    if (argc < 2) return 2;
    std::ifstream in(argv[1], std::ios::binary);
    std::vector<uint8_t> buf((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
    GGUFFile f;
    try {
        f = parse(buf.data(), buf.size());
    } catch (const GGUFError& e) {
        std::printf("error %s\n", e.what());
        return 0;
    }
    std::printf("version %u tensors %llu data_offset %llu\n", f.version, (unsigned long long)f.tensor_count,
                (unsigned long long)f.tensor_data_offset);
    std::string s;
    uint32_t u;
    float fl;
    bool b;
    if (f.getString("general.architecture", s)) std::printf("arch %s\n", s.c_str());
    if (f.getU32("test.block_count", u)) std::printf("block_count %u\n", u);
    if (f.getF32("test.rope_base", fl)) std::printf("rope_base %.1f\n", fl);
    if (f.getBool("test.flag", b)) std::printf("flag %d\n", (int)b);
    if (auto p = f.get("test.list"))
        if (auto arr = std::get_if<MetadataArray>(&p->v)) std::printf("list %zu\n", arr->size());
    const bool device = argc > 2 && std::strcmp(argv[2], "--device") == 0;
    zc_ctx* ctx = nullptr;
    if (device && zc_init(0, &ctx) != ZC_OK) {
        std::printf("error no device\n");
        return 1;
    }
    for (const auto& t : f.tensors) {
        unsigned long long sum = 0;
        try {
            const uint8_t* p = tensorBytes(f, t, buf.data(), buf.size());
            for (uint64_t i = 0; i < t.sizeBytes(); ++i) sum += p[i];
        } catch (const GGUFError& e) {
            std::printf("tensor %s error %s\n", t.name.c_str(), e.what());
            continue;
        }
        std::printf("tensor %s n_dims %u dims %llu %llu %llu type %u offset %llu bytes %llu sum %llu\n", t.name.c_str(),
                    t.n_dims, (unsigned long long)t.dims[0], (unsigned long long)t.dims[1],
                    (unsigned long long)t.dims[2], t.type_, (unsigned long long)t.offset,
                    (unsigned long long)t.sizeBytes(), sum);
        if (device) {
            const bool shard = t.n_dims == 2 && t.dims[1] % 2 == 0;
            LoadedTensor lt = loadTensor(ctx, f, t, buf.data(), buf.size(), shard ? 1 : 0, shard ? 2 : 1);
            std::vector<uint8_t> back(lt.size);
            if (zc_download(ctx, back.data(), lt.gpu_buffer, 0, lt.size) != ZC_OK) return 1;
            const uint8_t* p = tensorBytes(f, t, buf.data(), buf.size()) + (shard ? t.sizeBytes() / 2 : 0);
            std::printf("upload %s bytes %llu %s\n", t.name.c_str(), (unsigned long long)lt.size,
                        std::memcmp(back.data(), p, lt.size) == 0 ? "same" : "DIFFERENT");
            zc_free(ctx, lt.gpu_buffer);
        }
    }
    if (ctx) zc_destroy(ctx);
    return 0;
}
