// GGUF container reader and tensor upload for the quantized-matmul library: parses the header the way
// the reference does (src/model/gguf.zig:335-414: magic, version, metadata key/values, tensor table,
// data section aligned to general.alignment or 32) and hands a tensor's raw block bytes to the device
// unchanged (src/model/loader.zig:32-37 LoadedTensor). Header-only; needs zinc_cuda.h for the upload.
//
// Names follow the reference: GGUFFile, TensorInfo{name, n_dims, dims, type_, offset}, numElements,
// sizeBytes, findTensor, getString / getU32 / getF32 / getBool; errors InvalidMagic and
// UnexpectedEof are exceptions of type zinc::GGUFError.
#pragma once

#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <variant>
#include <vector>

#include "zinc_cuda.h"

namespace zinc {

struct GGUFError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

constexpr uint32_t GGUF_MAGIC = 0x46554747u;  // "GGUF" little-endian (src/model/gguf.zig)

struct MetadataValue;
using MetadataArray = std::vector<MetadataValue>;
// GGUF value types 0..12: u8 i8 u16 i16 u32 i32 f32 bool string array u64 i64 f64
struct MetadataValue {
    std::variant<uint8_t, int8_t, uint16_t, int16_t, uint32_t, int32_t, float, bool, std::string, MetadataArray,
                 uint64_t, int64_t, double>
        v;

    // Conversions with the reference's widening rules (src/model/gguf.zig:141-193); false when not representable.
    bool asString(std::string& out) const {
        if (auto p = std::get_if<std::string>(&v)) return out = *p, true;
        return false;
    }
    bool asU64(uint64_t& out) const {
        if (auto p = std::get_if<uint64_t>(&v)) return out = *p, true;
        if (auto p = std::get_if<uint32_t>(&v)) return out = *p, true;
        if (auto p = std::get_if<int64_t>(&v)) return *p >= 0 ? (out = (uint64_t)*p, true) : false;
        return false;
    }
    bool asU32(uint32_t& out) const {
        if (auto p = std::get_if<uint32_t>(&v)) return out = *p, true;
        if (auto p = std::get_if<int32_t>(&v)) return *p >= 0 ? (out = (uint32_t)*p, true) : false;
        if (auto p = std::get_if<uint64_t>(&v)) return *p <= 0xFFFFFFFFull ? (out = (uint32_t)*p, true) : false;
        return false;
    }
    bool asF32(float& out) const {
        if (auto p = std::get_if<float>(&v)) return out = *p, true;
        if (auto p = std::get_if<double>(&v)) return out = (float)*p, true;
        return false;
    }
    bool asBool(bool& out) const {
        if (auto p = std::get_if<bool>(&v)) return out = *p, true;
        if (auto p = std::get_if<uint8_t>(&v)) return out = *p != 0, true;
        if (auto p = std::get_if<uint32_t>(&v)) return out = *p != 0, true;
        if (auto p = std::get_if<int32_t>(&v)) return out = *p != 0, true;
        return false;
    }
};

struct TensorInfo {  // src/model/gguf.zig:196-229
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint32_t type_ = 0;   // GGML type id
    uint64_t offset = 0;  // from the start of the tensor data section

    uint64_t numElements() const {
        uint64_t n = 1;
        for (uint32_t d = 0; d < n_dims; ++d) n *= dims[d];
        return n;
    }
    // whole blocks, rounded up; 0 for a type the library does not know
    uint64_t sizeBytes() const { return zc_tensor_size_bytes(type_, numElements()); }
    // matrix view used by the matmul path: dims[0] = K (contiguous), dims[1] = M rows, dims[2] = experts
    uint64_t cols() const { return dims[0]; }
    uint64_t rows() const { return n_dims >= 2 ? dims[1] : 1; }
    uint64_t experts() const { return n_dims >= 3 ? dims[2] : 1; }
};

struct GGUFFile {  // src/model/gguf.zig:232-240
    uint32_t version = 0;
    uint64_t tensor_count = 0;
    std::map<std::string, MetadataValue> metadata;
    std::vector<TensorInfo> tensors;
    uint64_t tensor_data_offset = 0;  // file offset where tensor data begins

    const TensorInfo* findTensor(const std::string& name) const {
        for (const auto& t : tensors)
            if (t.name == name) return &t;
        return nullptr;
    }
    const MetadataValue* get(const std::string& key) const {
        auto it = metadata.find(key);
        return it == metadata.end() ? nullptr : &it->second;
    }
    bool getString(const std::string& key, std::string& out) const { auto p = get(key); return p && p->asString(out); }
    bool getU32(const std::string& key, uint32_t& out) const { auto p = get(key); return p && p->asU32(out); }
    bool getF32(const std::string& key, float& out) const { auto p = get(key); return p && p->asF32(out); }
    bool getBool(const std::string& key, bool& out) const { auto p = get(key); return p && p->asBool(out); }
};

namespace detail {
struct Reader {
    const uint8_t* data;
    uint64_t size, pos = 0;
    template <typename T>
    T read() {
        if (pos + sizeof(T) > size) throw GGUFError("UnexpectedEof");
        T v;
        std::memcpy(&v, data + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string readString() {
        const uint64_t n = read<uint64_t>();
        if (n > size - pos) throw GGUFError("UnexpectedEof");
        std::string s(reinterpret_cast<const char*>(data + pos), (size_t)n);
        pos += n;
        return s;
    }
    MetadataValue readValue(uint32_t type, int depth = 0) {
        MetadataValue m;
        switch (type) {
            case 0: m.v = read<uint8_t>(); break;
            case 1: m.v = read<int8_t>(); break;
            case 2: m.v = read<uint16_t>(); break;
            case 3: m.v = read<int16_t>(); break;
            case 4: m.v = read<uint32_t>(); break;
            case 5: m.v = read<int32_t>(); break;
            case 6: m.v = read<float>(); break;
            case 7: m.v = (bool)(read<uint8_t>() != 0); break;
            case 8: m.v = readString(); break;
            case 9: {
                if (depth > 4) throw GGUFError("InvalidMetadata: arrays nested too deeply");
                const uint32_t et = read<uint32_t>();
                const uint64_t n = read<uint64_t>();
                if (n > size - pos) throw GGUFError("UnexpectedEof");  // every element takes at least one byte
                MetadataArray arr;
                arr.reserve((size_t)(n < (1u << 20) ? n : (1u << 20)));  // a count is a claim: grow beyond this as read
                for (uint64_t i = 0; i < n; ++i) arr.push_back(readValue(et, depth + 1));
                m.v = std::move(arr);
                break;
            }
            case 10: m.v = read<uint64_t>(); break;
            case 11: m.v = read<int64_t>(); break;
            case 12: m.v = read<double>(); break;
            default: throw GGUFError("InvalidMetadata: unknown value type " + std::to_string(type));
        }
        return m;
    }
};
}  // namespace detail

// parse (src/model/gguf.zig:335-414)
inline GGUFFile parse(const void* data, uint64_t size) {
    detail::Reader r{static_cast<const uint8_t*>(data), size};
    if (r.read<uint32_t>() != GGUF_MAGIC) throw GGUFError("InvalidMagic");
    GGUFFile f;
    f.version = r.read<uint32_t>();
    f.tensor_count = r.read<uint64_t>();
    const uint64_t metadata_count = r.read<uint64_t>();
    for (uint64_t i = 0; i < metadata_count; ++i) {
        std::string key = r.readString();
        const uint32_t type = r.read<uint32_t>();
        f.metadata[std::move(key)] = r.readValue(type);
    }
    for (uint64_t i = 0; i < f.tensor_count; ++i) {
        TensorInfo t;
        t.name = r.readString();
        t.n_dims = r.read<uint32_t>();
        if (t.n_dims > 4) throw GGUFError("InvalidTensor: more than 4 dimensions");
        for (uint32_t d = 0; d < t.n_dims; ++d) t.dims[d] = r.read<uint64_t>();
        {  // the element count must fit 64 bits (a wrapped product would pass the byte-range check further down)
            uint64_t n = 1;
            for (uint32_t d = 0; d < t.n_dims; ++d)
                if (__builtin_mul_overflow(n, t.dims[d], &n)) throw GGUFError("InvalidTensor: element count overflows");
        }
        t.type_ = r.read<uint32_t>();
        t.offset = r.read<uint64_t>();
        f.tensors.push_back(std::move(t));
    }
    uint64_t alignment = 32;
    if (auto p = f.get("general.alignment")) {
        uint64_t a;
        if (p->asU64(a) && a != 0 && (a & (a - 1)) == 0) alignment = a;
    }
    f.tensor_data_offset = (r.pos + alignment - 1) & ~(alignment - 1);
    return f;
}

// A tensor's bytes inside the mapped file; throws when the table points outside it.
inline const uint8_t* tensorBytes(const GGUFFile& f, const TensorInfo& t, const void* data, uint64_t size) {
    const uint64_t begin = f.tensor_data_offset + t.offset, n = t.sizeBytes();
    if (begin > size || n > size - begin) throw GGUFError("InvalidTensor: '" + t.name + "' lies outside the file");
    return static_cast<const uint8_t*>(data) + begin;
}

struct LoadedTensor {  // src/model/loader.zig:32-37
    TensorInfo info;
    void* gpu_buffer = nullptr;  // raw GGUF block bytes, exactly as in the file
    uint64_t size = 0;
};

// Upload one tensor unchanged. rank/world select a tensor-parallel row shard (rows [rank*M/world, ...):
// a contiguous byte range of the tensor, since a row is a whole number of blocks).
inline LoadedTensor loadTensor(zc_ctx* ctx, const GGUFFile& f, const TensorInfo& t, const void* data, uint64_t size,
                               uint32_t rank = 0, uint32_t world = 1) {
    const uint8_t* src = tensorBytes(f, t, data, size);
    LoadedTensor out;
    out.info = t;
    uint64_t begin = 0, n = t.sizeBytes();
    if (world > 1) {
        const uint64_t rows = t.rows() * t.experts();
        if (t.n_dims < 2 || t.experts() != 1 || rows % world) throw GGUFError("row shard: rows do not divide over the ranks");
        const uint64_t row_bytes = zc_tensor_size_bytes(t.type_, t.cols());
        begin = (uint64_t)rank * (rows / world) * row_bytes;
        n = (rows / world) * row_bytes;
        out.info.dims[1] = rows / world;
    }
    if (zc_alloc(ctx, n, &out.gpu_buffer) != ZC_OK || zc_upload(ctx, out.gpu_buffer, 0, src + begin, n) != ZC_OK)
        throw GGUFError(std::string("upload of '") + t.name + "' failed: " + zc_last_error(ctx));
    out.size = n;
    return out;
}

}  // namespace zinc
