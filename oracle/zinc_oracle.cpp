// CPU oracle for the quantized matmul path of the ZINC inference engine.
//
// THIS FILE IS TEST INFRASTRUCTURE. It is a plain CPU restatement of the
// reference's own CPU math for the path (dequantRow, getScaleMinK4, the two
// routing rules, the activation and combine steps) and of the per-lane
// accumulation order of its decode shaders. Only the test-suite, the smoke
// check and the benchmark's cpu_baseline / reference arm may load it; the
// shipped CUDA library never links or calls it.
//
// Parity status: pinned against the known-answer tests the reference holds
// for getScaleMinK4, Q4_K, Q5_K, Q8_0, Q5_0, Q5_1, F16, F32, MXFP4 (e=127),
// topKSoftmax, topKSoftmaxWeight, expertSliceBytes, sizeBytes and SiLU.
// Unpinned by known answers (the reference has none): Q6_K values, the
// MXFP4 e=0 branch and swiglu_oai; those follow the cited lines only.
//
// Every function cites the reference lines it follows, as
// <path inside the reference project>:<lines>.
//
// Build: see oracle/Makefile (g++ -O3 -march=x86-64-v3 -ffp-contract=off -fopenmp -shared).

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

// GGML type ids: src/model/gguf.zig:38-69
enum : uint32_t {
    T_F32 = 0, T_F16 = 1, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8,
    T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_BF16 = 30, T_MXFP4 = 39,
};

inline float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            // subnormal: renormalise
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
inline uint32_t rd32(const uint8_t* p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

// src/model/gguf.zig:75-91
uint32_t block_size(uint32_t t) {
    switch (t) {
        case T_F32: case T_F16: case T_BF16: return 1;
        case T_Q5_0: case T_Q5_1: case T_Q8_0: case T_MXFP4: return 32;
        case T_Q4_K: case T_Q5_K: case T_Q6_K: return 256;
        case 2: case 3: case 9: return 32;            // q4_0 q4_1 q8_1
        case 10: case 11: case 15: return 256;        // q2_k q3_k q8_k
        default: return 1;
    }
}

// src/model/gguf.zig:97-122
uint32_t bytes_per_block(uint32_t t) {
    switch (t) {
        case T_F32: return 4;  case T_F16: return 2;  case T_BF16: return 2;
        case 28: return 8;     case 24: return 1;     case 25: return 2;
        case 26: return 4;     case 27: return 8;
        case 2: return 18;     case 3: return 20;
        case T_Q5_0: return 22; case T_Q5_1: return 24;
        case T_Q8_0: return 34; case 9: return 36;
        case 10: return 84;    case 11: return 110;
        case T_Q4_K: return 144; case T_Q5_K: return 176; case T_Q6_K: return 210;
        case 15: return 292;
        case T_MXFP4: return 17;
        default: return 0;
    }
}

// src/compute/forward.zig:229-238
inline void get_scale_min_k4(int j, const uint8_t* s, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

const float kMxfp4Lut[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                             -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

// Dequantise one row. Every product and difference below is a separately
// rounded f32 operation, as in the reference (no fused multiply-add): the
// Makefile compiles this file with -ffp-contract=off.
// src/compute/forward.zig:242-465; Q5_1 from src/compute/forward_metal.zig:6704-6729
int dequant_row(const uint8_t* raw, uint64_t row, uint32_t cols, uint32_t type, float* out) {
    switch (type) {
    case T_F32: {  // forward.zig:244-249
        std::memcpy(out, raw + row * (uint64_t)cols * 4, (size_t)cols * 4);
        return 0;
    }
    case T_F16: {  // forward.zig:250-257
        const uint8_t* p = raw + row * (uint64_t)cols * 2;
        for (uint32_t i = 0; i < cols; ++i) out[i] = half_to_float(rd16(p + 2 * i));
        return 0;
    }
    case T_Q8_0: {  // forward.zig:258-275
        const uint64_t bpr = cols / 32;
        const uint8_t* p = raw + row * bpr * 34;
        size_t o = 0;
        for (uint64_t b = 0; b < bpr; ++b, p += 34) {
            const float scale = half_to_float(rd16(p));
            for (int j = 0; j < 32; ++j) out[o++] = (float)(int8_t)p[2 + j] * scale;
        }
        return 0;
    }
    case T_Q6_K: {  // forward.zig:276-325
        const uint64_t bpr = cols / 256;
        const uint8_t* bb = raw + row * bpr * 210;
        size_t o = 0;
        for (uint64_t b = 0; b < bpr; ++b, bb += 210) {
            const float d = half_to_float(rd16(bb + 208));
            const uint8_t* ql = bb;
            const uint8_t* qh = bb + 128;
            const uint8_t* sc = bb + 192;
            for (int half = 0; half < 2; ++half) {
                for (int l = 0; l < 32; ++l) {
                    const int is = l / 16;
                    const uint8_t ql_lo = ql[l], ql_hi = ql[l + 32], qh_v = qh[l];
                    const int rq1 = (ql_lo & 0xF) | (((qh_v >> 0) & 3) << 4);
                    const int rq2 = (ql_hi & 0xF) | (((qh_v >> 2) & 3) << 4);
                    const int rq3 = (ql_lo >> 4) | (((qh_v >> 4) & 3) << 4);
                    const int rq4 = (ql_hi >> 4) | (((qh_v >> 6) & 3) << 4);
                    const float q1 = (float)(rq1 - 32), q2 = (float)(rq2 - 32);
                    const float q3 = (float)(rq3 - 32), q4 = (float)(rq4 - 32);
                    const float ds0 = d * (float)(int8_t)sc[is + 0];
                    const float ds2 = d * (float)(int8_t)sc[is + 2];
                    const float ds4 = d * (float)(int8_t)sc[is + 4];
                    const float ds6 = d * (float)(int8_t)sc[is + 6];
                    out[o + l + 0] = ds0 * q1;
                    out[o + l + 32] = ds2 * q2;
                    out[o + l + 64] = ds4 * q3;
                    out[o + l + 96] = ds6 * q4;
                }
                ql += 64; qh += 32; sc += 8; o += 128;
            }
        }
        return 0;
    }
    case T_Q5_K: {  // forward.zig:326-369
        const uint64_t bpr = cols / 256;
        const uint8_t* bb = raw + row * bpr * 176;
        size_t o = 0;
        for (uint64_t b = 0; b < bpr; ++b, bb += 176) {
            const float d = half_to_float(rd16(bb));
            const float dmin = half_to_float(rd16(bb + 2));
            const uint8_t* scales = bb + 4;
            const uint8_t* qh = bb + 16;
            const uint8_t* qs = bb + 48;
            int is = 0;
            for (int j = 0; j < 4; ++j) {
                uint8_t sc, m;
                get_scale_min_k4(is, scales, &sc, &m);
                const float d1 = d * (float)sc;
                const float m1 = dmin * (float)m;
                get_scale_min_k4(is + 1, scales, &sc, &m);
                const float d2 = d * (float)sc;
                const float m2 = dmin * (float)m;
                for (int l = 0; l < 32; ++l) {
                    const uint8_t lo = qs[j * 32 + l] & 0xF, hi = qs[j * 32 + l] >> 4;
                    const uint8_t hb_lo = (qh[l] >> (j * 2)) & 1, hb_hi = (qh[l] >> (j * 2 + 1)) & 1;
                    const float p1 = d1 * (float)(lo | (hb_lo << 4));
                    const float p2 = d2 * (float)(hi | (hb_hi << 4));
                    out[o + l] = p1 - m1;
                    out[o + 32 + l] = p2 - m2;
                }
                o += 64; is += 2;
            }
        }
        return 0;
    }
    case T_Q4_K: {  // forward.zig:370-409
        const uint64_t bpr = cols / 256;
        const uint8_t* bb = raw + row * bpr * 144;
        size_t o = 0;
        for (uint64_t b = 0; b < bpr; ++b, bb += 144) {
            const float d = half_to_float(rd16(bb));
            const float dmin = half_to_float(rd16(bb + 2));
            const uint8_t* scales = bb + 4;
            const uint8_t* qs = bb + 16;
            int is = 0;
            for (int g = 0; g < 4; ++g) {
                uint8_t sc, m;
                get_scale_min_k4(is, scales, &sc, &m);
                const float d1 = d * (float)sc;
                const float m1 = dmin * (float)m;
                get_scale_min_k4(is + 1, scales, &sc, &m);
                const float d2 = d * (float)sc;
                const float m2 = dmin * (float)m;
                for (int l = 0; l < 32; ++l) {
                    const float p = d1 * (float)(qs[l] & 0xF);
                    out[o++] = p - m1;
                }
                for (int l = 0; l < 32; ++l) {
                    const float p = d2 * (float)(qs[l] >> 4);
                    out[o++] = p - m2;
                }
                qs += 32; is += 2;
            }
        }
        return 0;
    }
    case T_Q5_0: {  // forward.zig:410-440
        const uint64_t bpr = cols / 32;
        const uint8_t* bb = raw + row * bpr * 22;
        size_t o = 0;
        for (uint64_t b = 0; b < bpr; ++b, bb += 22) {
            const float d = half_to_float(rd16(bb));
            const uint32_t qh = rd32(bb + 2);
            for (int j = 0; j < 16; ++j) {
                const uint32_t qb = bb[6 + j];
                const uint32_t q0 = (qb & 0xF) | (((qh >> j) & 1) << 4);
                const uint32_t q1 = (qb >> 4) | (((qh >> (j + 16)) & 1) << 4);
                out[o + j] = d * ((float)q0 - 16.0f);
                out[o + 16 + j] = d * ((float)q1 - 16.0f);
            }
            o += 32;
        }
        return 0;
    }
    case T_Q5_1: {  // forward_metal.zig:6704-6729
        const uint64_t bpr = cols / 32;
        const uint8_t* bb = raw + row * bpr * 24;
        size_t o = 0;
        for (uint64_t b = 0; b < bpr; ++b, bb += 24) {
            const float d = half_to_float(rd16(bb));
            const float mn = half_to_float(rd16(bb + 2));
            const uint32_t qh = rd32(bb + 4);
            for (int j = 0; j < 16; ++j) {
                const uint32_t qb = bb[8 + j];
                const uint32_t q0 = (qb & 0xF) | (((qh >> j) & 1) << 4);
                const uint32_t q1 = (qb >> 4) | (((qh >> (j + 16)) & 1) << 4);
                const float p0 = d * (float)q0;
                const float p1 = d * (float)q1;
                out[o + j] = p0 + mn;
                out[o + 16 + j] = p1 + mn;
            }
            o += 32;
        }
        return 0;
    }
    case T_MXFP4: {  // forward.zig:441-459
        const uint64_t bpr = cols / 32;
        const uint8_t* bo = raw + row * bpr * 17;
        size_t o = 0;
        for (uint64_t b = 0; b < bpr; ++b, bo += 17) {
            const uint32_t bits = bo[0] == 0 ? 0x00400000u : ((uint32_t)bo[0] << 23);
            float d;
            std::memcpy(&d, &bits, 4);
            for (int j = 0; j < 16; ++j) {
                out[o + j] = d * kMxfp4Lut[bo[1 + j] & 0xF];
                out[o + j + 16] = d * kMxfp4Lut[bo[1 + j] >> 4];
            }
            o += 32;
        }
        return 0;
    }
    default:  // forward.zig:460-463: unsupported types produce zeros
        for (uint32_t i = 0; i < cols; ++i) out[i] = 0.0f;
        return -1;
    }
}

inline uint64_t row_bytes(uint32_t type, uint32_t K) {
    return (uint64_t)(K / block_size(type)) * bytes_per_block(type);
}

}  // namespace

extern "C" {

uint32_t zo_block_size(uint32_t t) { return block_size(t); }
uint32_t zo_bytes_per_block(uint32_t t) { return bytes_per_block(t); }

// TensorInfo.sizeBytes: src/model/gguf.zig:222-229
uint64_t zo_tensor_size_bytes(uint32_t type, uint64_t n_elements) {
    const uint64_t bs = block_size(type), bpb = bytes_per_block(type);
    return ((n_elements + bs - 1) / bs) * bpb;
}

// expertSliceBytes: src/compute/forward.zig:650-656 (u32 arithmetic, as there)
uint32_t zo_expert_slice_bytes(uint32_t type, uint32_t rows, uint32_t cols) {
    const uint32_t bs = block_size(type), bpb = bytes_per_block(type);
    if (bs == 0 || bpb == 0) return rows * cols * 4;
    return rows * (cols / bs) * bpb;
}

// DMMV bytes model of the reference's micro-benchmark: weights + x + y.
// src/bench_hot_decode.zig:323-330
uint64_t zo_dmmv_bytes_model(uint32_t type, uint32_t M, uint32_t K) {
    return (uint64_t)M * row_bytes(type, K) + (uint64_t)K * 4 + (uint64_t)M * 4;
}

void zo_get_scale_min_k4(uint32_t j, const uint8_t* scales, uint8_t* sc, uint8_t* m) {
    get_scale_min_k4((int)j, scales, sc, m);
}

int32_t zo_dequant_row(const uint8_t* raw, uint64_t row, uint32_t cols, uint32_t type, float* out) {
    return dequant_row(raw, row, cols, type, out);
}

int32_t zo_dequant_rows(const uint8_t* raw, uint64_t rows, uint32_t cols, uint32_t type, float* out) {
    int rc = 0;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; ++r) {
        if (dequant_row(raw, (uint64_t)r, cols, type, out + (size_t)r * cols) != 0) rc = -1;
    }
    return rc;
}

// y (+)= W x with the expected value the reference's kernel tests use:
// dequantRow, then a sequential f32 dot in index order.
// src/compute/forward_metal.zig:11324-11327, 11487-11492
int32_t zo_dmmv_f32seq(const uint8_t* raw, uint32_t type, uint32_t M, uint32_t K,
                       const float* x, float* y, uint32_t acc_mode) {
    int rc = 0;
#pragma omp parallel
    {
        std::vector<float> rowbuf(K);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < (int64_t)M; ++r) {
            if (dequant_row(raw, (uint64_t)r, K, type, rowbuf.data()) != 0) rc = -1;
            float acc = 0.0f;
            for (uint32_t i = 0; i < K; ++i) {
                const float p = rowbuf[i] * x[i];
                acc = acc + p;
            }
            y[r] = acc_mode ? y[r] + acc : acc;
        }
    }
    return rc;
}

// Same product with an f64 accumulator, as the reference's in-engine
// validation does. src/compute/forward.zig:6772-6774
int32_t zo_dmmv_f64(const uint8_t* raw, uint32_t type, uint32_t M, uint32_t K,
                    const float* x, double* y) {
    int rc = 0;
#pragma omp parallel
    {
        std::vector<float> rowbuf(K);
#pragma omp for schedule(static)
        for (int64_t r = 0; r < (int64_t)M; ++r) {
            if (dequant_row(raw, (uint64_t)r, K, type, rowbuf.data()) != 0) rc = -1;
            double acc = 0.0;
            for (uint32_t i = 0; i < K; ++i) acc += (double)rowbuf[i] * (double)x[i];
            y[r] = acc;
        }
    }
    return rc;
}

// Batched product Y[c][M] = W X[c][K], f64 accumulate. X rows may be given
// as f32; `round_bf16` rounds both operands to bf16 first (the precision
// the tensor-core prefill path computes in), so that path can be compared
// against its own arithmetic as well as against the exact product.
// Layouts: src/compute/forward.zig:8141-8146
static inline float bf16_round(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return f;
    u += 0x7FFFu + ((u >> 16) & 1u);
    u &= 0xFFFF0000u;
    std::memcpy(&f, &u, 4);
    return f;
}

int32_t zo_gemm_f64(const uint8_t* raw, uint32_t type, uint32_t M, uint32_t K,
                    const float* X, uint32_t T, double* Y, uint32_t round_bf16) {
    int rc = 0;
    std::vector<float> Xr;
    const float* Xp = X;
    if (round_bf16) {
        Xr.resize((size_t)T * K);
        for (size_t i = 0; i < Xr.size(); ++i) Xr[i] = bf16_round(X[i]);
        Xp = Xr.data();
    }
#pragma omp parallel
    {
        std::vector<float> rowbuf(K);
#pragma omp for schedule(dynamic, 8)
        for (int64_t r = 0; r < (int64_t)M; ++r) {
            if (dequant_row(raw, (uint64_t)r, K, type, rowbuf.data()) != 0) rc = -1;
            if (round_bf16)
                for (uint32_t i = 0; i < K; ++i) rowbuf[i] = bf16_round(rowbuf[i]);
            for (uint32_t c = 0; c < T; ++c) {
                const float* xc = Xp + (size_t)c * K;
                double acc = 0.0;
                for (uint32_t i = 0; i < K; ++i) acc += (double)rowbuf[i] * (double)xc[i];
                Y[(size_t)c * M + r] = acc;
            }
        }
    }
    return rc;
}

// ---------------------------------------------------------------------------
// Shader-order DMMV: the timed CPU baseline. Restates the per-lane work split
// of the reference's decode shaders (64 lanes per workgroup, two rows per
// workgroup) and reduces the 64 lane partials at the end, as subgroupAdd does.
//   Q4_K : src/shaders/dmmv_q4k.comp:63-112  (16 lanes per super-block, 4 in flight)
//   Q5_K : src/shaders/dmmv_q5k.comp:62-182  (same mapping + 5th bit)
//   Q6_K : src/shaders/dmmv_q6k.comp:65-137  (16 lanes per super-block)
//   Q8_0 : src/shaders/dmmv_q8_0.comp:80-108 (lane per 32-block, stride 64)
//   MXFP4: src/shaders/dmmv_mxfp4.comp:67-105 (lane per 17-byte block)
// Other types fall back to the sequential f32 dot.
// ---------------------------------------------------------------------------
static float row_dot_shader_order(const uint8_t* row, uint32_t type, uint32_t K, const float* x) {
    float lane[64];
    for (int i = 0; i < 64; ++i) lane[i] = 0.0f;
    switch (type) {
    case T_Q4_K:
    case T_Q5_K: {
        const uint32_t bpb = type == T_Q4_K ? 144 : 176;
        const uint32_t qs_off = type == T_Q4_K ? 16 : 48;
        const uint32_t bpr = K / 256;
        for (int tid = 0; tid < 64; ++tid) {
            const int itid = tid % 16, ix = tid / 16;
            const int il = itid / 4, ir = itid % 4;
            const int v_im = il / 2, v_in = il % 2;
            const int l0 = 4 * (2 * ir + v_in);
            const int q_offset = 32 * v_im + l0;
            const int y_off = 64 * v_im + l0;
            float sum = 0.0f;
            for (uint32_t i = ix; i < bpr; i += 4) {
                const uint8_t* b = row + (size_t)i * bpb;
                const float d = half_to_float(rd16(b)), dmin = half_to_float(rd16(b + 2));
                const float* xb = x + (size_t)i * 256 + y_off;
                uint8_t sc[4], mn[4];
                get_scale_min_k4(2 * v_im + 0, b + 4, &sc[0], &mn[0]);
                get_scale_min_k4(2 * v_im + 1, b + 4, &sc[1], &mn[1]);
                get_scale_min_k4(2 * v_im + 4, b + 4, &sc[2], &mn[2]);
                get_scale_min_k4(2 * v_im + 5, b + 4, &sc[3], &mn[3]);
                const uint8_t* q0 = b + qs_off + q_offset;
                const uint8_t* q1 = q0 + 64;
                for (int part = 0; part < 4; ++part) {
                    const float f = d * (float)sc[part], bias = dmin * (float)mn[part];
                    const uint8_t* q = part < 2 ? q0 : q1;
                    const float* xp = xb + (part & 1) * 32 + (part >> 1) * 128;
                    const int sub = 2 * v_im + (part & 1) + (part >> 1) * 4;  // sub-block 0..7
                    float dot = 0.0f;
                    for (int e = 0; e < 4; ++e) {
                        uint32_t nib = (part & 1) ? (q[e] >> 4) : (q[e] & 0xF);
                        if (type == T_Q5_K) {
                            const uint8_t qh = b[16 + l0 + e];
                            nib |= ((qh >> sub) & 1u) << 4;
                        }
                        dot += (f * (float)nib - bias) * xp[e];
                    }
                    sum += dot;
                }
            }
            lane[tid] = sum;
        }
        break;
    }
    case T_Q6_K: {
        const uint32_t bpr = K / 256;
        for (int tid = 0; tid < 64; ++tid) {
            const int itid = tid % 16, ix = tid / 16;
            const int v_im = itid / 8;          // which 128-half
            const int v_in = itid % 8;
            const int l0 = 4 * v_in;            // 4 consecutive l per lane
            const int is = l0 / 16;
            float sum = 0.0f;
            for (uint32_t i = ix; i < bpr; i += 4) {
                const uint8_t* b = row + (size_t)i * 210;
                const float d = half_to_float(rd16(b + 208));
                const uint8_t* ql = b + 64 * v_im;
                const uint8_t* qh = b + 128 + 32 * v_im;
                const int8_t* sc = (const int8_t*)(b + 192 + 8 * v_im);
                const float* xb = x + (size_t)i * 256 + 128 * v_im;
                const float ds0 = d * (float)sc[is], ds2 = d * (float)sc[is + 2];
                const float ds4 = d * (float)sc[is + 4], ds6 = d * (float)sc[is + 6];
                for (int e = 0; e < 4; ++e) {
                    const int l = l0 + e;
                    const uint32_t q1 = (ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4);
                    const uint32_t q2 = (ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4);
                    const uint32_t q3 = (ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4);
                    const uint32_t q4 = (ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4);
                    sum += ds0 * ((float)q1 - 32.0f) * xb[l];
                    sum += ds2 * ((float)q2 - 32.0f) * xb[l + 32];
                    sum += ds4 * ((float)q3 - 32.0f) * xb[l + 64];
                    sum += ds6 * ((float)q4 - 32.0f) * xb[l + 96];
                }
            }
            lane[tid] = sum;
        }
        break;
    }
    case T_Q8_0: {
        const uint32_t bpr = K / 32;
        for (int tid = 0; tid < 64; ++tid) {
            float sum = 0.0f;
            for (uint32_t i = tid; i < bpr; i += 64) {
                const uint8_t* b = row + (size_t)i * 34;
                const float d = half_to_float(rd16(b));
                const float* xb = x + (size_t)i * 32;
                float dot = 0.0f;
                for (int j = 0; j < 32; ++j) dot += (float)(int8_t)b[2 + j] * xb[j];
                sum += d * dot;
            }
            lane[tid] = sum;
        }
        break;
    }
    case T_MXFP4: {
        const uint32_t bpr = K / 32;
        for (int tid = 0; tid < 64; ++tid) {
            float sum = 0.0f;
            for (uint32_t i = tid; i < bpr; i += 64) {
                const uint8_t* b = row + (size_t)i * 17;
                const uint32_t bits = b[0] == 0 ? 0x00400000u : ((uint32_t)b[0] << 23);
                float d;
                std::memcpy(&d, &bits, 4);
                const float* xb = x + (size_t)i * 32;
                float dot = 0.0f;
                for (int j = 0; j < 16; ++j) {
                    dot += kMxfp4Lut[b[1 + j] & 0xF] * xb[j];
                    dot += kMxfp4Lut[b[1 + j] >> 4] * xb[j + 16];
                }
                sum += d * dot;
            }
            lane[tid] = sum;
        }
        break;
    }
    default: {
        std::vector<float> buf(K);
        const uint8_t* base = row;  // row 0 of a one-row view
        dequant_row(base, 0, K, type, buf.data());
        float acc = 0.0f;
        for (uint32_t i = 0; i < K; ++i) acc += buf[i] * x[i];
        return acc;
    }
    }
    // subgroupAdd: tree reduction over the 64 lanes
    for (int s = 32; s > 0; s >>= 1)
        for (int i = 0; i < s; ++i) lane[i] += lane[i + s];
    return lane[0];
}

int32_t zo_dmmv_shader_order(const uint8_t* raw, uint32_t type, uint32_t M, uint32_t K,
                             const float* x, float* y, uint32_t acc_mode, int32_t n_threads) {
    if (bytes_per_block(type) == 0) return -1;
    const uint64_t rb = row_bytes(type, K);
#ifdef _OPENMP
    if (n_threads > 0) omp_set_num_threads(n_threads);
#endif
    // one "workgroup" = two rows, as the shaders launch (M+1)/2 workgroups
#pragma omp parallel for schedule(static)
    for (int64_t wg = 0; wg < (int64_t)((M + 1) / 2); ++wg) {
        for (int rr = 0; rr < 2; ++rr) {
            const uint64_t r = (uint64_t)wg * 2 + rr;
            if (r >= M) break;
            const float v = row_dot_shader_order(raw + r * rb, type, K, x);
            y[r] = acc_mode ? y[r] + v : v;
        }
    }
    return 0;
}

int32_t zo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// ---------------------------------------------------------------------------
// MoE routing. Both write out_ids[k] and out_weights[k].
// ---------------------------------------------------------------------------

// topKSoftmax: softmax over all experts, pick top-k probabilities (strict >,
// ascending scan, so ties go to the lowest index), renormalise.
// src/compute/forward.zig:496-537
void zo_topk_softmax(const float* logits, uint32_t n, uint32_t k, uint32_t* out_ids, float* out_w) {
    float max_val = -std::numeric_limits<float>::infinity();
    for (uint32_t i = 0; i < n; ++i) if (logits[i] > max_val) max_val = logits[i];
    std::vector<float> probs(n);
    float sum = 0.0f;
    for (uint32_t i = 0; i < n; ++i) { probs[i] = std::exp(logits[i] - max_val); sum += probs[i]; }
    if (sum > 0) for (uint32_t i = 0; i < n; ++i) probs[i] /= sum;
    std::vector<char> used(n, 0);
    for (uint32_t ki = 0; ki < k; ++ki) {
        uint32_t best = 0; float bv = -1.0f;
        for (uint32_t i = 0; i < n; ++i) if (!used[i] && probs[i] > bv) { bv = probs[i]; best = i; }
        out_ids[ki] = best; out_w[ki] = bv; used[best] = 1;
    }
    float ws = 0.0f;
    for (uint32_t i = 0; i < k; ++i) ws += out_w[i];
    if (ws > 0) for (uint32_t i = 0; i < k; ++i) out_w[i] /= ws;
}

// topKSoftmaxWeight: top-k on the raw logits, softmax over the selected set.
// The GPU router (src/shaders/softmax_topk.comp:35-103) computes the same.
// src/compute/forward.zig:541-571
void zo_topk_softmax_weight(const float* logits, uint32_t n, uint32_t k, uint32_t* out_ids, float* out_w) {
    std::vector<char> used(n, 0);
    const float ninf = -std::numeric_limits<float>::infinity();
    for (uint32_t ki = 0; ki < k; ++ki) {
        uint32_t best = 0; float bv = ninf;
        for (uint32_t i = 0; i < n; ++i) if (!used[i] && logits[i] > bv) { bv = logits[i]; best = i; }
        out_ids[ki] = best; out_w[ki] = logits[best]; used[best] = 1;
    }
    float mx = ninf;
    for (uint32_t i = 0; i < k; ++i) if (out_w[i] > mx) mx = out_w[i];
    float sum = 0.0f;
    for (uint32_t i = 0; i < k; ++i) { out_w[i] = std::exp(out_w[i] - mx); sum += out_w[i]; }
    if (sum > 0) for (uint32_t i = 0; i < k; ++i) out_w[i] /= sum;
}

// ---------------------------------------------------------------------------
// Activation and combine steps either side of the expert matmuls.
// ---------------------------------------------------------------------------

// Fused RMS norm + f32 router matvec, src/shaders/rms_norm_dmmv_f32.comp:78-127:
// rms_inv = 1 / sqrt(sum(x^2) / K + eps); norm_out[i] = w[i] * (x[i] * rms_inv) in f32 with that
// multiplication order; logits[m] = sum_i W[m][i] * norm_out[i] (accumulated in f64 here).
void zo_rms_norm_dmmv_f32(const float* x, const float* w, const float* W, float* norm_out, double* logits, uint32_t M,
                          uint32_t K, float eps) {
    double ss = 0.0;
    for (uint32_t i = 0; i < K; ++i) ss += (double)x[i] * (double)x[i];
    const float rms_inv = (float)(1.0 / std::sqrt(ss / (double)K + (double)eps));
    for (uint32_t i = 0; i < K; ++i) norm_out[i] = w[i] * (x[i] * rms_inv);
    for (uint32_t m = 0; m < M; ++m) {
        double acc = 0.0;
        for (uint32_t i = 0; i < K; ++i) acc += (double)W[(size_t)m * K + i] * (double)norm_out[i];
        logits[m] = acc;
    }
}

// Merge of split-K flash-attention partials into the attention output vector,
// src/shaders/dmmv_q4k_o_proj_merge.comp:104-148: per head M_full = max over the chunks' maxima (and the sink, a
// NaN sink meaning none), w_c = exp(M_c - M_full) for chunks with L_c > 0, L_full = sum_c w_c L_c (+ the sink's
// exp), out[head*hd + d] = (sum_c fma(w_c, partial[(head*nc + c)*hd + d], acc)) / L_full (0 when L_full is 0).
// The LSE region {M_c, L_c} follows the partials at float index n_heads * nc * hd.
void zo_attn_merge(const float* partial, const float* sinks, float* out, uint32_t n_heads, uint32_t nc, uint32_t hd,
                   uint32_t sink_offset) {
    const size_t lse_base = (size_t)n_heads * nc * hd;
    for (uint32_t head = 0; head < n_heads; ++head) {
        const float* lse = partial + lse_base + (size_t)head * nc * 2;
        float Mg = lse[0];
        for (uint32_t c = 1; c < nc; ++c) Mg = std::max(Mg, lse[2 * c]);
        const float sink = sinks ? sinks[sink_offset + head] : NAN;
        const bool has_sink = !std::isnan(sink);
        const float Mf = has_sink ? std::max(Mg, sink) : Mg;
        std::vector<float> w(nc);
        float Lf = 0.0f;
        for (uint32_t c = 0; c < nc; ++c) {
            w[c] = lse[2 * c + 1] > 0.0f ? std::exp(lse[2 * c] - Mf) : 0.0f;
            Lf += w[c] * lse[2 * c + 1];
        }
        if (has_sink) Lf += std::exp(sink - Mf);
        const float inv = Lf > 0.0f ? 1.0f / Lf : 0.0f;
        for (uint32_t d = 0; d < hd; ++d) {
            float acc = 0.0f;
            for (uint32_t c = 0; c < nc; ++c) acc = std::fmaf(w[c], partial[((size_t)head * nc + c) * hd + d], acc);
            out[(size_t)head * hd + d] = acc * inv;
        }
    }
}

// src/shaders/swiglu.comp:25-33
void zo_swiglu(const float* gate, const float* up, float* out, uint32_t n) {
    for (uint32_t i = 0; i < n; ++i) {
        const float g = gate[i];
        out[i] = (g / (1.0f + std::exp(-g))) * up[i];
    }
}

// src/compute/forward.zig:607-616; src/shaders/swiglu_oai.comp:24-34
void zo_swiglu_oai(const float* gate, const float* up, float* out, uint32_t n) {
    const float alpha = 1.702f, limit = 7.0f;
    for (uint32_t i = 0; i < n; ++i) {
        const float g = std::fmin(gate[i], limit);
        const float u = std::fmax(-limit, std::fmin(up[i], limit));
        const float glu = g / (1.0f + std::exp(alpha * (-g)));
        out[i] = glu * (u + 1.0f);
    }
}

// a[i] += sum_j w_j * b[j*stride + i]; routing = [k ids][k f32-bit weights].
// src/shaders/moe_weighted_acc.comp:23-33
void zo_moe_weighted_acc(float* a, const float* b, const uint32_t* routing,
                         uint32_t n, uint32_t n_used, uint32_t src_stride) {
    for (uint32_t i = 0; i < n; ++i) {
        float sum = 0.0f;
        for (uint32_t j = 0; j < n_used; ++j) {
            float w;
            std::memcpy(&w, &routing[n_used + j], 4);
            sum += w * b[(size_t)j * src_stride + i];
        }
        a[i] += sum;
    }
}

// counts[e] = #cells equal to e over (ne01 rows) x (ne00 cells); strides in u32.
// src/shaders/count_experts.comp:58-83
void zo_count_experts(const uint32_t* a, uint32_t* counts, uint32_t n_experts,
                      uint32_t ne00, uint32_t ne01, uint32_t nb00, uint32_t nb01, uint32_t a_offset) {
    for (uint32_t e = 0; e < n_experts; ++e) {
        uint32_t c = 0;
        for (uint32_t i01 = 0; i01 < ne01; ++i01)
            for (uint32_t i00 = 0; i00 < ne00; ++i00)
                c += a[a_offset + (size_t)i01 * nb01 + (size_t)i00 * nb00] == e;
        counts[e] = c;
    }
}

// Per expert, the packed list of route ids (token*k + slot) in token order.
// src/shaders/metal/moe_route_pack.metal:13-36
void zo_moe_route_pack(const uint32_t* routing, uint32_t n_tokens, uint32_t n_experts, uint32_t k,
                       uint32_t routing_stride, uint32_t ids_stride, uint32_t* counts, uint32_t* ids) {
    for (uint32_t e = 0; e < n_experts; ++e) {
        uint32_t n = 0;
        for (uint32_t t = 0; t < n_tokens; ++t)
            for (uint32_t s = 0; s < k; ++s)
                if (routing[(size_t)t * routing_stride + s] == e) ids[(size_t)e * ids_stride + n++] = t * k + s;
        counts[e] = n;
    }
}

// dst[token][d] += sum_slot w * src[token*k + slot][d]
// src/shaders/metal/moe_route_scatter.metal:20-96
void zo_moe_route_scatter(const uint32_t* routing, const float* src, float* dst, uint32_t n_tokens,
                          uint32_t hidden, uint32_t k, uint32_t routing_stride) {
    for (uint32_t t = 0; t < n_tokens; ++t)
        for (uint32_t d = 0; d < hidden; ++d) {
            float sum = 0.0f;
            for (uint32_t s = 0; s < k; ++s) {
                float w;
                std::memcpy(&w, &routing[(size_t)t * routing_stride + k + s], 4);
                sum += w * src[((size_t)t * k + s) * hidden + d];
            }
            dst[(size_t)t * hidden + d] += sum;
        }
}

// MoE DMMV: Y[s][M] = W[routing[s]] X[s*x_expert_stride ..], f64 accumulate.
// src/compute/dmmv.zig:709-739; src/shaders/dmmv_q4k_moe_kpar.comp:56-175
int32_t zo_moe_dmmv_f64(const uint8_t* raw, uint32_t type, uint32_t M, uint32_t K,
                        uint64_t expert_stride, const uint32_t* routing, uint32_t n_used,
                        uint32_t x_expert_stride, const float* x, double* y) {
    for (uint32_t s = 0; s < n_used; ++s) {
        const int rc = zo_dmmv_f64(raw + (uint64_t)routing[s] * expert_stride, type, M, K,
                                   x + (size_t)s * x_expert_stride, y + (size_t)s * M);
        if (rc) return rc;
    }
    return 0;
}

}  // extern "C"
