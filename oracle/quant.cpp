// CPU restatement of zig-nn's block codecs and quantised dot products.
// Test infrastructure only — see zq_oracle.h.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

#include "zq_oracle.h"

namespace {

constexpr size_t QK = 32;  // BLOCK_SIZE, src/gguf/dequant.zig:47
constexpr size_t VL = 16;  // f32 lanes of the reference's SIMD vectors on an AVX-512 host

inline uint16_t load_u16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
inline void store_u16(uint8_t* p, uint16_t v) {
    p[0] = (uint8_t)(v & 0xFF);
    p[1] = (uint8_t)(v >> 8);
}

// In-order reduction of VL lanes: what @reduce(.Add, v) does for floats in strict mode.
inline float reduce_lanes(const float* acc) {
    float s = acc[0];
    for (size_t l = 1; l < VL; ++l) s += acc[l];
    return s;
}

// One block of the f32-activation dots (src/gguf/dequant.zig:153-161): two vector steps of VL
// lanes, acc = 0 + v[l]*x[l], then + v[l+16]*x[l+16]; lanes reduced in order.
inline float block_dot_lanes(const float* vals, const float* x) {
    float acc[VL];
    for (size_t l = 0; l < VL; ++l) acc[l] = 0.0f;
    for (size_t k = 0; k + VL <= QK; k += VL)
        for (size_t l = 0; l < VL; ++l) acc[l] += vals[k + l] * x[k + l];
    return reduce_lanes(acc);
}

inline float block_sum_lanes(const float* x) {
    float acc[VL];
    for (size_t l = 0; l < VL; ++l) acc[l] = 0.0f;
    for (size_t k = 0; k + VL <= QK; k += VL)
        for (size_t l = 0; l < VL; ++l) acc[l] += x[k + l];
    return reduce_lanes(acc);
}

// dot_i8x32 (src/gguf/simd_dot.zig:71-81): exact int32 dot of 32 int8 pairs.
inline int32_t dot_i8x32(const int8_t* a, const int8_t* b) {
    int32_t s = 0;
    for (size_t i = 0; i < QK; ++i) s += (int32_t)a[i] * (int32_t)b[i];
    return s;
}

}  // namespace

extern "C" {

size_t zqo_block_size(int type) {
    switch (type) {
        case ZQ_TYPE_F32:
        case ZQ_TYPE_F16: return 1;
        case ZQ_TYPE_Q4_0:
        case ZQ_TYPE_Q4_1:
        case ZQ_TYPE_Q8_0: return QK;
        default: return 0;
    }
}

size_t zqo_bytes_per_block(int type) {
    switch (type) {
        case ZQ_TYPE_F32: return 4;
        case ZQ_TYPE_F16: return 2;
        case ZQ_TYPE_Q4_0: return 18;
        case ZQ_TYPE_Q4_1: return 20;
        case ZQ_TYPE_Q8_0: return 34;
        default: return 0;
    }
}

size_t zqo_tensor_bytes(int type, size_t n) {
    size_t bs = zqo_block_size(type);
    if (bs == 0) return 0;
    return (n / bs) * zqo_bytes_per_block(type);
}

float zqo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    uint32_t exp = (h >> 10) & 0x1F;
    uint32_t man = h & 0x3FF;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: normalise
            int e = -1;
            do {
                man <<= 1;
                ++e;
            } while ((man & 0x400) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t zqo_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000);
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) return sign | (absx > 0x7F800000u ? 0x7E00 : 0x7C00);
    if (absx >= 0x477FF000u) return sign | 0x7C00;  // rounds to >= 65520 -> inf
    if (absx < 0x33000001u) return sign;            // below half the smallest subnormal
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7FFFFFu) | 0x800000u;
    uint32_t half;
    if (e < -14) {  // subnormal result
        int shift = 13 + (-14 - e);
        uint32_t q = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (q & 1))) ++q;
        half = q;
    } else {
        uint32_t q = m >> 13;
        uint32_t rem = m & 0x1FFF;
        if (rem > 0x1000 || (rem == 0x1000 && (q & 1))) ++q;
        half = ((uint32_t)(e + 15) << 10) + (q - 0x400);
    }
    return sign | (uint16_t)half;
}

// ---------------------------------------------------------------- encoders

void zqo_quantize_q4_0(const float* x, uint8_t* out, size_t n) {
    for (size_t b = 0; b < n / QK; ++b) {
        const float* xb = x + b * QK;
        uint8_t* ob = out + b * 18;
        float amax = 0.0f, smax = 0.0f;
        for (size_t j = 0; j < QK; ++j)
            if (std::fabs(xb[j]) > amax) {
                amax = std::fabs(xb[j]);
                smax = xb[j];
            }
        const float d = smax / -8.0f;
        store_u16(ob, zqo_f32_to_f16(d));
        uint8_t q[QK];
        for (size_t j = 0; j < QK; ++j) {
            float r = (d != 0.0f) ? std::round(xb[j] / d) + 8.0f : 8.0f;
            q[j] = (uint8_t)std::min(15.0f, std::max(0.0f, r));
        }
        for (size_t j = 0; j < 16; ++j) ob[2 + j] = (uint8_t)(q[j] | (q[j + 16] << 4));
    }
}

void zqo_quantize_q4_1(const float* x, uint8_t* out, size_t n) {
    for (size_t b = 0; b < n / QK; ++b) {
        const float* xb = x + b * QK;
        uint8_t* ob = out + b * 20;
        float mn = xb[0], mx = xb[0];
        for (size_t j = 1; j < QK; ++j) {
            mn = std::min(mn, xb[j]);
            mx = std::max(mx, xb[j]);
        }
        const float d = (mx - mn) / 15.0f;
        store_u16(ob, zqo_f32_to_f16(d));
        store_u16(ob + 2, zqo_f32_to_f16(mn));
        uint8_t q[QK];
        for (size_t j = 0; j < QK; ++j) {
            float r = (d != 0.0f) ? std::round((xb[j] - mn) / d) : 0.0f;
            q[j] = (uint8_t)std::min(15.0f, std::max(0.0f, r));
        }
        for (size_t j = 0; j < 16; ++j) ob[4 + j] = (uint8_t)(q[j] | (q[j + 16] << 4));
    }
}

void zqo_quantize_q8_0(const float* x, uint8_t* out, size_t n) {
    for (size_t b = 0; b < n / QK; ++b) {
        const float* xb = x + b * QK;
        uint8_t* ob = out + b * 34;
        float amax = 0.0f;
        for (size_t j = 0; j < QK; ++j) amax = std::max(amax, std::fabs(xb[j]));
        const float scale = (amax == 0.0f) ? 0.0f : amax / 127.0f;
        const float inv = (scale == 0.0f) ? 0.0f : 1.0f / scale;
        store_u16(ob, zqo_f32_to_f16(scale));
        for (size_t j = 0; j < QK; ++j) {
            int qi = (int)std::round(xb[j] * inv);
            qi = std::max(-128, std::min(127, qi));
            ob[2 + j] = (uint8_t)(int8_t)qi;
        }
    }
}

int zqo_quantize(int type, const float* x, uint8_t* out, size_t n) {
    switch (type) {
        case ZQ_TYPE_Q4_0: zqo_quantize_q4_0(x, out, n); return 0;
        case ZQ_TYPE_Q4_1: zqo_quantize_q4_1(x, out, n); return 0;
        case ZQ_TYPE_Q8_0: zqo_quantize_q8_0(x, out, n); return 0;
        default: return 1;
    }
}

// ---------------------------------------------------------------- decoders

int zqo_dequantize(int type, const uint8_t* src, float* dst, size_t n) {
    switch (type) {
        case ZQ_TYPE_F32:  // dequant.zig:68-73
            memcpy(dst, src, n * 4);
            return 0;
        case ZQ_TYPE_F16:  // dequant.zig:76-83
            for (size_t i = 0; i < n; ++i) dst[i] = zqo_f16_to_f32(load_u16(src + 2 * i));
            return 0;
        case ZQ_TYPE_Q4_0:  // dequant.zig:88-105
            for (size_t b = 0; b < n / QK; ++b) {
                const uint8_t* blk = src + b * 18;
                const float d = zqo_f16_to_f32(load_u16(blk));
                for (size_t j = 0; j < 16; ++j) {
                    const int lo = (int)(blk[2 + j] & 0x0F) - 8;
                    const int hi = (int)(blk[2 + j] >> 4) - 8;
                    dst[b * QK + j] = (float)lo * d;
                    dst[b * QK + j + 16] = (float)hi * d;
                }
            }
            return 0;
        case ZQ_TYPE_Q4_1:  // dequant.zig:191-207
            for (size_t b = 0; b < n / QK; ++b) {
                const uint8_t* blk = src + b * 20;
                const float d = zqo_f16_to_f32(load_u16(blk));
                const float m = zqo_f16_to_f32(load_u16(blk + 2));
                for (size_t j = 0; j < 16; ++j) {
                    const float lo = (float)(blk[4 + j] & 0x0F);
                    const float hi = (float)(blk[4 + j] >> 4);
                    dst[b * QK + j] = lo * d + m;
                    dst[b * QK + j + 16] = hi * d + m;
                }
            }
            return 0;
        case ZQ_TYPE_Q8_0:  // dequant.zig:110-123
            for (size_t b = 0; b < n / QK; ++b) {
                const uint8_t* blk = src + b * 34;
                const float d = zqo_f16_to_f32(load_u16(blk));
                for (size_t j = 0; j < QK; ++j) dst[b * QK + j] = (float)(int8_t)blk[2 + j] * d;
            }
            return 0;
        default: return 1;
    }
}

// ------------------------------------------------- f32-activation dots

float zqo_dot_f32(int type, const uint8_t* row, const float* x, size_t in_dim) {
    const size_t nb = in_dim / QK;
    float sum = 0.0f;
    float vals[QK];
    if (type == ZQ_TYPE_Q4_0) {  // dequant.zig:133-164
        for (size_t b = 0; b < nb; ++b) {
            const uint8_t* blk = row + b * 18;
            const float d = zqo_f16_to_f32(load_u16(blk));
            for (size_t j = 0; j < 16; ++j) {
                vals[j] = (float)((int)(blk[2 + j] & 0x0F) - 8);
                vals[j + 16] = (float)((int)(blk[2 + j] >> 4) - 8);
            }
            sum += block_dot_lanes(vals, x + b * QK) * d;
        }
    } else if (type == ZQ_TYPE_Q4_1) {  // dequant.zig:210-243
        for (size_t b = 0; b < nb; ++b) {
            const uint8_t* blk = row + b * 20;
            const float d = zqo_f16_to_f32(load_u16(blk));
            const float m = zqo_f16_to_f32(load_u16(blk + 2));
            for (size_t j = 0; j < 16; ++j) {
                vals[j] = (float)(blk[4 + j] & 0x0F);
                vals[j + 16] = (float)(blk[4 + j] >> 4);
            }
            const float a = block_dot_lanes(vals, x + b * QK) * d;
            const float c = block_sum_lanes(x + b * QK) * m;
            sum += a + c;
        }
    } else if (type == ZQ_TYPE_Q8_0) {  // dequant.zig:265-294
        for (size_t b = 0; b < nb; ++b) {
            const uint8_t* blk = row + b * 34;
            const float d = zqo_f16_to_f32(load_u16(blk));
            for (size_t j = 0; j < QK; ++j) vals[j] = (float)(int8_t)blk[2 + j];
            sum += block_dot_lanes(vals, x + b * QK) * d;
        }
    } else if (type == ZQ_TYPE_F32) {  // f32 weight branch of linear_forward_q, gpt2.zig:652-671
        const float* w = (const float*)row;
        float acc[VL];
        for (size_t l = 0; l < VL; ++l) acc[l] = 0.0f;
        size_t k = 0;
        for (; k + VL <= in_dim; k += VL)
            for (size_t l = 0; l < VL; ++l) acc[l] += x[k + l] * w[k + l];
        sum = reduce_lanes(acc);
        for (; k < in_dim; ++k) sum += x[k] * w[k];
    }
    return sum;
}

int zqo_matmul_f32(int type, const uint8_t* w, const float* x, float* y, size_t out_dim,
                   size_t in_dim, int n_threads) {
    if (type != ZQ_TYPE_Q4_0 && type != ZQ_TYPE_Q4_1 && type != ZQ_TYPE_Q8_0 &&
        type != ZQ_TYPE_F32)
        return 1;
    const size_t row_bytes = zqo_tensor_bytes(type, in_dim);
    // Row split across threads never changes a row's arithmetic (dequant.zig:341-403).
#pragma omp parallel for schedule(static) num_threads(n_threads > 0 ? n_threads : 1)
    for (long j = 0; j < (long)out_dim; ++j)
        y[j] = zqo_dot_f32(type, w + (size_t)j * row_bytes, x, in_dim);
    return 0;
}

// ------------------------------------------------- Q8 activation path

void zqo_quantize_row_q8(const float* x, zqo_q8_block* out, size_t n) {
    for (size_t b = 0; b < n / QK; ++b) {  // simd_dot.zig:25-64
        const float* c = x + b * QK;
        float amax = 0.0f;
        for (size_t j = 0; j < QK; ++j) amax = std::max(amax, std::fabs(c[j]));
        const float scale = (amax > 0.0f) ? amax / 127.0f : 1.0f;
        const float inv = 1.0f / scale;
        zqo_q8_block blk;
        blk.scale = scale;
        int32_t s = 0;
        for (size_t j = 0; j < QK; ++j) {
            const float v = c[j] * inv;
            float r = std::round(v);  // half away from zero, as std.math.round
            r = std::min(127.0f, std::max(-127.0f, r));
            blk.q[j] = (int8_t)r;
            s += blk.q[j];
        }
        blk.sum = s;
        out[b] = blk;
    }
}

float zqo_dot_q8(int type, const uint8_t* row, const zqo_q8_block* xq, size_t nb) {
    float sum = 0.0f;
    int8_t wi[QK];
    if (type == ZQ_TYPE_Q4_0) {  // simd_dot.zig:86-106
        for (size_t b = 0; b < nb; ++b) {
            const uint8_t* blk = row + b * 18;
            const float d = zqo_f16_to_f32(load_u16(blk));
            for (size_t j = 0; j < 16; ++j) {
                wi[j] = (int8_t)((int)(blk[2 + j] & 0x0F) - 8);
                wi[j + 16] = (int8_t)((int)(blk[2 + j] >> 4) - 8);
            }
            const int32_t idot = dot_i8x32(wi, xq[b].q);
            sum += d * xq[b].scale * (float)idot;  // (d*s)*idot, left to right
        }
    } else if (type == ZQ_TYPE_Q4_1) {  // simd_dot.zig:110-134
        for (size_t b = 0; b < nb; ++b) {
            const uint8_t* blk = row + b * 20;
            const float d = zqo_f16_to_f32(load_u16(blk));
            const float m = zqo_f16_to_f32(load_u16(blk + 2));
            for (size_t j = 0; j < 16; ++j) {
                wi[j] = (int8_t)(blk[4 + j] & 0x0F);
                wi[j + 16] = (int8_t)(blk[4 + j] >> 4);
            }
            const int32_t idot = dot_i8x32(wi, xq[b].q);
            const float s = xq[b].scale;
            const float t1 = d * s * (float)idot;
            const float t2 = m * s * (float)xq[b].sum;
            sum += t1 + t2;
        }
    } else if (type == ZQ_TYPE_Q8_0) {  // simd_dot.zig:137-152
        for (size_t b = 0; b < nb; ++b) {
            const uint8_t* blk = row + b * 34;
            const float d = zqo_f16_to_f32(load_u16(blk));
            const int32_t idot = dot_i8x32((const int8_t*)(blk + 2), xq[b].q);
            sum += d * xq[b].scale * (float)idot;
        }
    }
    return sum;
}

int zqo_matmul_q8(int type, const uint8_t* w, const float* x, float* y, size_t out_dim,
                  size_t in_dim, int n_threads, int allow_long) {
    if (type != ZQ_TYPE_Q4_0 && type != ZQ_TYPE_Q4_1 && type != ZQ_TYPE_Q8_0) return 1;
    if (in_dim > 8192 && !allow_long) return 2;  // MAX_Q8_BLOCKS = 256, thread_pool.zig:21
    const size_t nb = in_dim / QK;
    const size_t row_bytes = zqo_tensor_bytes(type, in_dim);
    std::vector<zqo_q8_block> xq(nb);
    zqo_quantize_row_q8(x, xq.data(), in_dim);  // once, before the row split (thread_pool.zig:111-114)
    const zqo_q8_block* xqp = xq.data();
#pragma omp parallel for schedule(static) num_threads(n_threads > 0 ? n_threads : 1)
    for (long j = 0; j < (long)out_dim; ++j)
        y[j] = zqo_dot_q8(type, w + (size_t)j * row_bytes, xqp, nb);
    return 0;
}

int zqo_linear(int type, const uint8_t* w, const float* x, float* y, size_t m_rows,
               size_t out_dim, size_t in_dim, int act_mode, int n_threads) {
    for (size_t m = 0; m < m_rows; ++m) {
        int rc = act_mode == 1 ? zqo_matmul_q8(type, w, x + m * in_dim, y + m * out_dim, out_dim,
                                               in_dim, n_threads, 1)
                               : zqo_matmul_f32(type, w, x + m * in_dim, y + m * out_dim, out_dim,
                                                in_dim, n_threads);
        if (rc) return rc;
    }
    return 0;
}


// ------------------------------------------------- transposed matmul (backward w.r.t. activations)

// grad_x[m][k] (+)= sum_j grad_out[m][j] * W[j][k], j ascending, f32: the statement of
// matmul_q4_0_trans_batched / _q4_1_ / _q8_0_ (src/backend/shaders/nn_training_kernels.metal:1149-1242):
// each weight is decoded as there (d * (q - 8), d * q + m, d * q) and `acc += g * w` runs over the weight
// rows in order; the finished sum is added to grad_x (the shader accumulates; accumulate == 0 stores).
int zqo_matmul_transposed(int type, const uint8_t* w, const float* grad_out, float* grad_x, size_t m_rows,
                          size_t out_dim, size_t in_dim, int accumulate, int n_threads) {
    if (type != ZQ_TYPE_Q4_0 && type != ZQ_TYPE_Q4_1 && type != ZQ_TYPE_Q8_0) return 1;
    const size_t row_bytes = zqo_tensor_bytes(type, in_dim);
#pragma omp parallel num_threads(n_threads > 0 ? n_threads : 1)
    {
        std::vector<float> wrow(in_dim), acc(in_dim);
#pragma omp for schedule(static)
        for (long m = 0; m < (long)m_rows; ++m) {
            std::fill(acc.begin(), acc.end(), 0.0f);
            for (size_t j = 0; j < out_dim; ++j) {
                zqo_dequantize(type, w + j * row_bytes, wrow.data(), in_dim);
                const float g = grad_out[(size_t)m * out_dim + j];
                for (size_t k = 0; k < in_dim; ++k) acc[k] += g * wrow[k];
            }
            float* o = grad_x + (size_t)m * in_dim;
            for (size_t k = 0; k < in_dim; ++k) o[k] = accumulate ? o[k] + acc[k] : acc[k];
        }
    }
    return 0;
}

}  // extern "C"
