// CPU restatement of the small f32 ops between the quantised linears.
// Test infrastructure only — see zq_oracle.h.
#include <cmath>
#include <cstring>
#include <limits>

#include "zq_oracle.h"

namespace {
constexpr size_t VL = 16;

// Transcendentals are evaluated in double and rounded once to f32 (correctly rounded for all but
// about one argument in 2^29). The reference calls Zig's own f32 routines (@exp, @cos, @sin,
// std.math.tanh), whose last bit is implementation-defined and not reproducible without a Zig
// toolchain; the double-rounded value is the deterministic stand-in both the oracle and the CUDA
// kernels use.
inline float exp_f32(float x) { return (float)std::exp((double)x); }
inline float tanh_f32(float x) { return (float)std::tanh((double)x); }
inline float cos_f32(float x) { return (float)std::cos((double)x); }
inline float sin_f32(float x) { return (float)std::sin((double)x); }

inline float reduce_lanes(const float* acc) {
    float s = acc[0];
    for (size_t l = 1; l < VL; ++l) s += acc[l];
    return s;
}

// dot of two f32 vectors the way the attention loops do it: VL lane accumulators over the
// multiple-of-VL prefix, in-order reduce, scalar tail (gpt2.zig:816-828, gemma3.zig:1087-1098).
inline float dot_lanes(const float* a, const float* b, size_t n) {
    float acc[VL];
    for (size_t l = 0; l < VL; ++l) acc[l] = 0.0f;
    size_t d = 0;
    for (; d + VL <= n; d += VL)
        for (size_t l = 0; l < VL; ++l) acc[l] += a[d + l] * b[d + l];
    float dot = reduce_lanes(acc);
    for (; d < n; ++d) dot += a[d] * b[d];
    return dot;
}
}  // namespace

extern "C" {

void zqo_layer_norm_rows(const float* x, const float* w, const float* b, float* out, size_t rows,
                         size_t dim) {
    const float eps = 1e-5f;
    for (size_t r = 0; r < rows; ++r) {
        const float* row = x + r * dim;
        float* o = out + r * dim;
        float acc[VL];
        for (size_t l = 0; l < VL; ++l) acc[l] = 0.0f;
        size_t i = 0;
        for (; i + VL <= dim; i += VL)
            for (size_t l = 0; l < VL; ++l) acc[l] += row[i + l];
        float mean = reduce_lanes(acc);
        for (; i < dim; ++i) mean += row[i];
        mean /= (float)dim;

        for (size_t l = 0; l < VL; ++l) acc[l] = 0.0f;
        for (i = 0; i + VL <= dim; i += VL)
            for (size_t l = 0; l < VL; ++l) {
                const float d = row[i + l] - mean;
                acc[l] += d * d;
            }
        float var = reduce_lanes(acc);
        for (; i < dim; ++i) {
            const float d = row[i] - mean;
            var += d * d;
        }
        var /= (float)dim;
        const float inv_std = 1.0f / std::sqrt(var + eps);
        for (i = 0; i < dim; ++i) o[i] = (row[i] - mean) * inv_std * w[i] + b[i];
    }
}

// One-pass statistics: var = E[x^2] - mean^2 (runtime_kernels.zig:148-213).
void zqo_layer_norm_forward(const float* x, float* out, const float* gamma, const float* beta,
                            size_t rows, size_t dim, float eps) {
    for (size_t r = 0; r < rows; ++r) {
        const float* row = x + r * dim;
        float* o = out + r * dim;
        float s = 0.0f, ss = 0.0f;
        for (size_t i = 0; i < dim; ++i) {
            s += row[i];
            ss += row[i] * row[i];
        }
        const float mean = s / (float)dim;
        const float var = ss / (float)dim - mean * mean;
        const float inv_std = 1.0f / std::sqrt(var + eps);
        for (size_t i = 0; i < dim; ++i) o[i] = (row[i] - mean) * inv_std * gamma[i] + beta[i];
    }
}

void zqo_rms_norm_rows(const float* x, const float* w, float* out, size_t rows, size_t dim,
                       float eps) {
    for (size_t r = 0; r < rows; ++r) {
        const float* row = x + r * dim;
        float* o = out + r * dim;
        float acc[VL];
        for (size_t l = 0; l < VL; ++l) acc[l] = 0.0f;
        size_t i = 0;
        for (; i + VL <= dim; i += VL)
            for (size_t l = 0; l < VL; ++l) acc[l] += row[i + l] * row[i + l];
        float ss = reduce_lanes(acc);
        for (; i < dim; ++i) ss += row[i] * row[i];
        const float inv = 1.0f / std::sqrt(ss / (float)dim + eps);
        for (i = 0; i < dim; ++i) o[i] = row[i] * inv * w[i];
    }
}

void zqo_rms_norm_in_place(float* x, const float* w, size_t dim, float eps) {
    float ss = 0.0f;
    for (size_t i = 0; i < dim; ++i) ss += x[i] * x[i];
    const float inv = 1.0f / std::sqrt(ss / (float)dim + eps);
    for (size_t i = 0; i < dim; ++i) x[i] = x[i] * inv * w[i];
}

void zqo_gelu_in_place(float* x, size_t n) {
    const float c = 0.7978845608f;
    for (size_t i = 0; i < n; ++i) {
        const float v = x[i];
        const float inner = c * (v + 0.044715f * v * v * v);
        x[i] = 0.5f * v * (1.0f + tanh_f32(inner));
    }
}

void zqo_softmax_gpt2(float* x, size_t n) {
    float mx = -std::numeric_limits<float>::infinity();
    for (size_t i = 0; i < n; ++i)
        if (x[i] > mx) mx = x[i];
    float sum = 0.0f;
    for (size_t j = 0; j < n; ++j) {
        x[j] = exp_f32(x[j] - mx);
        sum += x[j];
    }
    const float inv = 1.0f / sum;
    size_t i = 0;
    for (; i + VL <= n; i += VL)
        for (size_t l = 0; l < VL; ++l) x[i + l] *= inv;
    for (; i < n; ++i) x[i] /= sum;  // the scalar tail divides (gpt2.zig:728-730)
}

void zqo_softmax_gemma(float* x, size_t n) {
    float mx = -std::numeric_limits<float>::infinity();
    for (size_t i = 0; i < n; ++i)
        if (x[i] > mx) mx = x[i];
    float sum = 0.0f;
    for (size_t j = 0; j < n; ++j) {
        x[j] = exp_f32(x[j] - mx);
        sum += x[j];
    }
    const float inv = 1.0f / sum;
    for (size_t j = 0; j < n; ++j) x[j] *= inv;
}

void zqo_softmax_forward(float* data, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; ++r) zqo_softmax_gemma(data + r * cols, cols);
}

void zqo_rope_freqs(size_t head_dim, float base, float* freqs) {
    for (size_t i = 0; i < head_dim / 2; ++i) {
        const float e = -(float)(i * 2) / (float)head_dim;
        freqs[i] = std::pow(base, e);
    }
}

void zqo_rope(float* x, size_t pos, const float* freqs, size_t n_freqs) {
    const float p = (float)pos;
    for (size_t i = 0; i < n_freqs; ++i) {
        const float theta = p * freqs[i];
        const float c = cos_f32(theta), s = sin_f32(theta);
        const float x0 = x[2 * i], x1 = x[2 * i + 1];
        x[2 * i] = x0 * c - x1 * s;
        x[2 * i + 1] = x0 * s + x1 * c;
    }
}

uint32_t zqo_argmax(const float* logits, size_t n) {
    uint32_t best = 0;
    float bv = logits[0];
    for (size_t i = 1; i < n; ++i)
        if (logits[i] > bv) {
            bv = logits[i];
            best = (uint32_t)i;
        }
    return best;
}

void zqo_cached_attention(const float* q, const float* k_cache, const float* v_cache, float* out,
                          float* scores, size_t kv_len, size_t n_head, size_t head_dim,
                          size_t embed) {
    const float scale = 1.0f / std::sqrt((float)head_dim);
    memset(out, 0, embed * sizeof(float));
    for (size_t h = 0; h < n_head; ++h) {
        const size_t off = h * head_dim;
        for (size_t ki = 0; ki < kv_len; ++ki)
            scores[ki] = dot_lanes(q + off, k_cache + ki * embed + off, head_dim) * scale;
        zqo_softmax_gpt2(scores, kv_len);
        for (size_t ki = 0; ki < kv_len; ++ki) {
            const float w = scores[ki];
            const float* v = v_cache + ki * embed + off;
            for (size_t d = 0; d < head_dim; ++d) out[off + d] += w * v[d];
        }
    }
}

void zqo_causal_self_attention(const float* qkv, float* out, float* scores, size_t seq_len,
                               size_t n_head, size_t head_dim, size_t embed) {
    const float scale = 1.0f / std::sqrt((float)head_dim);
    memset(out, 0, seq_len * embed * sizeof(float));
    for (size_t h = 0; h < n_head; ++h) {
        const size_t qo = h * head_dim, ko = embed + h * head_dim, vo = 2 * embed + h * head_dim;
        for (size_t qi = 0; qi < seq_len; ++qi) {
            for (size_t ki = 0; ki <= qi; ++ki)
                scores[ki] =
                    dot_lanes(qkv + qi * 3 * embed + qo, qkv + ki * 3 * embed + ko, head_dim) *
                    scale;
            zqo_softmax_gpt2(scores, qi + 1);
            for (size_t ki = 0; ki <= qi; ++ki) {
                const float w = scores[ki];
                const float* v = qkv + ki * 3 * embed + vo;
                float* o = out + qi * embed + h * head_dim;
                for (size_t d = 0; d < head_dim; ++d) o[d] += w * v[d];
            }
        }
    }
}

void zqo_gqa_cached_attention(const float* q, const float* k_cache, const float* v_cache,
                              float* out, float* scores, size_t kv_start, size_t kv_end,
                              size_t n_head, size_t head_dim, size_t q_dim, size_t kv_dim) {
    const float scale = 1.0f / std::sqrt((float)head_dim);
    const size_t kv_len = kv_end - kv_start;
    memset(out, 0, q_dim * sizeof(float));
    for (size_t h = 0; h < n_head; ++h) {
        const size_t qo = h * head_dim;  // every query head reads KV head 0 (gemma3.zig:1083-1084)
        for (size_t ki = kv_start; ki < kv_end; ++ki)
            scores[ki - kv_start] = dot_lanes(q + qo, k_cache + ki * kv_dim, head_dim) * scale;
        zqo_softmax_gemma(scores, kv_len);
        for (size_t ki = kv_start; ki < kv_end; ++ki) {
            const float w = scores[ki - kv_start];
            const float* v = v_cache + ki * kv_dim;
            for (size_t d = 0; d < head_dim; ++d) out[qo + d] += w * v[d];
        }
    }
}

void zqo_gqa_causal_attention_prefill(const float* q, const float* k_cache, const float* v_cache,
                                      float* out, size_t seq_len, size_t n_head, size_t head_dim,
                                      size_t q_dim, size_t kv_dim, size_t window) {
    const float scale = 1.0f / std::sqrt((float)head_dim);
    memset(out, 0, seq_len * q_dim * sizeof(float));
    float* scores = new float[seq_len];
    for (size_t h = 0; h < n_head; ++h) {
        const size_t qo = h * head_dim;
        for (size_t qi = 0; qi < seq_len; ++qi) {
            const size_t kv_start = (qi + 1 > window) ? qi + 1 - window : 0;
            const size_t kv_end = qi + 1;
            for (size_t ki = kv_start; ki < kv_end; ++ki)
                scores[ki - kv_start] =
                    dot_lanes(q + qi * q_dim + qo, k_cache + ki * kv_dim, head_dim) * scale;
            zqo_softmax_gemma(scores, kv_end - kv_start);
            for (size_t ki = kv_start; ki < kv_end; ++ki) {
                const float w = scores[ki - kv_start];
                const float* v = v_cache + ki * kv_dim;
                float* o = out + qi * q_dim + qo;
                for (size_t d = 0; d < head_dim; ++d) o[d] += w * v[d];
            }
        }
    }
    delete[] scores;
}

}  // extern "C"
