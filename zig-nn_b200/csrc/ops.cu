// Small f32 ops that sit between the quantised linears: norms, RoPE, GELU / GeGLU, softmax,
// KV-cache write, single-query attention, and the forward kernels behind zig-nn's
// src/cuda_ops.zig dispatchers (softmax, layer norm, gelu, broadcast add / mul, gather, scale).
#include <math.h>

#include "zq_internal.h"

namespace zq {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    return v;
}

// Block-wide sum / max; every thread gets the result. `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

__device__ __forceinline__ float gelu_tanh(float v) {
    const float inner = 0.7978845608f * (v + 0.044715f * v * v * v);
    return 0.5f * v * (1.0f + tanhf(inner));
}

// mode 0: out = norm(x)*w ; mode 1: out(residual) += norm(x)*w
__global__ void __launch_bounds__(256)
rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out,
                uint32_t dim, float eps, int mode) {
    __shared__ float red[33];
    const float* row = x + (size_t)blockIdx.x * dim;
    float* o = out + (size_t)blockIdx.x * dim;
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = __fmul_rn(__fmul_rn(row[i], inv), w[i]);
        o[i] = mode ? o[i] + v : v;
    }
}

// One warp per vector (per-head q/k norm, src/models/gemma3.zig:949-959).
__global__ void rms_norm_vec_kernel(float* __restrict__ x, const float* __restrict__ w, uint32_t dim,
                                    uint32_t n_vec, float eps) {
    const uint32_t v = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (v >= n_vec) return;
    float* p = x + (size_t)v * dim;
    float ss = 0.0f;
    for (uint32_t i = lane; i < dim; i += 32) ss = fmaf(p[i], p[i], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    for (uint32_t i = lane; i < dim; i += 32) p[i] = __fmul_rn(__fmul_rn(p[i], inv), w[i]);
}

__global__ void rope_kernel(float* __restrict__ x, const float* __restrict__ freqs, uint32_t half_dim,
                            uint32_t n_heads, float pos) {
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= half_dim * n_heads) return;
    const uint32_t i = idx % half_dim, h = idx / half_dim;
    const float theta = __fmul_rn(pos, freqs[i]);
    float s, c;
    sincosf(theta, &s, &c);
    float* p = x + (size_t)h * half_dim * 2 + 2 * i;
    const float x0 = p[0], x1 = p[1];
    p[0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    p[1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

__global__ void gelu_kernel(float* __restrict__ out, const float* __restrict__ x, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = gelu_tanh(x[i]);
}
__global__ void gelu_mul_kernel(float* __restrict__ gate, const float* __restrict__ up, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) gate[i] = gelu_tanh(gate[i]) * up[i];
}
__global__ void add_broadcast_kernel(float* __restrict__ out, const float* __restrict__ a,
                                     const float* __restrict__ b, size_t a_total, size_t b_total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < a_total) out[i] = a[i] + b[i % b_total];
}
__global__ void mul_broadcast_kernel(float* __restrict__ out, const float* __restrict__ a,
                                     const float* __restrict__ b, size_t a_total, size_t b_total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < a_total) out[i] = a[i] * b[i % b_total];
}
__global__ void gather_kernel(float* __restrict__ out, const float* __restrict__ table,
                              const int32_t* __restrict__ idx, uint32_t num, uint32_t dim) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)num * dim) return;
    const size_t r = i / dim, c = i - r * dim;
    out[i] = table[(size_t)idx[r] * dim + c];
}
__global__ void scale_kernel(float* __restrict__ out, const float* __restrict__ x, float s, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = x[i] * s;
}
__global__ void write_kv_kernel(const float* __restrict__ k, const float* __restrict__ v,
                                float* __restrict__ kc, float* __restrict__ vc, uint32_t pos,
                                uint32_t kv_dim) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < kv_dim) {
        kc[(size_t)pos * kv_dim + i] = k[i];
        vc[(size_t)pos * kv_dim + i] = v[i];
    }
}

// Row softmax: max, exp(x - max), times 1/sum (runtime_kernels.zig:40-81).
__global__ void __launch_bounds__(256)
softmax_kernel(float* __restrict__ out, const float* __restrict__ x, uint32_t cols) {
    __shared__ float red[33];
    const float* row = x + (size_t)blockIdx.x * cols;
    float* o = out + (size_t)blockIdx.x * cols;
    float mx = -INFINITY;
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, red);
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
        const float e = expf(row[i] - mx);
        o[i] = e;
        s += e;
    }
    s = block_sum(s, red);
    const float inv = 1.0f / s;
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) o[i] *= inv;
}

// Two-pass layer norm: mean, then sum (x-mean)^2 (gpt2.zig:541-596; forward_structured.cu:154-198).
__global__ void __launch_bounds__(256)
layer_norm_kernel(float* __restrict__ out, const float* __restrict__ x, const float* __restrict__ gamma,
                  const float* __restrict__ beta, uint32_t cols, float eps) {
    __shared__ float red[33];
    const float* row = x + (size_t)blockIdx.x * cols;
    float* o = out + (size_t)blockIdx.x * cols;
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) s += row[i];
    const float mean = block_sum(s, red) / (float)cols;
    float v = 0.0f;
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
        const float d = row[i] - mean;
        v = fmaf(d, d, v);
    }
    const float var = block_sum(v, red) / (float)cols;
    const float inv_std = 1.0f / sqrtf(var + eps);
    for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x)
        o[i] = __fadd_rn(__fmul_rn(__fmul_rn(row[i] - mean, inv_std), gamma[i]), beta[i]);
}

// Single-query attention over a KV cache, one CTA per query head.
// scores[p] = dot(q_h, k[p]) / sqrt(head_dim) for kv_start <= p < kv_end, softmax, out = sum w*v.
__global__ void __launch_bounds__(256)
attention_decode_kernel(const float* __restrict__ q, const float* __restrict__ kc,
                        const float* __restrict__ vc, float* __restrict__ out, uint32_t n_head,
                        uint32_t n_kv_head, uint32_t head_dim, uint32_t kv_start, uint32_t kv_end) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[33];
    const uint32_t h = blockIdx.x;
    const uint32_t kvh = h / (n_head / n_kv_head);
    const uint32_t kv_dim = n_kv_head * head_dim;
    const uint32_t kv_len = kv_end - kv_start;
    float* scores = sm;            // kv_len
    float* part = sm + kv_len;     // groups * head_dim
    const float* qh = q + (size_t)h * head_dim;
    const float scale = 1.0f / sqrtf((float)head_dim);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;

    for (uint32_t p = warp; p < kv_len; p += nw) {
        const float* kr = kc + (size_t)(kv_start + p) * kv_dim + (size_t)kvh * head_dim;
        float acc = 0.0f;
        for (uint32_t d = lane; d < head_dim; d += 32) acc = fmaf(qh[d], kr[d], acc);
        acc = warp_sum(acc);
        if (lane == 0) scores[p] = acc * scale;
    }
    __syncthreads();
    float mx = -INFINITY;
    for (uint32_t p = threadIdx.x; p < kv_len; p += blockDim.x) mx = fmaxf(mx, scores[p]);
    mx = block_max(mx, red);
    float s = 0.0f;
    for (uint32_t p = threadIdx.x; p < kv_len; p += blockDim.x) {
        const float e = expf(scores[p] - mx);
        scores[p] = e;
        s += e;
    }
    s = block_sum(s, red);
    const float inv = 1.0f / s;
    for (uint32_t p = threadIdx.x; p < kv_len; p += blockDim.x) scores[p] *= inv;
    __syncthreads();

    // Weighted sum of V: thread groups of head_dim lanes split the positions.
    const uint32_t groups = blockDim.x / head_dim > 0 ? blockDim.x / head_dim : 1;
    if (head_dim <= blockDim.x) {
        const uint32_t grp = threadIdx.x / head_dim, d = threadIdx.x % head_dim;
        if (grp < groups) {
            float acc = 0.0f;
            for (uint32_t p = grp; p < kv_len; p += groups)
                acc = fmaf(scores[p], vc[(size_t)(kv_start + p) * kv_dim + (size_t)kvh * head_dim + d], acc);
            part[grp * head_dim + d] = acc;
        }
        __syncthreads();
        if (threadIdx.x < head_dim) {
            float acc = 0.0f;
            for (uint32_t g2 = 0; g2 < groups; ++g2) acc += part[g2 * head_dim + threadIdx.x];
            out[(size_t)h * head_dim + threadIdx.x] = acc;
        }
    } else {
        for (uint32_t d = threadIdx.x; d < head_dim; d += blockDim.x) {
            float acc = 0.0f;
            for (uint32_t p = 0; p < kv_len; ++p)
                acc = fmaf(scores[p], vc[(size_t)(kv_start + p) * kv_dim + (size_t)kvh * head_dim + d], acc);
            out[(size_t)h * head_dim + d] = acc;
        }
    }
}

inline unsigned grid1d(size_t n, unsigned threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace
}  // namespace zq

using namespace zq;

extern "C" {

int zq_rms_norm(const float* d_x, const float* d_w, float* d_out, uint32_t dim, uint32_t rows,
                float eps, zq_stream stream) {
    if (!d_x || !d_w || !d_out || dim == 0) return ZQ_ERR_BAD_ARG;
    if (rows == 0) return ZQ_OK;
    rms_norm_kernel<<<rows, 256, 0, as_stream(stream)>>>(d_x, d_w, d_out, dim, eps, 0);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_rms_norm_residual(const float* d_x, const float* d_w, float* d_residual, uint32_t dim,
                         uint32_t rows, float eps, zq_stream stream) {
    if (!d_x || !d_w || !d_residual || dim == 0) return ZQ_ERR_BAD_ARG;
    if (rows == 0) return ZQ_OK;
    rms_norm_kernel<<<rows, 256, 0, as_stream(stream)>>>(d_x, d_w, d_residual, dim, eps, 1);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_rms_norm_in_place(float* d_x, const float* d_w, uint32_t dim, uint32_t n_vec, float eps,
                         zq_stream stream) {
    if (!d_x || !d_w || dim == 0) return ZQ_ERR_BAD_ARG;
    if (n_vec == 0) return ZQ_OK;
    rms_norm_vec_kernel<<<grid1d((size_t)n_vec * 32, 128), 128, 0, as_stream(stream)>>>(d_x, d_w, dim,
                                                                                       n_vec, eps);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_rope(float* d_x, const float* d_freqs, uint32_t half_dim, uint32_t n_heads, float pos,
            zq_stream stream) {
    if (!d_x || !d_freqs || half_dim == 0) return ZQ_ERR_BAD_ARG;
    if (n_heads == 0) return ZQ_OK;
    rope_kernel<<<grid1d((size_t)half_dim * n_heads, 128), 128, 0, as_stream(stream)>>>(
        d_x, d_freqs, half_dim, n_heads, pos);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_rope_freqs_host(uint32_t head_dim, float rope_base, float* h_freqs) {
    if (!h_freqs || head_dim == 0 || head_dim % 2) return ZQ_ERR_BAD_ARG;
    for (uint32_t i = 0; i < head_dim / 2; ++i) {
        const float e = -(float)(i * 2) / (float)head_dim;
        h_freqs[i] = powf(rope_base, e);
    }
    return ZQ_OK;
}

int zq_gelu_mul(float* d_gate, const float* d_up, size_t n, zq_stream stream) {
    if (!d_gate || !d_up) return ZQ_ERR_BAD_ARG;
    if (n == 0) return ZQ_OK;
    gelu_mul_kernel<<<grid1d(n, 256), 256, 0, as_stream(stream)>>>(d_gate, d_up, n);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_write_kv_cache(const float* d_k, const float* d_v, float* d_k_cache, float* d_v_cache,
                      uint32_t pos, uint32_t kv_dim, zq_stream stream) {
    if (!d_k || !d_v || !d_k_cache || !d_v_cache || kv_dim == 0) return ZQ_ERR_BAD_ARG;
    write_kv_kernel<<<grid1d(kv_dim, 256), 256, 0, as_stream(stream)>>>(d_k, d_v, d_k_cache, d_v_cache,
                                                                      pos, kv_dim);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_attention_decode(const float* d_q, const float* d_k_cache, const float* d_v_cache,
                        float* d_out, uint32_t n_head, uint32_t n_kv_head, uint32_t head_dim,
                        uint32_t kv_start, uint32_t kv_end, zq_stream stream) {
    if (!d_q || !d_k_cache || !d_v_cache || !d_out) return ZQ_ERR_BAD_ARG;
    if (n_head == 0 || n_kv_head == 0 || head_dim == 0 || n_head % n_kv_head) return ZQ_ERR_BAD_ARG;
    if (kv_end <= kv_start) return ZQ_ERR_BAD_ARG;
    const uint32_t kv_len = kv_end - kv_start;
    const unsigned threads = 256;
    const uint32_t groups = threads / head_dim > 0 ? threads / head_dim : 1;
    const size_t smem = ((size_t)kv_len + (size_t)groups * head_dim) * sizeof(float);
    if (smem > 200 * 1024) return ZQ_ERR_LIMIT;
    if (smem > 48 * 1024)
        ZQ_CUDA(cudaFuncSetAttribute(attention_decode_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attention_decode_kernel<<<n_head, threads, smem, as_stream(stream)>>>(
        d_q, d_k_cache, d_v_cache, d_out, n_head, n_kv_head, head_dim, kv_start, kv_end);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_softmax_out(float* d_out, const float* d_x, uint32_t rows, uint32_t cols, zq_stream stream) {
    if (!d_out || !d_x || cols == 0) return ZQ_ERR_BAD_ARG;
    if (rows == 0) return ZQ_OK;
    softmax_kernel<<<rows, 256, 0, as_stream(stream)>>>(d_out, d_x, cols);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_softmax(float* d_data, uint32_t rows, uint32_t cols, zq_stream stream) {
    return zq_softmax_out(d_data, d_data, rows, cols, stream);
}

int zq_layer_norm(float* d_out, const float* d_x, const float* d_gamma, const float* d_beta,
                  uint32_t rows, uint32_t cols, float eps, zq_stream stream) {
    if (!d_out || !d_x || !d_gamma || !d_beta || cols == 0) return ZQ_ERR_BAD_ARG;
    if (rows == 0) return ZQ_OK;
    layer_norm_kernel<<<rows, 256, 0, as_stream(stream)>>>(d_out, d_x, d_gamma, d_beta, cols, eps);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_gelu(float* d_out, const float* d_x, size_t n, zq_stream stream) {
    if (!d_out || !d_x) return ZQ_ERR_BAD_ARG;
    if (n == 0) return ZQ_OK;
    gelu_kernel<<<grid1d(n, 256), 256, 0, as_stream(stream)>>>(d_out, d_x, n);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_add_broadcast(float* d_out, const float* d_a, const float* d_b, size_t a_total, size_t b_total,
                     zq_stream stream) {
    if (!d_out || !d_a || !d_b || b_total == 0) return ZQ_ERR_BAD_ARG;
    if (a_total == 0) return ZQ_OK;
    add_broadcast_kernel<<<grid1d(a_total, 256), 256, 0, as_stream(stream)>>>(d_out, d_a, d_b, a_total,
                                                                            b_total);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_mul_broadcast(float* d_out, const float* d_a, const float* d_b, size_t a_total, size_t b_total,
                     zq_stream stream) {
    if (!d_out || !d_a || !d_b || b_total == 0) return ZQ_ERR_BAD_ARG;
    if (a_total == 0) return ZQ_OK;
    mul_broadcast_kernel<<<grid1d(a_total, 256), 256, 0, as_stream(stream)>>>(d_out, d_a, d_b, a_total,
                                                                            b_total);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_gather(float* d_out, const float* d_table, const int32_t* d_idx, uint32_t num_indices,
              uint32_t embed_dim, zq_stream stream) {
    if (!d_out || !d_table || !d_idx || embed_dim == 0) return ZQ_ERR_BAD_ARG;
    if (num_indices == 0) return ZQ_OK;
    gather_kernel<<<grid1d((size_t)num_indices * embed_dim, 256), 256, 0, as_stream(stream)>>>(
        d_out, d_table, d_idx, num_indices, embed_dim);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_scale(float* d_out, const float* d_x, float s, size_t n, zq_stream stream) {
    if (!d_out || !d_x) return ZQ_ERR_BAD_ARG;
    if (n == 0) return ZQ_OK;
    scale_kernel<<<grid1d(n, 256), 256, 0, as_stream(stream)>>>(d_out, d_x, s, n);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

}  // extern "C"
