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

// Transcendentals are evaluated in double and rounded once to f32, the same definition the CPU
// checker uses; every multiply and add below is a separate rounding (no FMA contraction), in the
// order the CPU code performs them.
__device__ __forceinline__ float exp_f32(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float tanh_f32(float x) { return (float)tanh((double)x); }

// 0.5*v*(1+tanh(0.7978845608*(v+0.044715*v*v*v))) — src/models/gpt2.zig:690-697
__device__ __forceinline__ float gelu_tanh(float v) {
    const float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v);
    const float inner = __fmul_rn(0.7978845608f, __fadd_rn(v, cube));
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanh_f32(inner)));
}

// Sum of squares in the order of the CPU loop (src/models/gemma3.zig:920-930): 16 lane
// accumulators over the multiple-of-16 prefix (lane l takes x[l], x[l+16], ...), lanes added in
// order 0..15, then the tail elements one by one. `xs` is the row in shared memory; the result is
// returned to every thread through `bc`.
__device__ __forceinline__ float sumsq_lanes16(const float* xs, uint32_t dim, float* part, float* bc) {
    const uint32_t dim16 = dim & ~15u;
    if (threadIdx.x < 16) {
        // eight loads and squares at a time, then the eight dependent adds: the add chain, not the
        // shared-memory latency, sets the time
        float acc = 0.0f;
        uint32_t i = threadIdx.x;
        for (; i + 16 * 7 < dim16; i += 16 * 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = xs[i + 16 * u];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __fmul_rn(v[u], v[u]);
#pragma unroll
            for (int u = 0; u < 8; ++u) acc = __fadd_rn(acc, v[u]);
        }
        for (; i < dim16; i += 16) acc = __fadd_rn(acc, __fmul_rn(xs[i], xs[i]));
        part[threadIdx.x] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float ss = part[0];
#pragma unroll
        for (int l = 1; l < 16; ++l) ss = __fadd_rn(ss, part[l]);
        for (uint32_t i = dim16; i < dim; ++i) ss = __fadd_rn(ss, __fmul_rn(xs[i], xs[i]));
        *bc = ss;
    }
    __syncthreads();
    return *bc;
}

// Squares added one by one in index order (rms_norm_in_place, src/models/gemma3.zig:949-959), with the
// loads and squares of eight elements issued ahead of their adds.
__device__ __forceinline__ float sumsq_sequential(const float* xs, uint32_t dim) {
    float ss = 0.0f;
    uint32_t i = 0;
    for (; i + 8 <= dim; i += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = xs[i + u];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __fmul_rn(v[u], v[u]);
#pragma unroll
        for (int u = 0; u < 8; ++u) ss = __fadd_rn(ss, v[u]);
    }
    for (; i < dim; ++i) ss = __fadd_rn(ss, __fmul_rn(xs[i], xs[i]));
    return ss;
}

// mode 0: out = norm(x)*w ; mode 1: out(residual) += norm(x)*w.  Bit-identical to rms_norm_rows.
__global__ void __launch_bounds__(256)
rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out,
                uint32_t dim, float eps, int mode) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float part[16];
    __shared__ float bc;
    const float* row = x + (size_t)blockIdx.x * dim;
    float* o = out + (size_t)blockIdx.x * dim;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) xs[i] = row[i];
    __syncthreads();
    const float ss = sumsq_lanes16(xs, dim, part, &bc);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = __fmul_rn(__fmul_rn(xs[i], inv), w[i]);
        o[i] = mode ? __fadd_rn(o[i], v) : v;
    }
}

// One CTA of 64 threads per vector, squares summed one by one as rms_norm_in_place does
// (src/models/gemma3.zig:949-959).
__global__ void __launch_bounds__(64)
rms_norm_vec_kernel(float* __restrict__ x, const float* __restrict__ w, uint32_t dim, float eps) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float bc;
    float* p = x + (size_t)blockIdx.x * dim;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) xs[i] = p[i];
    __syncthreads();
    if (threadIdx.x == 0) bc = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq_sequential(xs, dim), (float)dim), eps)));
    __syncthreads();
    const float inv = bc;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) p[i] = __fmul_rn(__fmul_rn(xs[i], inv), w[i]);
}

__global__ void rope_kernel(float* __restrict__ x, const float* __restrict__ freqs, uint32_t half_dim,
                            uint32_t n_heads, float pos) {
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= half_dim * n_heads) return;
    const uint32_t i = idx % half_dim, h = idx / half_dim;
    const float theta = __fmul_rn(pos, freqs[i]);
    const float c = (float)cos((double)theta), s = (float)sin((double)theta);
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
    if (i < n) gate[i] = __fmul_rn(gelu_tanh(gate[i]), up[i]);
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
// Plain copy as a kernel: unlike a copy-engine transfer it chains with the next kernel by programmatic
// dependent launch, and its source may be page-locked host memory that the device can address.
__global__ void __launch_bounds__(256)
copy_f32_kernel(float* __restrict__ dst, const float* __restrict__ src, size_t n) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = src[i];
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
    pdl_launch_dependents();
    pdl_wait();
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

// Single-query attention over a KV cache in the arithmetic order of gqa_cached_attention /
// cached_attention (src/models/gemma3.zig:1062-1120, src/models/gpt2.zig:796-849), two launches.
//
// Scores: each dot product keeps 16 lane accumulators (lane l takes elements l, l+16, ...), adds
// the lanes in order 0..15, then any tail elements, then multiplies by 1/sqrt(head_dim). A CTA of
// 256 threads handles 16 positions x 16 lanes.
__global__ void __launch_bounds__(256)
attention_scores_kernel(const float* __restrict__ q, const float* __restrict__ kc,
                        float* __restrict__ scores, uint32_t n_head, uint32_t n_kv_head,
                        uint32_t head_dim, uint32_t kv_start, uint32_t kv_end) {
    __shared__ float part[16][17];
    const uint32_t h = blockIdx.y;
    const uint32_t kvh = h / (n_head / n_kv_head);
    const uint32_t kv_dim = n_kv_head * head_dim;
    const uint32_t kv_len = kv_end - kv_start;
    const uint32_t pp = threadIdx.x >> 4, l = threadIdx.x & 15;
    const uint32_t p = blockIdx.x * 16 + pp;
    const uint32_t dim16 = head_dim & ~15u;
    const float* qh = q + (size_t)h * head_dim;
    const float* kr = kc + (size_t)(kv_start + min(p, kv_len - 1)) * kv_dim + (size_t)kvh * head_dim;
    float acc = 0.0f;
    for (uint32_t d = l; d < dim16; d += 16) acc = __fadd_rn(acc, __fmul_rn(qh[d], kr[d]));
    part[pp][l] = acc;
    __syncthreads();
    if (l == 0 && p < kv_len) {
        float s = part[pp][0];
#pragma unroll
        for (int j = 1; j < 16; ++j) s = __fadd_rn(s, part[pp][j]);
        for (uint32_t d = dim16; d < head_dim; ++d) s = __fadd_rn(s, __fmul_rn(qh[d], kr[d]));
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)head_dim));
        scores[(size_t)h * kv_len + p] = __fmul_rn(s, scale);
    }
}

// Softmax and weighted sum of V, one CTA per query head: maximum, exp(s - max), the exponentials
// added one by one, weights = e * (1/sum), then out[d] += w[p] * v[p][d] for p in order.
// gpt2_tail: the GPT-2 softmax divides its last (n % 16) elements by the sum instead of multiplying
// by the reciprocal (src/models/gpt2.zig:721-730).
__global__ void __launch_bounds__(256)
attention_softmax_v_kernel(const float* __restrict__ scores, const float* __restrict__ vc,
                           float* __restrict__ out, uint32_t n_head, uint32_t n_kv_head,
                           uint32_t head_dim, uint32_t kv_start, uint32_t kv_end, int gpt2_tail) {
    extern __shared__ __align__(16) float w[];  // kv_len
    __shared__ float red[33];
    __shared__ float bc;
    const uint32_t h = blockIdx.x;
    const uint32_t kvh = h / (n_head / n_kv_head);
    const uint32_t kv_dim = n_kv_head * head_dim;
    const uint32_t kv_len = kv_end - kv_start;
    const float* sh = scores + (size_t)h * kv_len;
    float mx = -INFINITY;
    for (uint32_t p = threadIdx.x; p < kv_len; p += blockDim.x) {
        const float v = sh[p];
        w[p] = v;
        mx = fmaxf(mx, v);
    }
    mx = block_max(mx, red);
    for (uint32_t p = threadIdx.x; p < kv_len; p += blockDim.x) w[p] = exp_f32(__fsub_rn(w[p], mx));
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        uint32_t p = 0;
        for (; p + 8 <= kv_len; p += 8) {
            const float4 a = *reinterpret_cast<const float4*>(w + p);
            const float4 b = *reinterpret_cast<const float4*>(w + p + 4);
            s = __fadd_rn(s, a.x); s = __fadd_rn(s, a.y); s = __fadd_rn(s, a.z); s = __fadd_rn(s, a.w);
            s = __fadd_rn(s, b.x); s = __fadd_rn(s, b.y); s = __fadd_rn(s, b.z); s = __fadd_rn(s, b.w);
        }
        for (; p < kv_len; ++p) s = __fadd_rn(s, w[p]);
        bc = s;
    }
    __syncthreads();
    const float sum = bc;
    const float inv = __fdiv_rn(1.0f, sum);
    const uint32_t vec_end = gpt2_tail ? (kv_len & ~15u) : kv_len;
    for (uint32_t p = threadIdx.x; p < kv_len; p += blockDim.x)
        w[p] = p < vec_end ? __fmul_rn(w[p], inv) : __fdiv_rn(w[p], sum);
    __syncthreads();
    for (uint32_t d = threadIdx.x; d < head_dim; d += blockDim.x) {
        const float* vp = vc + (size_t)kv_start * kv_dim + (size_t)kvh * head_dim + d;
        float acc = 0.0f;
        uint32_t p = 0;
        for (; p + 8 <= kv_len; p += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = vp[(size_t)(p + j) * kv_dim];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = __fadd_rn(acc, __fmul_rn(w[p + j], v[j]));
        }
        for (; p < kv_len; ++p) acc = __fadd_rn(acc, __fmul_rn(w[p], vp[(size_t)p * kv_dim]));
        out[(size_t)h * head_dim + d] = acc;
    }
}

// ------------------------------------------------------------------------------------------
// Fused decode-step kernels for the engines. The sequence position lives in device memory
// (state[1]) so that one captured launch sequence serves every step; each kernel performs the
// same roundings in the same order as the separate kernels above, so results do not change.

// quantize_row_q8 (src/gguf/simd_dot.zig:17-43) of the 32 values held one per lane of a warp.
__device__ __forceinline__ void quantize_block_warp(float v, size_t blk, int lane, int8_t* __restrict__ q,
                                                    float* __restrict__ scale, int32_t* __restrict__ sum) {
    float amax = fabsf(v);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, s);
    float r = roundf(__fmul_rn(v, inv));
    r = fminf(127.0f, fmaxf(-127.0f, r));
    const int qi = (int)r;
    int acc = qi;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    q[blk * 32 + lane] = (int8_t)qi;
    if (lane == 0) {
        scale[blk] = s;
        sum[blk] = acc;
    }
}

// RES = false:  h = rms_norm(src, w1)                               -> quantised
// RES = true:   res += rms_norm(src, w1);  h = rms_norm(res, w2)     -> quantised
// (gemma3.zig:662-666, 725-737, 768-773: post-norm + residual, then the next block's pre-norm.)
// One CTA; dim is a multiple of 32.
// PER > 0: dim <= 256 * PER and every global operand is fetched into registers up front, so the
// kernel pays one memory round trip instead of one per phase; PER = 0 is the general form.
template <bool RES, int PER>
__global__ void __launch_bounds__(256)
norm_quant_kernel(const float* __restrict__ src, const float* __restrict__ w1, float* __restrict__ res,
                  const float* __restrict__ w2, uint32_t dim, float eps, int8_t* __restrict__ q,
                  float* __restrict__ scale, int32_t* __restrict__ sum, uint32_t src_stride) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float part[16];
    __shared__ float bc;
    constexpr int P = PER > 0 ? PER : 1;
    float rw1[P], rw2[P], rres[P];
    {   // one CTA per row (decode: one row; batched prefill: one per token)
        const size_t row = blockIdx.x;
        src += row * src_stride;
        if (RES) res += row * dim;
        q += row * dim;
        scale += row * (dim >> 5);
        sum += row * (dim >> 5);
    }
    pdl_launch_dependents();
    if (PER > 0) {
#pragma unroll
        for (int u = 0; u < P; ++u) {
            const uint32_t i = threadIdx.x + u * 256;
            rw1[u] = i < dim ? w1[i] : 0.0f;
            rw2[u] = (RES && i < dim) ? w2[i] : 0.0f;
        }
    } else {
        for (uint32_t i = threadIdx.x * 32; i < dim; i += blockDim.x * 32) {  // norm weights: one line per thread
            prefetch_l2_line(w1 + i);
            if (RES) prefetch_l2_line(w2 + i);
        }
    }
    pdl_wait();
    if (PER > 0) {
        float rs[P];
#pragma unroll
        for (int u = 0; u < P; ++u) {
            const uint32_t i = threadIdx.x + u * 256;
            rs[u] = i < dim ? src[i] : 0.0f;
            rres[u] = (RES && i < dim) ? res[i] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < P; ++u) {
            const uint32_t i = threadIdx.x + u * 256;
            if (i < dim) xs[i] = rs[u];
        }
    } else {
        for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) xs[i] = src[i];
    }
    __syncthreads();
    float ss = sumsq_lanes16(xs, dim, part, &bc);
    float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
    if (RES) {
        if (PER > 0) {
#pragma unroll
            for (int u = 0; u < P; ++u) {
                const uint32_t i = threadIdx.x + u * 256;
                if (i < dim) {
                    const float r = __fadd_rn(rres[u], __fmul_rn(__fmul_rn(xs[i], inv), rw1[u]));
                    res[i] = r;
                    xs[i] = r;
                }
            }
        } else {
            for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
                const float r = __fadd_rn(res[i], __fmul_rn(__fmul_rn(xs[i], inv), w1[i]));
                res[i] = r;
                xs[i] = r;
            }
        }
        __syncthreads();
        ss = sumsq_lanes16(xs, dim, part, &bc);
        inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
    }
    const int lane = threadIdx.x & 31;
    if (PER > 0) {
#pragma unroll
        for (int u = 0; u < P; ++u) {
            const uint32_t i = threadIdx.x + u * 256;
            if (i < dim)  // dim is a multiple of 32: whole warps
                quantize_block_warp(__fmul_rn(__fmul_rn(xs[i], inv), RES ? rw2[u] : rw1[u]), i >> 5, lane, q, scale, sum);
        }
    } else {
        const float* wq = RES ? w2 : w1;
        for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x)
            quantize_block_warp(__fmul_rn(__fmul_rn(xs[i], inv), wq[i]), i >> 5, lane, q, scale, sum);
    }
}

// Per-head work between the QKV projection and attention (gemma3.zig:689-716): q and k heads get
// rms_norm_in_place then RoPE at the current position; q stays in place, k and v go to row `pos` of
// the caches. Grid: n_head + 2 * n_kv_head CTAs (q heads, k heads, v heads).
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_kernel(float* __restrict__ qkv, const float* __restrict__ q_norm_w,
                       const float* __restrict__ k_norm_w, const float* __restrict__ freqs,
                       float* __restrict__ kc, float* __restrict__ vc, const uint32_t* __restrict__ state,
                       uint32_t n_head, uint32_t n_kv_head, uint32_t head_dim, float eps, uint32_t qkv_stride,
                       const uint32_t* __restrict__ row_pos, size_t cache_stride) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float bc;
    pdl_launch_dependents();
    pdl_wait();
    // blockIdx.y: a token of a batched prefill (position state[1] + row, one cache), or — row_pos given —
    // one of several independent sequences (own position, own cache cache_stride floats further)
    const uint32_t pos = row_pos ? row_pos[blockIdx.y] : state[1] + blockIdx.y;
    qkv += (size_t)blockIdx.y * qkv_stride;
    if (row_pos) {
        kc += (size_t)blockIdx.y * cache_stride;
        vc += (size_t)blockIdx.y * cache_stride;
    }
    const uint32_t b = blockIdx.x, kv_dim = n_kv_head * head_dim;
    if (b >= n_head + n_kv_head) {  // v head: copy
        const uint32_t hv = b - n_head - n_kv_head;
        const float* src = qkv + (size_t)(n_head + n_kv_head + hv) * head_dim;
        float* dst = vc + (size_t)pos * kv_dim + (size_t)hv * head_dim;
        for (uint32_t i = threadIdx.x; i < head_dim; i += blockDim.x) dst[i] = src[i];
        return;
    }
    const bool is_k = b >= n_head;
    float* p = qkv + (size_t)b * head_dim;
    const float* w = is_k ? k_norm_w : q_norm_w;
    for (uint32_t i = threadIdx.x; i < head_dim; i += blockDim.x) xs[i] = p[i];
    __syncthreads();
    if (threadIdx.x == 0)
        bc = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq_sequential(xs, head_dim), (float)head_dim), eps)));
    __syncthreads();
    const float inv = bc;
    float* dst = is_k ? kc + (size_t)pos * kv_dim + (size_t)(b - n_head) * head_dim : p;
    const float fpos = (float)pos;
    for (uint32_t i = threadIdx.x; i < head_dim / 2; i += blockDim.x) {
        const float x0 = __fmul_rn(__fmul_rn(xs[2 * i], inv), w[2 * i]);
        const float x1 = __fmul_rn(__fmul_rn(xs[2 * i + 1], inv), w[2 * i + 1]);
        const float theta = __fmul_rn(fpos, freqs[i]);
        const float c = (float)cos((double)theta), s = (float)sin((double)theta);
        dst[2 * i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        dst[2 * i + 1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
}

// g = gelu(gate) * up, quantised (gemma3.zig:750-765 followed by the row quantiser of the down
// projection). One warp per 32-block.
__global__ void __launch_bounds__(256)
gelu_mul_quant_kernel(const float* __restrict__ gate, const float* __restrict__ up, uint32_t n_blocks,
                      int8_t* __restrict__ q, float* __restrict__ scale, int32_t* __restrict__ sum,
                      uint32_t blocks_per_row, uint32_t in_stride) {
    const uint32_t blk = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    pdl_launch_dependents();
    pdl_wait();
    if (blk >= n_blocks) return;
    // rows of gate / up are in_stride floats apart; the quantised output is dense
    const size_t i = (size_t)(blk / blocks_per_row) * in_stride + (size_t)(blk % blocks_per_row) * 32 + lane;
    quantize_block_warp(__fmul_rn(gelu_tanh(gate[i]), up[i]), blk, lane, q, scale, sum);
}

// The window a decode step attends to: positions [kv_start, pos]; `window` = 0 means all of them.
__device__ __forceinline__ void step_window(const uint32_t* state, uint32_t window, uint32_t* kv_start,
                                            uint32_t* kv_len, uint32_t token = 0, const uint32_t* row_pos = nullptr) {
    const uint32_t end = (row_pos ? row_pos[token] : state[1] + token) + 1;
    const uint32_t len = (window && end > window) ? window : end;
    *kv_start = end - len;
    *kv_len = len;
}

// Optional per-head RMSNorm + RoPE of q and of this step's k inside the scores kernel (decode only): the
// raw projection outputs come in, every CTA normalises and rotates the query head it needs (and the new
// key, if it scores the current position or stores the cache row) with the arithmetic of
// qk_norm_rope_kv_kernel, so that kernel's launch disappears from the step.
struct QkNormRope {
    const float* q_norm_w;  // nullptr: q and k_new are used as they are
    const float* k_norm_w;
    const float* freqs;
    float eps;
};

// attention_scores_kernel with the window taken from the device-side position. The grid covers the
// largest possible window; CTAs past the current one leave at once.
template <bool LOOP>  // LOOP: a CTA walks over several key tiles (many rows in flight); else one tile per CTA
__global__ void __launch_bounds__(256)
attention_scores_step_kernel(const float* __restrict__ q, float* __restrict__ kc, float* __restrict__ vc,
                             const float* __restrict__ k_new, const float* __restrict__ v_new,
                             float* __restrict__ scores, uint32_t n_head, uint32_t n_kv_head,
                             uint32_t head_dim, const uint32_t* __restrict__ state, uint32_t window,
                             uint32_t q_stride, uint32_t scores_stride, const uint32_t* __restrict__ row_pos,
                             size_t cache_stride, QkNormRope nr) {
    __shared__ float part[16][17];
    __shared__ float inv2[2];
    extern __shared__ __align__(16) float qk[];  // nr: normalised + rotated q head, then k head
    pdl_launch_dependents();
    pdl_wait();
    uint32_t kv_start, kv_len;
    step_window(state, window, &kv_start, &kv_len, blockIdx.z, row_pos);  // blockIdx.z: token or sequence
    q += (size_t)blockIdx.z * q_stride;
    if (k_new) {
        k_new += (size_t)blockIdx.z * q_stride;
        v_new += (size_t)blockIdx.z * q_stride;
    }
    scores += (size_t)blockIdx.z * scores_stride;
    if (row_pos) {
        kc += (size_t)blockIdx.z * cache_stride;
        vc += (size_t)blockIdx.z * cache_stride;
    }
    const uint32_t h = blockIdx.y;
    const uint32_t group = n_head / n_kv_head;
    const uint32_t kvh = h / group;
    const uint32_t kv_dim = n_kv_head * head_dim;
    // k_new / v_new: this step's key and value rows are not in the caches yet. The first CTA of each kv
    // head stores them (gpt2.zig:812-816); the score of the current position reads the new key directly.
    const uint32_t pos = kv_start + kv_len - 1;
    // A CTA takes the 16-key tiles blockIdx.x, blockIdx.x + gridDim.x, ... of the window.
    const bool writer = k_new != nullptr && blockIdx.x == 0 && h % group == 0;
    const bool in_window = blockIdx.x * 16 < kv_len;
    if (!in_window && !writer) return;
    const float* qh = q + (size_t)h * head_dim;
    const float* knew = k_new ? k_new + (size_t)kvh * head_dim : nullptr;
    if (nr.q_norm_w != nullptr) {
        // the new key is needed by the writer and by the CTA whose tiles include the last position
        const bool need_k = writer || (in_window && (LOOP ? ((kv_len - 1) / 16) % gridDim.x == blockIdx.x
                                                           : blockIdx.x * 16 + 16 > kv_len - 1));
        float* qn = qk;
        float* kn = qk + head_dim;
        for (uint32_t i = threadIdx.x; i < head_dim; i += blockDim.x) {
            qn[i] = qh[i];
            if (need_k) kn[i] = knew[i];
        }
        __syncthreads();
        // squares added one by one in index order (rms_norm_in_place), q by thread 0, k by thread 32
        if (threadIdx.x == 0)
            inv2[0] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq_sequential(qn, head_dim), (float)head_dim), nr.eps)));
        if (threadIdx.x == 32 && need_k)
            inv2[1] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq_sequential(kn, head_dim), (float)head_dim), nr.eps)));
        __syncthreads();
        const float fpos = (float)pos;
        for (uint32_t i = threadIdx.x; i < head_dim; i += blockDim.x) {  // i < head_dim / 2: q pair; above: k pair
            const bool is_k = i >= head_dim / 2;
            if (is_k && !need_k) continue;
            const uint32_t j = is_k ? i - head_dim / 2 : i;
            float* v = is_k ? kn : qn;
            const float* wn = is_k ? nr.k_norm_w : nr.q_norm_w;
            const float inv = inv2[is_k ? 1 : 0];
            const float x0 = __fmul_rn(__fmul_rn(v[2 * j], inv), wn[2 * j]);
            const float x1 = __fmul_rn(__fmul_rn(v[2 * j + 1], inv), wn[2 * j + 1]);
            const float theta = __fmul_rn(fpos, nr.freqs[j]);
            const float c = (float)cos((double)theta), sn = (float)sin((double)theta);
            v[2 * j] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
            v[2 * j + 1] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
        }
        __syncthreads();
        qh = qn;
        knew = kn;
    }
    if (writer) {
        const float* vsrc = v_new + (size_t)kvh * head_dim;
        for (uint32_t i = threadIdx.x; i < head_dim; i += blockDim.x) {
            kc[(size_t)pos * kv_dim + (size_t)kvh * head_dim + i] = knew[i];
            vc[(size_t)pos * kv_dim + (size_t)kvh * head_dim + i] = vsrc[i];
        }
    }
    if (!in_window) return;
    const uint32_t pp = threadIdx.x >> 4, l = threadIdx.x & 15;
    const uint32_t dim16 = head_dim & ~15u;
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)head_dim));
    for (uint32_t p0 = blockIdx.x * 16; p0 < kv_len; p0 += gridDim.x * 16) {
        const uint32_t p = p0 + pp;
        const uint32_t pc = min(p, kv_len - 1);
        const float* kr = (k_new != nullptr && pc == kv_len - 1)
                              ? knew
                              : kc + (size_t)(kv_start + pc) * kv_dim + (size_t)kvh * head_dim;
        float acc = 0.0f;
        for (uint32_t d = l; d < dim16; d += 16) acc = __fadd_rn(acc, __fmul_rn(qh[d], kr[d]));
        part[pp][l] = acc;
        __syncthreads();
        if (l == 0 && p < kv_len) {
            float s = part[pp][0];
#pragma unroll
            for (int j = 1; j < 16; ++j) s = __fadd_rn(s, part[pp][j]);
            for (uint32_t d = dim16; d < head_dim; ++d) s = __fadd_rn(s, __fmul_rn(qh[d], kr[d]));
            scores[(size_t)h * kv_len + p] = __fmul_rn(s, scale);
        }
        if (!LOOP) break;
        __syncthreads();  // `part` is rewritten by the next tile
    }
}

// Softmax and weighted sum of V for one decode step, device-side window. Same arithmetic as
// attention_softmax_v_kernel (exponentials added one by one, out[d] += w[p] * v[p][d] for p in order), laid
// out for long windows: a CTA owns 64 output dimensions of one head (grid = heads x head_dim / 64) and
// streams V through shared memory in tiles of 64 positions — all 256 threads fetch the next tile
// (coalesced 256-byte rows, 16 loads in flight each) while 64 threads run the add chain of the current
// one, so the chain, not the memory latency, sets the time. QUANT additionally quantises the head's output
// in 32-blocks for the output projection; the f32 output is optional.
constexpr int kAttnTile = 64;  // positions per V tile
constexpr int kAttnDims = 64;  // output dimensions per CTA

template <bool QUANT>
__global__ void __launch_bounds__(256)
attention_softmax_v_step_kernel(const float* __restrict__ scores, const float* __restrict__ vc,
                                float* __restrict__ out, int8_t* __restrict__ oq, float* __restrict__ oscale,
                                int32_t* __restrict__ osum, uint32_t n_head, uint32_t n_kv_head,
                                uint32_t head_dim, const uint32_t* __restrict__ state, uint32_t window,
                                int gpt2_tail, uint32_t scores_stride, const uint32_t* __restrict__ row_pos,
                                size_t cache_stride) {
    extern __shared__ __align__(16) float w[];  // max window length
    __shared__ float vt[kAttnTile][kAttnDims];
    __shared__ float red[33];
    __shared__ float bc;
    pdl_launch_dependents();
    pdl_wait();
    uint32_t kv_start, kv_len;
    step_window(state, window, &kv_start, &kv_len, blockIdx.z, row_pos);  // blockIdx.z: token or sequence
    scores += (size_t)blockIdx.z * scores_stride;
    if (row_pos) vc += (size_t)blockIdx.z * cache_stride;
    const size_t out_row = (size_t)blockIdx.z * n_head * head_dim;
    const uint32_t h = blockIdx.x;
    const uint32_t kvh = h / (n_head / n_kv_head);
    const uint32_t kv_dim = n_kv_head * head_dim;
    const uint32_t d0 = blockIdx.y * kAttnDims;
    const uint32_t pg = threadIdx.x >> 6, dl = threadIdx.x & 63;
    const bool d_ok = d0 + dl < head_dim;
    const float* vbase = vc + (size_t)kv_start * kv_dim + (size_t)kvh * head_dim + d0 + dl;

    // rows pg*16 .. pg*16+15 of a tile, one element per row and thread
    float vreg[16];
    auto fetch = [&](uint32_t p0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t p = p0 + pg * 16 + i;
            vreg[i] = (d_ok && p < kv_len) ? vbase[(size_t)p * kv_dim] : 0.0f;
        }
    };
    fetch(0);  // in flight during the softmax below

    const float* sh = scores + (size_t)h * kv_len;
    float mx = -INFINITY;
    for (uint32_t p = threadIdx.x; p < kv_len; p += blockDim.x) {
        const float v = sh[p];
        w[p] = v;
        mx = fmaxf(mx, v);
    }
    mx = block_max(mx, red);
    for (uint32_t p = threadIdx.x; p < kv_len; p += blockDim.x) w[p] = exp_f32(__fsub_rn(w[p], mx));
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        uint32_t p = 0;
        for (; p + 8 <= kv_len; p += 8) {
            const float4 a = *reinterpret_cast<const float4*>(w + p);
            const float4 b = *reinterpret_cast<const float4*>(w + p + 4);
            s = __fadd_rn(s, a.x); s = __fadd_rn(s, a.y); s = __fadd_rn(s, a.z); s = __fadd_rn(s, a.w);
            s = __fadd_rn(s, b.x); s = __fadd_rn(s, b.y); s = __fadd_rn(s, b.z); s = __fadd_rn(s, b.w);
        }
        for (; p < kv_len; ++p) s = __fadd_rn(s, w[p]);
        bc = s;
    }
    __syncthreads();
    const float sum = bc;
    const float inv = __fdiv_rn(1.0f, sum);
    const uint32_t vec_end = gpt2_tail ? (kv_len & ~15u) : kv_len;
    for (uint32_t p = threadIdx.x; p < kv_len; p += blockDim.x)
        w[p] = p < vec_end ? __fmul_rn(w[p], inv) : __fdiv_rn(w[p], sum);

    float acc = 0.0f;
    for (uint32_t p0 = 0; p0 < kv_len; p0 += kAttnTile) {
        __syncthreads();  // the previous tile has been consumed (first pass: the weights are complete)
#pragma unroll
        for (int i = 0; i < 16; ++i) vt[pg * 16 + i][dl] = vreg[i];
        __syncthreads();
        if (p0 + kAttnTile < kv_len) fetch(p0 + kAttnTile);
        if (pg == 0) {
            const uint32_t n = min((uint32_t)kAttnTile, kv_len - p0);
            uint32_t i = 0;
            for (; i + 8 <= n; i += 8) {
                float v[8], ww[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    v[j] = vt[i + j][dl];
                    ww[j] = w[p0 + i + j];
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) acc = __fadd_rn(acc, __fmul_rn(ww[j], v[j]));
            }
            for (; i < n; ++i) acc = __fadd_rn(acc, __fmul_rn(w[p0 + i], vt[i][dl]));
        }
    }
    if (pg == 0) {  // two whole warps: 32-blocks of the output line up with warps
        const size_t o = out_row + (size_t)h * head_dim + d0 + dl;
        if (d_ok && out) out[o] = acc;
        if (QUANT && d0 + (dl & ~31u) < head_dim) quantize_block_warp(acc, o >> 5, threadIdx.x & 31, oq, oscale, osum);
    }
}

// GPT-2 embedding and cache write at the device-side position (gpt2.zig:449-453, 812-816).
// blockIdx.y: token of a batched prefill (ids in `tokens`); decoding uses the token in state[0].
__global__ void gpt2_embed_step_kernel(float* __restrict__ x, const float* __restrict__ wte,
                                       const float* __restrict__ wpe, const uint32_t* __restrict__ state,
                                       const int32_t* __restrict__ tokens, uint32_t embed) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    const uint32_t tok = tokens ? (uint32_t)tokens[r] : state[0];
    if (i < embed) x[(size_t)r * embed + i] = wte[(size_t)tok * embed + i] + wpe[(size_t)(state[1] + r) * embed + i];
}
// k / v rows of the batch (in_stride floats apart) -> cache rows state[1] + r
__global__ void write_kv_step_kernel(const float* __restrict__ k, const float* __restrict__ v,
                                     float* __restrict__ kc, float* __restrict__ vc,
                                     const uint32_t* __restrict__ state, uint32_t kv_dim, uint32_t in_stride) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x, r = blockIdx.y;
    const uint32_t pos = state[1] + r;
    if (i < kv_dim) {
        kc[(size_t)pos * kv_dim + i] = k[(size_t)r * in_stride + i];
        vc[(size_t)pos * kv_dim + i] = v[(size_t)r * in_stride + i];
    }
}

inline unsigned grid1d(size_t n, unsigned threads) { return (unsigned)((n + threads - 1) / threads); }

}  // namespace

// ---- launchers used by the engines (declared in zq_internal.h) ----------------------------

int launch_norm_quant(const float* src, const float* w1, float* res, const float* w2, uint32_t dim, float eps,
                      int8_t* q, float* scale, int32_t* sum, uint32_t rows, uint32_t src_stride, cudaStream_t st) {
    if (dim == 0 || dim % 32 || dim > 48 * 1024 / 4) return ZQ_ERR_LIMIT;
    if (rows == 0) return ZQ_OK;
    const size_t smem = dim * sizeof(float);
    cudaError_t e;
    if (dim <= 256 * 5) {
        e = res ? launch_pdl(norm_quant_kernel<true, 5>, dim3(rows), dim3(256), smem, st, src, w1, res, w2, dim, eps, q,
                             scale, sum, src_stride)
                : launch_pdl(norm_quant_kernel<false, 5>, dim3(rows), dim3(256), smem, st, src, w1, nullptr, nullptr,
                             dim, eps, q, scale, sum, src_stride);
    } else {
        e = res ? launch_pdl(norm_quant_kernel<true, 0>, dim3(rows), dim3(256), smem, st, src, w1, res, w2, dim, eps, q,
                             scale, sum, src_stride)
                : launch_pdl(norm_quant_kernel<false, 0>, dim3(rows), dim3(256), smem, st, src, w1, nullptr, nullptr,
                             dim, eps, q, scale, sum, src_stride);
    }
    ZQ_CUDA(e);
    return ZQ_OK;
}

int launch_qk_norm_rope_kv(float* qkv, const float* q_norm_w, const float* k_norm_w, const float* freqs,
                           float* kc, float* vc, const uint32_t* state, uint32_t n_head, uint32_t n_kv_head,
                           uint32_t head_dim, float eps, uint32_t rows, uint32_t qkv_stride, const uint32_t* row_pos,
                           size_t cache_stride, cudaStream_t st) {
    if (head_dim % 2 || head_dim > 48 * 1024 / 4) return ZQ_ERR_LIMIT;
    if (rows == 0) return ZQ_OK;
    ZQ_CUDA(launch_pdl(qk_norm_rope_kv_kernel, dim3(n_head + 2 * n_kv_head, rows), dim3(128), head_dim * sizeof(float),
                       st, qkv, q_norm_w, k_norm_w, freqs, kc, vc, state, n_head, n_kv_head, head_dim, eps,
                       qkv_stride, row_pos, cache_stride));
    return ZQ_OK;
}

int launch_gelu_mul_quant(const float* gate, const float* up, uint32_t n, int8_t* q, float* scale,
                          int32_t* sum, uint32_t rows, uint32_t in_stride, cudaStream_t st) {
    if (n % 32) return ZQ_ERR_BAD_ARG;
    if (rows == 0) return ZQ_OK;
    const size_t total = (size_t)rows * n;
    ZQ_CUDA(launch_pdl(gelu_mul_quant_kernel, dim3(grid1d(total, 256)), dim3(256), 0, st, gate, up,
                       (uint32_t)(total / 32), q, scale, sum, n / 32, in_stride));
    return ZQ_OK;
}

int launch_attention_step(const float* q, float* kc, float* vc, const float* k_new, const float* v_new,
                          float* out, int8_t* oq, float* oscale, int32_t* osum, float* scores, uint32_t n_head,
                          uint32_t n_kv_head, uint32_t head_dim, const uint32_t* state, uint32_t window,
                          uint32_t max_len, int flags, uint32_t rows, uint32_t q_stride, const uint32_t* row_pos,
                          size_t cache_stride, const float* q_norm_w, const float* k_norm_w, const float* freqs,
                          float norm_eps, cudaStream_t st) {
    if (max_len == 0 || max_len > 180 * 1024 / 4) return ZQ_ERR_LIMIT;
    if (oq && head_dim % 32) return ZQ_ERR_BAD_ARG;
    if (rows == 0) return ZQ_OK;
    // new keys are taken from the caller's rows only when no row needs another row's key: one row, or
    // independent sequences
    if (rows > 65535u || (rows > 1 && k_new && !row_pos)) return ZQ_ERR_BAD_ARG;
    if (q_norm_w && (!k_new || !k_norm_w || !freqs || head_dim % 2)) return ZQ_ERR_BAD_ARG;
    const QkNormRope nr{q_norm_w, k_norm_w, freqs, norm_eps};
    const size_t smem_scores = q_norm_w ? 2 * (size_t)head_dim * sizeof(float) : 0;
    if (smem_scores > 40 * 1024) return ZQ_ERR_LIMIT;
    const size_t smem = (size_t)max_len * sizeof(float);
    const int tail = (flags & ZQ_ATTN_GPT2_SOFTMAX) ? 1 : 0;
    const uint32_t scores_stride = n_head * max_len;
    // One CTA per 16-key tile when few rows are in flight (a decode step: parallelism comes from the tiles);
    // with many rows (batched sequences, prefill chunks) a CTA walks over several tiles, which saves
    // launching thousands of CTAs that find their tile outside the row's window and repeats the per-CTA
    // q / k preparation less often.
    uint32_t tiles_x = (max_len + 15) / 16;
    const bool loop = rows >= 16 && tiles_x > 8;
    if (loop) tiles_x = 8;
    ZQ_CUDA(launch_pdl(loop ? attention_scores_step_kernel<true> : attention_scores_step_kernel<false>,
                       dim3(tiles_x, n_head, rows), dim3(256), smem_scores, st, q, kc, vc, k_new, v_new, scores, n_head,
                       n_kv_head, head_dim, state, window, q_stride, scores_stride, row_pos, cache_stride, nr));
    const dim3 grid(n_head, (head_dim + kAttnDims - 1) / kAttnDims, rows);
    if (oq) {
        auto kern = attention_softmax_v_step_kernel<true>;
        if (smem > 24 * 1024)  // the kernel also holds a 16 KB static tile
            ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        ZQ_CUDA(launch_pdl(kern, grid, dim3(256), smem, st, static_cast<const float*>(scores),
                           static_cast<const float*>(vc), out, oq, oscale, osum, n_head, n_kv_head, head_dim, state,
                           window, tail, scores_stride, row_pos, cache_stride));
    } else {
        auto kern = attention_softmax_v_step_kernel<false>;
        if (smem > 24 * 1024)
            ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        ZQ_CUDA(launch_pdl(kern, grid, dim3(256), smem, st, static_cast<const float*>(scores),
                           static_cast<const float*>(vc), out, nullptr, nullptr, nullptr, n_head, n_kv_head, head_dim,
                           state, window, tail, scores_stride, row_pos, cache_stride));
    }
    return ZQ_OK;
}

int launch_gpt2_embed_step(float* x, const float* wte, const float* wpe, const uint32_t* state,
                           const int32_t* tokens, uint32_t embed, uint32_t rows, cudaStream_t st) {
    if (rows == 0) return ZQ_OK;
    gpt2_embed_step_kernel<<<dim3(grid1d(embed, 256), rows), 256, 0, st>>>(x, wte, wpe, state, tokens, embed);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int launch_write_kv_step(const float* k, const float* v, float* kc, float* vc, const uint32_t* state,
                         uint32_t kv_dim, uint32_t rows, uint32_t in_stride, cudaStream_t st) {
    if (rows == 0) return ZQ_OK;
    write_kv_step_kernel<<<dim3(grid1d(kv_dim, 256), rows), 256, 0, st>>>(k, v, kc, vc, state, kv_dim, in_stride);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

}  // namespace zq

using namespace zq;

extern "C" {

int zq_rms_norm(const float* d_x, const float* d_w, float* d_out, uint32_t dim, uint32_t rows,
                float eps, zq_stream stream) {
    if (!d_x || !d_w || !d_out || dim == 0) return ZQ_ERR_BAD_ARG;
    if (rows == 0) return ZQ_OK;
    if (dim > 48 * 1024 / 4) return ZQ_ERR_LIMIT;
    rms_norm_kernel<<<rows, 256, dim * sizeof(float), as_stream(stream)>>>(d_x, d_w, d_out, dim, eps, 0);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_rms_norm_residual(const float* d_x, const float* d_w, float* d_residual, uint32_t dim,
                         uint32_t rows, float eps, zq_stream stream) {
    if (!d_x || !d_w || !d_residual || dim == 0) return ZQ_ERR_BAD_ARG;
    if (rows == 0) return ZQ_OK;
    if (dim > 48 * 1024 / 4) return ZQ_ERR_LIMIT;
    rms_norm_kernel<<<rows, 256, dim * sizeof(float), as_stream(stream)>>>(d_x, d_w, d_residual, dim, eps, 1);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_rms_norm_in_place(float* d_x, const float* d_w, uint32_t dim, uint32_t n_vec, float eps,
                         zq_stream stream) {
    if (!d_x || !d_w || dim == 0) return ZQ_ERR_BAD_ARG;
    if (n_vec == 0) return ZQ_OK;
    if (dim > 48 * 1024 / 4) return ZQ_ERR_LIMIT;
    rms_norm_vec_kernel<<<n_vec, 64, dim * sizeof(float), as_stream(stream)>>>(d_x, d_w, dim, eps);
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
                        float* d_out, float* d_scores, uint32_t n_head, uint32_t n_kv_head,
                        uint32_t head_dim, uint32_t kv_start, uint32_t kv_end, int flags,
                        zq_stream stream) {
    if (!d_q || !d_k_cache || !d_v_cache || !d_out || !d_scores) return ZQ_ERR_BAD_ARG;
    if (n_head == 0 || n_kv_head == 0 || head_dim == 0 || n_head % n_kv_head) return ZQ_ERR_BAD_ARG;
    if (kv_end <= kv_start) return ZQ_ERR_BAD_ARG;
    const uint32_t kv_len = kv_end - kv_start;
    if (kv_len > 48 * 1024 / 4) return ZQ_ERR_LIMIT;
    cudaStream_t st = as_stream(stream);
    attention_scores_kernel<<<dim3((kv_len + 15) / 16, n_head), 256, 0, st>>>(
        d_q, d_k_cache, d_scores, n_head, n_kv_head, head_dim, kv_start, kv_end);
    ZQ_LAUNCH_CHECK();
    attention_softmax_v_kernel<<<n_head, 256, kv_len * sizeof(float), st>>>(
        d_scores, d_v_cache, d_out, n_head, n_kv_head, head_dim, kv_start, kv_end,
        (flags & ZQ_ATTN_GPT2_SOFTMAX) ? 1 : 0);
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
    ZQ_CUDA(launch_pdl(layer_norm_kernel, dim3(rows), dim3(256), 0, as_stream(stream), d_out, d_x, d_gamma, d_beta, cols,
                       eps));
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

int zq_copy_f32(float* d_dst, const float* src, size_t n, zq_stream stream) {
    if (!d_dst || !src) return ZQ_ERR_BAD_ARG;
    if (n == 0) return ZQ_OK;
    const unsigned grid = grid1d(n, 256) < 64u ? grid1d(n, 256) : 64u;
    ZQ_CUDA(launch_pdl(copy_f32_kernel, dim3(grid), dim3(256), 0, as_stream(stream), d_dst, src, n));
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
