// The f32 forward kernels that zig-nn's CUDA backend loads BY NAME from an embedded module image
// (src/backend/cuda_kernels.cu:1-18 -> cuModuleLoadData at src/backend/cuda_context.zig:200-216) and
// launches through src/cuda_ops.zig with fixed geometry. This translation unit is compiled to an sm_100a
// image (cubin and fatbin, see build.py) that exports the same `extern "C"` names with the same parameter
// lists, so the existing dispatchers work unchanged on B200:
//
//   kernel                      parameters                                         geometry cuda_ops.zig uses
//   add_broadcast, mul_broadcast (out, a, b, a_total, b_total)                      1-D, 256 threads (:36-63)
//   gelu_kernel                  (out, x, n)                                        1-D (:65-86)
//   scale_kernel                 (out, x, s, n)                                     1-D (:236-260)
//   softmax_kernel               (data, rows, cols)                                 grid = rows, block =
//   softmax_out_kernel           (out, x, rows, cols)                                 next_pow2(min(cols, 1024)),
//   layernorm_kernel             (out, x, gamma, beta, rows, cols, eps)               dynamic shared = block * 4
//   layernorm_fwd_kernel         (out, x_norm, inv_stds, x, gamma, beta, rows, cols, eps)   (:88-146, 518-575)
//   reduction_sum_rows_kernel    (out, x, rows, cols)                               same row geometry (:996-1021)
//   reduction_sum_cols_kernel    (out, x, rows, cols)                               1-D over cols (:1023-1047)
//   reduction_sum_1d_kernel      (out, x, n)                                        ONE block (:1049-1069)
//   transpose_2d_kernel          (out, x, rows, cols)                               1-D (:147-170)
//   modulate_adaln_kernel        (out, norm, scale, beta_data, B, S, D)             1-D (:173-205)
//   gather_kernel                (out, table, indices, num_indices, embed_dim)      1-D (:207-234)
//
// The kernels accept any block size the dispatchers can produce (1 .. 1024 threads, also below one warp) and do
// not depend on the dynamic shared memory they are given: row reductions run as warp shuffles plus one
// 32-entry static exchange. Arithmetic follows the reference kernels (kernels/forward_*.cu,
// kernels/reduction_kernels.cu): max-subtracted expf softmax times 1/sum; two-pass mean / variance with
// rsqrtf(var + eps); tanh GELU with tanhf.
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

struct Sum {
    static __device__ __forceinline__ float id() { return 0.0f; }
    static __device__ __forceinline__ float op(float a, float b) { return a + b; }
};
struct Max {
    static __device__ __forceinline__ float id() { return -3.0e38f; }
    static __device__ __forceinline__ float op(float a, float b) { return fmaxf(a, b); }
};

// Reduction over the whole block; every thread receives the result. Works for any block size: the lanes of a
// partial warp (block sizes below 32 or not a multiple of it) shuffle under the mask of the lanes that exist.
template <typename R>
__device__ __forceinline__ float block_reduce(float v) {
    __shared__ float warp_part[32];
    __shared__ float result;
    const unsigned tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const unsigned n_threads = blockDim.x;
    const unsigned first = warp << 5;
    const unsigned lanes = n_threads - first < 32u ? n_threads - first : 32u;  // lanes this warp really has
    const unsigned mask = lanes == 32u ? 0xFFFFFFFFu : ((1u << lanes) - 1u);
#pragma unroll
    for (unsigned off = 16; off > 0; off >>= 1) {
        const float other = __shfl_down_sync(mask, v, off);
        if (lane + off < lanes) v = R::op(v, other);
    }
    __syncthreads();  // warp_part / result of an earlier call have been read by everyone
    if (lane == 0) warp_part[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const unsigned n_warps = (n_threads + 31u) >> 5;
        float t = lane < n_warps ? warp_part[lane] : R::id();
        const unsigned m0 = lanes == 32u ? 0xFFFFFFFFu : ((1u << lanes) - 1u);
#pragma unroll
        for (unsigned off = 16; off > 0; off >>= 1) {
            const float other = __shfl_down_sync(m0, t, off);
            if (lane + off < lanes) t = R::op(t, other);
        }
        if (lane == 0) result = t;
    }
    __syncthreads();
    return result;
}

__device__ __forceinline__ void softmax_row(float* dst, const float* src, int cols) {
    const int tid = threadIdx.x, nt = blockDim.x;
    float mx = Max::id();
    for (int j = tid; j < cols; j += nt) mx = fmaxf(mx, src[j]);
    mx = block_reduce<Max>(mx);
    float sum = 0.0f;
    for (int j = tid; j < cols; j += nt) {
        const float e = expf(src[j] - mx);
        dst[j] = e;
        sum += e;
    }
    sum = block_reduce<Sum>(sum);
    const float inv = 1.0f / sum;
    for (int j = tid; j < cols; j += nt) dst[j] *= inv;
}

// Returns (mean, 1 / sqrt(var + eps)) of one row: two passes, as the reference kernels do.
__device__ __forceinline__ float2 row_moments(const float* row, int cols, float eps) {
    const int tid = threadIdx.x, nt = blockDim.x;
    float s = 0.0f;
    for (int j = tid; j < cols; j += nt) s += row[j];
    const float mean = block_reduce<Sum>(s) / (float)cols;
    float v = 0.0f;
    for (int j = tid; j < cols; j += nt) {
        const float d = row[j] - mean;
        v += d * d;
    }
    const float var = block_reduce<Sum>(v) / (float)cols;
    return make_float2(mean, rsqrtf(var + eps));
}

}  // namespace

extern "C" {

__global__ void add_broadcast(float* out, const float* a, const float* b, int a_total, int b_total) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < a_total) out[i] = a[i] + b[i % b_total];
}

__global__ void mul_broadcast(float* out, const float* a, const float* b, int a_total, int b_total) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < a_total) out[i] = a[i] * b[i % b_total];
}

__global__ void gelu_kernel(float* out, const float* x, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = x[i];
    out[i] = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}

__global__ void scale_kernel(float* out, const float* x, float s, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = x[i] * s;
}

__global__ void softmax_kernel(float* data, int rows, int cols) {
    if ((int)blockIdx.x >= rows) return;
    float* row = data + (size_t)blockIdx.x * cols;
    softmax_row(row, row, cols);
}

__global__ void softmax_out_kernel(float* out, const float* x, int rows, int cols) {
    if ((int)blockIdx.x >= rows) return;
    softmax_row(out + (size_t)blockIdx.x * cols, x + (size_t)blockIdx.x * cols, cols);
}

__global__ void layernorm_kernel(float* out, const float* x, const float* gamma, const float* beta, int rows,
                                 int cols, float eps) {
    if ((int)blockIdx.x >= rows) return;
    const float* row = x + (size_t)blockIdx.x * cols;
    float* o = out + (size_t)blockIdx.x * cols;
    const float2 m = row_moments(row, cols, eps);
    for (int j = threadIdx.x; j < cols; j += blockDim.x) o[j] = (row[j] - m.x) * m.y * gamma[j] + beta[j];
}

// The training-side form: also stores the normalised row and 1/std for the backward pass.
__global__ void layernorm_fwd_kernel(float* out, float* x_norm, float* inv_stds, const float* x, const float* gamma,
                                     const float* beta, int rows, int cols, float eps) {
    if ((int)blockIdx.x >= rows) return;
    const float* row = x + (size_t)blockIdx.x * cols;
    float* o = out + (size_t)blockIdx.x * cols;
    float* xn = x_norm + (size_t)blockIdx.x * cols;
    const float2 m = row_moments(row, cols, eps);
    if (threadIdx.x == 0) inv_stds[blockIdx.x] = m.y;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) {
        const float n = (row[j] - m.x) * m.y;
        xn[j] = n;
        o[j] = n * gamma[j] + beta[j];
    }
}

__global__ void reduction_sum_rows_kernel(float* out, const float* x, int rows, int cols) {
    if ((int)blockIdx.x >= rows) return;
    const float* row = x + (size_t)blockIdx.x * cols;
    float s = 0.0f;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) s += row[j];
    s = block_reduce<Sum>(s);
    if (threadIdx.x == 0) out[blockIdx.x] = s;
}

__global__ void reduction_sum_cols_kernel(float* out, const float* x, int rows, int cols) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= cols) return;
    float s = 0.0f;
    for (int i = 0; i < rows; ++i) s += x[(size_t)i * cols + j];
    out[j] = s;
}

// out[0] += sum(x[0..n)). The dispatcher launches ONE block of next_pow2(min(n, 1024)) threads
// (cuda_ops.zig:1049-1069); the block strides over all n elements, so vectors longer than the block are summed
// completely (the reference kernel reads one element per thread). Like the reference it adds into out[0].
__global__ void reduction_sum_1d_kernel(float* out, const float* x, int n) {
    float s = 0.0f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (size_t)n; i += (size_t)gridDim.x * blockDim.x)
        s += x[i];
    s = block_reduce<Sum>(s);
    if (threadIdx.x == 0) atomicAdd(out, s);
}

__global__ void transpose_2d_kernel(float* out, const float* x, int rows, int cols) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * cols) return;
    const int r = i / cols, c = i - r * cols;
    out[(size_t)c * rows + r] = x[i];
}

// out[b][s][d] = norm[b][s][d] * scale[b][d] + beta_data[b][d]
__global__ void modulate_adaln_kernel(float* out, const float* norm, const float* scale, const float* beta_data, int B,
                                      int S, int D) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B * S * D) return;
    const int b = i / (S * D), d = i % D;
    out[i] = norm[i] * scale[b * D + d] + beta_data[b * D + d];
}

__global__ void gather_kernel(float* out, const float* table, const int* indices, int num_indices, int embed_dim) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_indices * embed_dim) return;
    const int r = i / embed_dim, d = i - r * embed_dim;
    out[i] = table[(size_t)indices[r] * embed_dim + d];
}

}  // extern "C"
