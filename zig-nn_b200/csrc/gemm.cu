// f32 rows -> fp16 rows with a power-of-two scale per row: the operand preparation of the transposed
// quantised product (gemm_trans.cu: grad_out rows; nn_training_kernels.metal:1149-1242 is the reference's
// statement of that product).
#include "gemm_common.cuh"

namespace zq {
namespace {

// x16[m][k] = fp16(x[m][k] * 2^-e_m), post[m] = 2^e_m, with e_m chosen so that the row's largest magnitude
// lands just under 2^14 (full fp16 precision for the large elements, no overflow). A row whose largest
// magnitude is below 2^-100 (vanishing gradients) is not scaled: 2^(13 - e) would overflow, and the row's
// products are zero at f32 accuracy anyway.
__global__ void __launch_bounds__(256)
convert_rows_f16_kernel(const float* __restrict__ x, __half* __restrict__ x16, float* __restrict__ post,
                        uint32_t K) {
    __shared__ float red[8];
    __shared__ float s_pre;
    const float* row = x + (size_t)blockIdx.x * K;
    __half* out = x16 + (size_t)blockIdx.x * K;
    float amax = 0.0f;
    for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = red[0];
        for (int w = 1; w < 8; ++w) a = fmaxf(a, red[w]);
        s_pre = ldexpf(1.0f, -row_scale_exponent(a));
        post[blockIdx.x] = ldexpf(1.0f, row_scale_exponent(a));
    }
    __syncthreads();
    const float pre = s_pre;
    for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) out[i] = __float2half_rn(row[i] * pre);
}

}  // namespace

int launch_convert_rows_f16(const float* x, __half* x16, float* post, uint32_t m_rows, uint32_t in_dim,
                            cudaStream_t st) {
    convert_rows_f16_kernel<<<m_rows, 256, 0, st>>>(x, x16, post, in_dim);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

}  // namespace zq
