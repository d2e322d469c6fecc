// Device functions shared by the fused decode-step kernels (ops.cu) and the GEMV that runs a norm as
// the last CTA's tail (gemv_q8.cu). Both reproduce the CPU loops' rounding order exactly.
#pragma once
#include "zq_internal.h"

namespace zq {
namespace step_common {

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

}  // namespace step_common
}  // namespace zq
