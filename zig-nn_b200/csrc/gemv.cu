// Decode GEMV kernels: quantised weight rows streamed from HBM with 128-bit loads, dequantised
// in registers, reduced with warp shuffles. Two activation treatments:
//   f32  — f32 activations times weights dequantised on the fly (zig-nn src/gguf/dequant.zig:133-309)
//   q8   — the activation quantiser lives here (quantize_row_q8); the exact int8 GEMV is in
//          gemv_q8.cu.
#include <stdlib.h>

#include "zq_internal.h"

namespace zq {
namespace {

constexpr int kThreads = 128;  // 4 warps per CTA
constexpr int kWarps = kThreads / 32;
constexpr int XPAD = 36;   // floats per activation block in shared memory: 32 + 4 so that lanes
                           // reading different blocks with 128-bit loads hit different banks

// ---- packed f32x2 arithmetic (sm_100) --------------------------------------------------

__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("{\n\t"
        ".reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "mov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t"
        "}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}

__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    float2 d;
    asm("{\n\t"
        ".reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t"
        "}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

// A 4-bit field sitting at bit p (p <= 19) of `q`, OR-ed under the exponent of 2^(23-p), reads
// as the float 2^(23-p) + n; subtracting 2^(23-p) + off leaves n - off exactly.
template <int P>
__device__ __forceinline__ float nib_as_float(uint32_t q) {
    return __uint_as_float((q & (0xFu << P)) | ((150u - P) << 23));
}
template <int P>
__device__ __forceinline__ constexpr float nib_bias(float off) {
    return -((float)(1u << (23 - P)) + off);
}

// Dot of the eight 4-bit weights of one 32-bit quant word with their activations.
// Word w of a block holds elements 4w..4w+3 (low nibbles) and 4w+16..4w+19 (high nibbles).
// OFF = 8 for q4_0 (n - 8), 0 for q4_1 (n).
template <int OFF>
__device__ __forceinline__ void q4_word_dot(uint32_t q, float4 xlo, float4 xhi, float2& acc) {
    const uint32_t s = q >> 12;
    float2 a01 = make_float2(nib_as_float<0>(q), nib_as_float<8>(q));
    float2 a23 = make_float2(nib_as_float<16>(q), nib_as_float<12>(s));
    float2 b01 = make_float2(nib_as_float<4>(q), nib_as_float<12>(q));
    float2 b23 = make_float2(nib_as_float<8>(s), nib_as_float<16>(s));
    a01 = fadd2(a01, make_float2(nib_bias<0>(OFF), nib_bias<8>(OFF)));
    a23 = fadd2(a23, make_float2(nib_bias<16>(OFF), nib_bias<12>(OFF)));
    b01 = fadd2(b01, make_float2(nib_bias<4>(OFF), nib_bias<12>(OFF)));
    b23 = fadd2(b23, make_float2(nib_bias<8>(OFF), nib_bias<16>(OFF)));
    acc = ffma2(a01, make_float2(xlo.x, xlo.y), acc);
    acc = ffma2(a23, make_float2(xlo.z, xlo.w), acc);
    acc = ffma2(b01, make_float2(xhi.x, xhi.y), acc);
    acc = ffma2(b23, make_float2(xhi.z, xhi.w), acc);
}

// Dot of the four int8 weights of one quant word with x[0..3]. Each byte, flipped to unsigned,
// is dropped under the exponent of 2^23: the float reads 2^23 + (b + 128).
__device__ __forceinline__ void q8_word_dot(uint32_t q, float4 x, float2& acc) {
    const uint32_t u = q ^ 0x80808080u;
    float2 a01 = make_float2(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7440)),
                             __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7441)));
    float2 a23 = make_float2(__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7442)),
                             __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7443)));
    const float2 bias = make_float2(-8388736.0f, -8388736.0f);
    a01 = fadd2(a01, bias);
    a23 = fadd2(a23, bias);
    acc = ffma2(a01, make_float2(x.x, x.y), acc);
    acc = ffma2(a23, make_float2(x.z, x.w), acc);
}

// 0.5*v*(1+tanh(0.7978845608*(v+0.044715*v*v*v))) — src/models/gpt2.zig:690-697. Every operation
// is a separate f32 rounding in the CPU code's order; tanh is evaluated in double and rounded once.
__device__ __forceinline__ float gelu_tanh(float v) {
    const float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v);
    const float inner = __fmul_rn(0.7978845608f, __fadd_rn(v, cube));
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, (float)tanh((double)inner)));
}

struct EpilogueArgs {
    const float* bias;
    const float* mul;
    const float* residual;
    int gelu;
};

__device__ __forceinline__ float apply_epilogue(float v, const EpilogueArgs& ep, size_t j) {
    if (ep.bias) v = __fadd_rn(v, ep.bias[j]);
    if (ep.gelu) v = gelu_tanh(v);
    if (ep.mul) v = __fmul_rn(v, ep.mul[j]);
    if (ep.residual) v = __fadd_rn(ep.residual[j], v);
    return v;
}

// ---- f32-activation GEMV, one activation row ---------------------------------------------
//
// A warp owns 32/G row groups of R consecutive rows; the G lanes of a group walk the blocks of
// those rows (lane g takes blocks g, g+G, ...). Per step a lane issues R independent 128-bit
// quant loads (2R for q8_0) and reuses one block of activations, read from shared memory, for
// all R rows.
template <int TYPE, int G, int R>
__global__ void __launch_bounds__(kThreads)
gemv_f32_kernel(const uint8_t* __restrict__ qs, const void* __restrict__ sc,
                const float* __restrict__ x, float* __restrict__ y, uint32_t N, uint32_t nb,
                uint32_t scp, EpilogueArgs ep) {
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;               // nb * XPAD
    float* xsum = smem + (size_t)nb * XPAD;  // nb (q4_1 only)
    const int tid = threadIdx.x;
    for (uint32_t i = tid; i < nb * 32; i += kThreads) xs[(i >> 5) * XPAD + (i & 31)] = x[i];
    __syncthreads();
    if (TYPE == ZQ_TYPE_Q4_1) {
        for (uint32_t b = tid; b < nb; b += kThreads) {
            float s = 0.0f;
            for (int j = 0; j < 32; ++j) s += xs[b * XPAD + j];
            xsum[b] = s;
        }
        __syncthreads();
    }

    constexpr int GROUPS = 32 / G;
    constexpr int ROWS_W = GROUPS * R;
    constexpr int QB = TYPE == ZQ_TYPE_Q8_0 ? 32 : 16;
    const int lane = tid & 31, warp = tid >> 5;
    const int g = lane % G, grp = lane / G;
    const uint32_t rows_per_cta = kWarps * ROWS_W;

    for (uint64_t tile = blockIdx.x; tile * rows_per_cta < N; tile += gridDim.x) {
        const uint32_t row0 = (uint32_t)(tile * rows_per_cta) + warp * ROWS_W + grp * R;
        float sum[R];
        const uint8_t* qrow[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            sum[r] = 0.0f;
            const uint32_t row = min(row0 + r, N - 1);  // clamp: out-of-range rows are never stored
            qrow[r] = qs + (size_t)row * ((nb + 3u) & ~3u) * QB;
        }
        for (uint32_t b = g; b < nb; b += G) {
            uint4 q[R][QB / 16];
            float d[R], mn[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                // the block's words are interleaved with its three quad neighbours: gather them
                const uint8_t* p = qrow[r];
                q[r][0] = make_uint4(__ldg(reinterpret_cast<const uint32_t*>(p + qs_word_offset(QB, b, 0))),
                                     __ldg(reinterpret_cast<const uint32_t*>(p + qs_word_offset(QB, b, 1))),
                                     __ldg(reinterpret_cast<const uint32_t*>(p + qs_word_offset(QB, b, 2))),
                                     __ldg(reinterpret_cast<const uint32_t*>(p + qs_word_offset(QB, b, 3))));
                if (QB == 32)
                    q[r][QB / 16 - 1] =
                        make_uint4(__ldg(reinterpret_cast<const uint32_t*>(p + qs_word_offset(QB, b, 4))),
                                   __ldg(reinterpret_cast<const uint32_t*>(p + qs_word_offset(QB, b, 5))),
                                   __ldg(reinterpret_cast<const uint32_t*>(p + qs_word_offset(QB, b, 6))),
                                   __ldg(reinterpret_cast<const uint32_t*>(p + qs_word_offset(QB, b, 7))));
                const uint32_t row = min(row0 + r, N - 1);
                if (TYPE == ZQ_TYPE_Q4_1) {
                    const __half2 dm = __ldg(reinterpret_cast<const __half2*>(sc) + (size_t)row * scp + b);
                    d[r] = __low2float(dm);
                    mn[r] = __high2float(dm);
                } else {
                    d[r] = __half2float(__ldg(reinterpret_cast<const __half*>(sc) + (size_t)row * scp + b));
                    mn[r] = 0.0f;
                }
            }
            const float4* xb = reinterpret_cast<const float4*>(xs + b * XPAD);
            float4 xv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) xv[i] = xb[i];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float2 acc = make_float2(0.0f, 0.0f);
                if (TYPE == ZQ_TYPE_Q8_0) {
                    const uint32_t w[8] = {q[r][0].x, q[r][0].y, q[r][0].z, q[r][0].w,
                                           q[r][QB / 16 - 1].x, q[r][QB / 16 - 1].y,
                                           q[r][QB / 16 - 1].z, q[r][QB / 16 - 1].w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) q8_word_dot(w[i], xv[i], acc);
                    sum[r] += (acc.x + acc.y) * d[r];
                } else {
                    const uint32_t w[4] = {q[r][0].x, q[r][0].y, q[r][0].z, q[r][0].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        q4_word_dot<TYPE == ZQ_TYPE_Q4_0 ? 8 : 0>(w[i], xv[i], xv[4 + i], acc);
                    if (TYPE == ZQ_TYPE_Q4_0)
                        sum[r] += (acc.x + acc.y) * d[r];
                    else
                        sum[r] += (acc.x + acc.y) * d[r] + xsum[b] * mn[r];
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int off = G / 2; off > 0; off >>= 1)
                sum[r] += __shfl_xor_sync(0xFFFFFFFFu, sum[r], off);
        }
        if (g == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r)
                if (row0 + r < N) y[row0 + r] = apply_epilogue(sum[r], ep, row0 + r);
        }
    }
}

// ---- quantize_row_q8 (src/gguf/simd_dot.zig:25-64): one warp per 32-element block ---------------

__global__ void quantize_q8_kernel(const float* __restrict__ x, int8_t* __restrict__ q,
                                   float* __restrict__ scale, int32_t* __restrict__ sum,
                                   size_t n_blocks) {
    const size_t blk = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (blk >= n_blocks) return;
    const float v = x[blk * 32 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, s);
    float r = roundf(__fmul_rn(v, inv));  // half away from zero, as std.math.round
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

// ---- f32 weight times one row (GPT-2 vocabulary head), one warp per output row -------------

__global__ void __launch_bounds__(256)
matvec_f32_kernel(const float* __restrict__ w, const float* __restrict__ x, float* __restrict__ y,
                  uint32_t N, uint32_t K, const float* __restrict__ ln_gamma, const float* __restrict__ ln_beta,
                  float ln_eps) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float red[10];
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t warps = blockDim.x >> 5;
    if (ln_gamma != nullptr) {
        // LayerNorm of the row in the prologue (two-pass mean / variance, gpt2.zig:541-596)
        float sum = 0.0f;
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) sum += x[i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
        if (lane == 0) red[warp] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (uint32_t i = 0; i < warps; ++i) t += red[i];
            red[8] = t / (float)K;
        }
        __syncthreads();
        const float mean = red[8];
        float var = 0.0f;
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) {
            const float d = x[i] - mean;
            var = fmaf(d, d, var);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) var += __shfl_xor_sync(0xFFFFFFFFu, var, off);
        __syncthreads();
        if (lane == 0) red[warp] = var;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.0f;
            for (uint32_t i = 0; i < warps; ++i) t += red[i];
            red[9] = 1.0f / sqrtf(t / (float)K + ln_eps);
        }
        __syncthreads();
        const float inv_std = red[9];
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x)
            xs[i] = __fadd_rn(__fmul_rn(__fmul_rn(x[i] - mean, inv_std), ln_gamma[i]), ln_beta[i]);
    } else {
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) xs[i] = x[i];
    }
    __syncthreads();
    const bool vec = (K % 4 == 0);
    for (uint64_t row = (uint64_t)blockIdx.x * warps + warp; row < N; row += (uint64_t)gridDim.x * warps) {
        const float* wr = w + row * K;
        float acc = 0.0f;
        if (vec) {
            const float4* w4 = reinterpret_cast<const float4*>(wr);
            const float4* x4 = reinterpret_cast<const float4*>(xs);
            const uint32_t n4 = K / 4;
            uint32_t i = lane;
            for (; i + 96 < n4; i += 128) {  // four independent 128-bit loads in flight per lane
                float4 a[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) a[u] = __ldg(w4 + i + 32 * u);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float4 b = x4[i + 32 * u];
                    acc = fmaf(a[u].x, b.x, acc);
                    acc = fmaf(a[u].y, b.y, acc);
                    acc = fmaf(a[u].z, b.z, acc);
                    acc = fmaf(a[u].w, b.w, acc);
                }
            }
            for (; i < n4; i += 32) {
                const float4 a = __ldg(w4 + i), b = x4[i];
                acc = fmaf(a.x, b.x, acc);
                acc = fmaf(a.y, b.y, acc);
                acc = fmaf(a.z, b.z, acc);
                acc = fmaf(a.w, b.w, acc);
            }
        } else {
            for (uint32_t i = lane; i < K; i += 32) acc = fmaf(__ldg(wr + i), xs[i], acc);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
        if (lane == 0) y[row] = acc;
    }
}

// ---- argmax, first maximum wins (src/models/gpt2.zig:980-990) --------------------------------

__device__ __forceinline__ void argmax_merge(float& v, uint32_t& i, float ov, uint32_t oi) {
    if (ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
    }
}

__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, uint32_t n, int32_t* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ uint32_t si[32];
    float v = -INFINITY;
    uint32_t idx = 0xFFFFFFFFu;
    // a NaN never compares greater, as in the CPU loop; index 0 is the fallback
    auto take = [&](float c, uint32_t i) {
        if (c > v || (c == v && i < idx)) {
            v = c;
            idx = i;
        }
    };
    uint32_t done = 0;
    if ((reinterpret_cast<uintptr_t>(logits) & 15u) == 0) {
        // four independent 128-bit loads in flight per thread: one CTA reads the row at L2 speed
        const float4* l4 = reinterpret_cast<const float4*>(logits);
        const uint32_t n4 = n / 4, stride = blockDim.x;
        uint32_t i = threadIdx.x;
        for (; i + 3 * stride < n4; i += 4 * stride) {
            float4 c[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) c[u] = __ldg(l4 + i + u * stride);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t b = (i + u * stride) * 4;
                take(c[u].x, b); take(c[u].y, b + 1); take(c[u].z, b + 2); take(c[u].w, b + 3);
            }
        }
        for (; i < n4; i += stride) {
            const float4 c = __ldg(l4 + i);
            take(c.x, i * 4); take(c.y, i * 4 + 1); take(c.z, i * 4 + 2); take(c.w, i * 4 + 3);
        }
        done = n4 * 4;
    }
    for (uint32_t i = done + threadIdx.x; i < n; i += blockDim.x) take(logits[i], i);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, v, off);
        const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, off);
        argmax_merge(v, idx, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) {
        sv[warp] = v;
        si[warp] = idx;
    }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        v = lane < nw ? sv[lane] : -INFINITY;
        idx = lane < nw ? si[lane] : 0xFFFFFFFFu;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, v, off);
            const uint32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, off);
            argmax_merge(v, idx, ov, oi);
        }
        if (lane == 0) out[0] = (idx == 0xFFFFFFFFu) ? 0 : (int32_t)idx;
    }
}

// ---- launch helpers ----------------------------------------------------------------------

// Lanes per row group: the power of two (4..32) that wastes the fewest lane-steps, larger first.
int pick_group(uint32_t nb, int g_max) {
    int best = 4;
    double best_eff = -1.0;
    for (int g = g_max; g >= 4; g >>= 1) {
        const uint32_t steps = (nb + g - 1) / g;
        const double eff = (double)nb / ((double)steps * g);
        if (eff > best_eff + 1e-9) {
            best_eff = eff;
            best = g;
        }
    }
    return best;
}

EpilogueArgs make_ep(const zq_epilogue* ep, size_t row_offset_elems) {
    EpilogueArgs a{nullptr, nullptr, nullptr, 0};
    if (ep) {
        a.bias = ep->d_bias;
        a.gelu = ep->gelu;
        a.mul = ep->d_mul ? ep->d_mul + row_offset_elems : nullptr;
        a.residual = ep->d_residual ? ep->d_residual + row_offset_elems : nullptr;
    }
    return a;
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
    if (bytes > 48 * 1024) {
        if (bytes > 227 * 1024) return ZQ_ERR_LIMIT;
        ZQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    }
    return ZQ_OK;
}

template <int TYPE, int G, int R>
int launch_f32_one(const zq_weight* w, const float* x, float* y, EpilogueArgs ep, cudaStream_t st) {
    const size_t smem = ((size_t)w->nb * XPAD + w->nb) * sizeof(float);
    int rc = set_smem(gemv_f32_kernel<TYPE, G, R>, smem);
    if (rc != ZQ_OK) return rc;
    const uint32_t rows_per_cta = kWarps * (32 / G) * R;
    const uint64_t tiles = ((uint64_t)w->out_dim + rows_per_cta - 1) / rows_per_cta;
    const uint64_t cap = (uint64_t)sm_count() * 8;
    const unsigned grid = (unsigned)(tiles < cap ? tiles : cap);
    gemv_f32_kernel<TYPE, G, R><<<grid, kThreads, smem, st>>>(w->qs, w->sc, x, y, w->out_dim, w->nb, w->scp, ep);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

template <int TYPE, int G>
int launch_f32_r(const zq_weight* w, const float* x, float* y, EpilogueArgs ep, cudaStream_t st) {
    // Fewer rows per lane when there are not enough rows to give every SM a few warps.
    const uint64_t warp_tiles4 = (uint64_t)w->out_dim / ((32 / G) * 4);
    if (warp_tiles4 >= (uint64_t)sm_count() * kWarps * 2) return launch_f32_one<TYPE, G, 4>(w, x, y, ep, st);
    const uint64_t warp_tiles2 = (uint64_t)w->out_dim / ((32 / G) * 2);
    if (warp_tiles2 >= (uint64_t)sm_count() * kWarps) return launch_f32_one<TYPE, G, 2>(w, x, y, ep, st);
    return launch_f32_one<TYPE, G, 1>(w, x, y, ep, st);
}

template <int TYPE>
int launch_f32_g(const zq_weight* w, const float* x, float* y, EpilogueArgs ep, cudaStream_t st) {
    switch (pick_group(w->nb, 32)) {
        case 32: return launch_f32_r<TYPE, 32>(w, x, y, ep, st);
        case 16: return launch_f32_r<TYPE, 16>(w, x, y, ep, st);
        case 8: return launch_f32_r<TYPE, 8>(w, x, y, ep, st);
        default: return launch_f32_r<TYPE, 4>(w, x, y, ep, st);
    }
}

}  // namespace

int launch_gemv_f32(const zq_weight* w, const float* x, float* y, uint32_t m_rows,
                    const zq_epilogue* ep, cudaStream_t st) {
    for (uint32_t m = 0; m < m_rows; ++m) {
        const size_t xo = (size_t)m * w->in_dim, yo = (size_t)m * w->out_dim;
        EpilogueArgs a = make_ep(ep, yo);
        int rc;
        switch (w->type) {
            case ZQ_TYPE_Q4_0: rc = launch_f32_g<ZQ_TYPE_Q4_0>(w, x + xo, y + yo, a, st); break;
            case ZQ_TYPE_Q4_1: rc = launch_f32_g<ZQ_TYPE_Q4_1>(w, x + xo, y + yo, a, st); break;
            case ZQ_TYPE_Q8_0: rc = launch_f32_g<ZQ_TYPE_Q8_0>(w, x + xo, y + yo, a, st); break;
            default: return ZQ_ERR_UNSUPPORTED;
        }
        if (rc != ZQ_OK) return rc;
    }
    return ZQ_OK;
}

int launch_quantize_rows_q8(const float* x, uint32_t m_rows, uint32_t in_dim, int8_t* q,
                            float* scale, int32_t* sum, cudaStream_t st) {
    const size_t n_blocks = (size_t)m_rows * (in_dim / 32);
    if (n_blocks == 0) return ZQ_OK;
    const unsigned threads = 256;
    const size_t grid = (n_blocks * 32 + threads - 1) / threads;
    if (grid > 0x7FFFFFFFull) return ZQ_ERR_LIMIT;
    quantize_q8_kernel<<<(unsigned)grid, threads, 0, st>>>(x, q, scale, sum, n_blocks);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int launch_matvec_ln_f32(const float* w, const float* x, float* y, uint32_t out_dim, uint32_t in_dim,
                         const float* ln_gamma, const float* ln_beta, float ln_eps, cudaStream_t st) {
    const size_t smem = (size_t)in_dim * sizeof(float);
    int rc = set_smem(matvec_f32_kernel, smem);
    if (rc != ZQ_OK) return rc;
    const uint64_t tiles = ((uint64_t)out_dim + 7) / 8;
    const uint64_t cap = (uint64_t)sm_count() * 8;
    ZQ_CUDA(launch_pdl(matvec_f32_kernel, dim3((unsigned)(tiles < cap ? tiles : cap)), dim3(256), smem, st, w, x, y,
                       out_dim, in_dim, ln_gamma, ln_beta, ln_eps));
    return ZQ_OK;
}

}  // namespace zq

using namespace zq;

extern "C" {

size_t zq_matmul_workspace_bytes(const zq_weight* w, uint32_t m_rows, int act_mode) {
    if (!w) return 0;
    if (act_mode == ZQ_ACT_Q8) {
        // int8 activations, then per-block f32 scales and int32 sums, each 256-byte aligned
        const size_t q = ((size_t)m_rows * w->in_dim + 255) & ~(size_t)255;
        const size_t s = ((size_t)m_rows * w->nb * 4 + 255) & ~(size_t)255;
        return q + 2 * s;
    }
    if ((act_mode == ZQ_ACT_F32 && m_rows >= kGemmMinRows) || (act_mode == ZQ_ACT_F16 && m_rows > 0)) {
        return gemm_tc_workspace_bytes(w, m_rows);
    }
    if (act_mode == ZQ_ACT_F32 && m_rows >= kStreamMinRowsF32 && gemm_stream_takes(w, m_rows))
        return gemm_tc_workspace_bytes(w, m_rows);
    return 0;
}

int zq_quantize_rows_q8(const float* d_x, uint32_t m_rows, uint32_t in_dim, int8_t* d_q,
                        float* d_scale, int32_t* d_sum, zq_stream stream) {
    if (!d_x || !d_q || !d_scale || !d_sum || in_dim == 0 || in_dim % 32) return ZQ_ERR_BAD_ARG;
    return launch_quantize_rows_q8(d_x, m_rows, in_dim, d_q, d_scale, d_sum, as_stream(stream));
}

int zq_matmul(const zq_weight* w, const float* d_x, float* d_y, uint32_t m_rows, int act_mode,
              const zq_epilogue* epilogue, void* d_workspace, size_t workspace_bytes,
              zq_stream stream) {
    if (!w) return ZQ_ERR_BAD_ARG;
    if (m_rows == 0) return ZQ_OK;
    if (!d_x || !d_y) return ZQ_ERR_BAD_ARG;
    if (check_weight_device(w) != ZQ_OK) return ZQ_ERR_BAD_ARG;  // the weight lives on another device
    cudaStream_t st = as_stream(stream);
    if (act_mode == ZQ_ACT_F32) {
        if (((uintptr_t)d_x & 15) != 0) return launch_gemv_f32(w, d_x, d_y, m_rows, epilogue, st);
        // many rows: the tensor-core GEMM, which needs the workspace for its fp16 activation image. A call
        // without one is refused rather than served by 16-row passes that are several times slower.
        if (m_rows >= kGemmMinRows) {
            if (!d_workspace || ((uintptr_t)d_workspace & 255) != 0 ||
                workspace_bytes < zq_matmul_workspace_bytes(w, m_rows, act_mode))
                return ZQ_ERR_BAD_ARG;
            return launch_gemm_tc(w, d_x, d_y, m_rows, epilogue, d_workspace, st);
        }
        // 17-48 rows of a large matrix: the weight-streaming tensor-core form when the caller brought the workspace
        // that zq_matmul_workspace_bytes asks for (two or three 16-row passes of the decode kernel otherwise)
        if (m_rows >= kStreamMinRowsF32 && gemm_stream_takes(w, m_rows) && d_workspace &&
            ((uintptr_t)d_workspace & 255) == 0 && workspace_bytes >= gemm_tc_workspace_bytes(w, m_rows))
            return launch_gemm_tc(w, d_x, d_y, m_rows, epilogue, d_workspace, st);
        // passes of up to 16 activation rows over the weights
        int rc = launch_gemv_mma_passes_f32(w, d_x, d_y, m_rows, epilogue, st);
        if (rc == ZQ_ERR_LIMIT)  // activation image too large for shared memory: row-at-a-time kernel
            rc = launch_gemv_f32(w, d_x, d_y, m_rows, epilogue, st);
        return rc;
    }
    if (act_mode == ZQ_ACT_F16) {  // the tensor-core GEMM whatever the row count
        if (((uintptr_t)d_x & 3) != 0) return ZQ_ERR_BAD_ARG;
        if (!d_workspace || ((uintptr_t)d_workspace & 255) ||
            workspace_bytes < zq_matmul_workspace_bytes(w, m_rows, act_mode))
            return ZQ_ERR_BAD_ARG;
        return launch_gemm_tc(w, d_x, d_y, m_rows, epilogue, d_workspace, st);
    }
    if (act_mode == ZQ_ACT_Q8) {
        if (w->in_dim > 16384) return ZQ_ERR_LIMIT;
        const size_t need = zq_matmul_workspace_bytes(w, m_rows, act_mode);
        if (!d_workspace || workspace_bytes < need || ((uintptr_t)d_workspace & 255)) return ZQ_ERR_BAD_ARG;
        const size_t qbytes = ((size_t)m_rows * w->in_dim + 255) & ~(size_t)255;
        const size_t sbytes = ((size_t)m_rows * w->nb * 4 + 255) & ~(size_t)255;
        int8_t* q = static_cast<int8_t*>(d_workspace);
        float* sc = reinterpret_cast<float*>(static_cast<char*>(d_workspace) + qbytes);
        int32_t* sm = reinterpret_cast<int32_t*>(static_cast<char*>(d_workspace) + qbytes + sbytes);
        int rc = launch_quantize_rows_q8(d_x, m_rows, w->in_dim, q, sc, sm, st);
        if (rc != ZQ_OK) return rc;
        // From two rows on, the exact int8 GEMM (weights read once for up to 64 rows) beats a GEMV per row:
        // measured 1.1-1.6x at 2-4 rows on the small matrices and 1.5-2.3x on the 170-320 MB vocabulary
        // head (4 rows: 71-89 us against 130-206 us). Both give the same bits.
        const uint32_t q8_gemm_min = 2;
        if (m_rows >= q8_gemm_min) return launch_gemm_q8(w, q, sc, sm, d_y, m_rows, epilogue, st);
        return launch_gemv_q8(w, q, sc, sm, d_y, m_rows, epilogue, st);
    }
    return ZQ_ERR_BAD_ARG;
}

int zq_matmul_gather(const zq_weight* w, const float* d_x, const zq_epilogue* epilogue,
                     float* const* h_y_peers_odd, float* const* h_y_peers_even, uint32_t* const* h_flag_peers,
                     uint32_t world, uint32_t rank, uint32_t row_offset, uint32_t* d_sync, zq_stream stream) {
    if (!w || !d_x || !h_y_peers_odd || !h_y_peers_even || !h_flag_peers || !d_sync) return ZQ_ERR_BAD_ARG;
    return launch_gemv_gather_f32(w, d_x, epilogue, h_y_peers_odd, h_y_peers_even, h_flag_peers, world, rank,
                                  row_offset, d_sync, as_stream(stream));
}

int zq_matmul_gather_tagged(const zq_weight* w, const float* d_x, const zq_epilogue* epilogue,
                            unsigned long long* const* h_inbox_peers_odd, unsigned long long* const* h_inbox_peers_even,
                            float* d_y_odd, float* d_y_even, uint32_t world, uint32_t rank, uint32_t* d_sync,
                            zq_stream stream) {
    if (!w || !d_x || !h_inbox_peers_odd || !h_inbox_peers_even || !d_y_odd || !d_y_even || !d_sync) return ZQ_ERR_BAD_ARG;
    return launch_gemv_gather_tagged_f32(w, d_x, epilogue, h_inbox_peers_odd, h_inbox_peers_even, d_y_odd, d_y_even, world,
                                         rank, d_sync, as_stream(stream));
}

int zq_matmul_argmax(const zq_weight* w, const float* d_x, const zq_epilogue* epilogue, float* d_y_local,
                     unsigned long long* const* h_inbox_peers_odd, unsigned long long* const* h_inbox_peers_even,
                     int32_t* d_index, float* d_value, uint32_t world, uint32_t rank, uint32_t* d_sync, zq_stream stream) {
    if (!w || !d_x || !d_index || !d_sync) return ZQ_ERR_BAD_ARG;
    return launch_gemv_argmax_f32(w, d_x, epilogue, d_y_local, h_inbox_peers_odd, h_inbox_peers_even, d_index, d_value,
                                  world, rank, d_sync, as_stream(stream));
}

int zq_matvec_f32(const float* d_w, const float* d_x, float* d_y, uint32_t out_dim, uint32_t in_dim,
                  zq_stream stream) {
    if (!d_w || !d_x || !d_y || out_dim == 0 || in_dim == 0) return ZQ_ERR_BAD_ARG;
    return launch_matvec_ln_f32(d_w, d_x, d_y, out_dim, in_dim, nullptr, nullptr, 0.0f, as_stream(stream));
}

int zq_argmax(const float* d_logits, uint32_t n, int32_t* d_index, zq_stream stream) {
    if (!d_logits || !d_index || n == 0) return ZQ_ERR_BAD_ARG;
    argmax_kernel<<<1, 1024, 0, as_stream(stream)>>>(d_logits, n, d_index);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

}  // extern "C"
