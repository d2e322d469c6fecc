// Batched quantised matmul for many activation rows (prefill, batched decode): y[M][N] = x[M][K] . W^T.
//
// The reference dequantises a weight row and multiplies it with f32 activations
// (zig-nn src/gguf/dequant.zig:133-309, src/models/gpt2.zig:623-671). With hundreds of activation
// rows the work is a GEMM, so the weights are dequantised once per CTA tile into fp16 shared-memory
// tiles — value = (n - 8) * d, n * d + m or q * d, rounded once to fp16 (relative error <= 2^-12) — the
// activations are pre-converted to fp16 with a per-row power-of-two scale (<= 2^-12 again), and the
// products are accumulated in f32 on the tensor cores. Outputs agree with the f32 CPU path to about
// 3e-4 relative L2, inside the 1e-3 bar of the path; the decode kernels (<= 16 rows) stay at 1e-7.
//
// Tile: 128 weight rows x 128 activation rows per CTA, K in steps of 128 (one quad of blocks per row),
// three stages. Shared tiles are [rows][64 halves] (128 bytes per row) with the 16-byte chunks of a row
// XOR-swizzled by (row & 7), the layout ldmatrix reads without bank conflicts.
#include "gemm_common.cuh"

namespace zq {
namespace {

using namespace gemm_common;

constexpr int BN = 128;      // weight rows per CTA (MMA M dimension)
constexpr int BM = 128;      // activation rows per CTA (MMA N dimension)
constexpr int BK = 128;      // K per stage: 4 blocks = one quad
constexpr int STAGES = 3;
constexpr int THREADS = 256;
constexpr uint32_t STAGE_BYTES = 4 * HALF_TILE;      // A lo/hi K-halves, B lo/hi K-halves

struct GemmEpilogue {
    const float* bias;
    const float* mul;
    const float* residual;
    int gelu;
};

__device__ __forceinline__ float gelu_tanh(float v) {
    const float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v);
    const float inner = __fmul_rn(0.7978845608f, __fadd_rn(v, cube));
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, (float)tanh((double)inner)));
}

// ---- activations: f32 rows -> fp16 rows with a power-of-two scale per row -----------------------
// x16[m][k] = fp16(x[m][k] * 2^-e_m), post[m] = 2^e_m, with e_m chosen so that the row's largest
// magnitude lands just under 2^14 (full fp16 precision for the large elements, no overflow).
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
        int e = 0;
        if (a > 0.0f && a < INFINITY) e = ilogbf(a) - 13;
        s_pre = ldexpf(1.0f, -e);
        post[blockIdx.x] = ldexpf(1.0f, e);
    }
    __syncthreads();
    const float pre = s_pre;
    for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) out[i] = __float2half_rn(row[i] * pre);
}

template <int TYPE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_f16_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ sc, const __half* __restrict__ x16,
                const float* __restrict__ post, float* __restrict__ y, uint32_t N, uint32_t K, uint32_t M,
                uint32_t nbp, uint32_t scp, GemmEpilogue ep) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QB = Q8 ? 32 : 16;
    constexpr uint32_t SB = Q41 ? 4 : 2;
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t smem32 = (uint32_t)__cvta_generic_to_shared(smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const uint32_t nq = nbp / 4;  // K stages

    // producer role: (row, half) of the weight tile
    const uint32_t prow = tid >> 1, phalf = tid & 1;
    const uint32_t wrow = min(n0 + prow, N - 1);
    const uint8_t* qrow = qs + (size_t)wrow * nbp * QB;
    const uint8_t* srow = sc + (size_t)wrow * scp * SB;

    // activation tile copy: 128 rows x 16 chunks per stage, 8 chunks per thread
    auto issue_b = [&](uint32_t stage, uint32_t kq) {
        const uint32_t b_tiles = smem32 + stage * STAGE_BYTES + 2 * HALF_TILE;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t idx = tid + i * THREADS;          // 0 .. 2047
            const uint32_t r = idx >> 4, c16 = idx & 15;     // row, 16-byte chunk within the 256-byte K slice
            const uint32_t m = m0 + r;
            const uint32_t k = kq * BK + c16 * 8;
            const bool ok = m < M && k < K;
            const __half* src = x16 + (size_t)(ok ? m : 0) * K + (ok ? k : 0);
            cp_async16_zfill(b_tiles + (c16 >> 3) * HALF_TILE + swz(r, c16 & 7), src, ok ? 16u : 0u);
        }
    };

    // consumer role: warp grid 4 (weight rows) x 2 (activation rows); warp tile 32 x 64
    const uint32_t wn = warp & 3, wm = warp >> 2;
    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;

    // ldmatrix lane addressing: A matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15); B matrices (n 0-7, k 0-7),
    // (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
    const uint32_t a_row = wn * 32 + (lane & 15), a_chunk = lane >> 4;
    const uint32_t b_row = wm * 64 + (lane & 7) + ((lane >> 4) << 3), b_chunk = (lane >> 3) & 1;

    PackedQuad<TYPE> pk;
    // prologue: stages 0 and 1
    load_packed<TYPE>(pk, qrow, srow, 0, phalf);
    issue_b(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    store_dequant<TYPE>(pk, smem32, prow, phalf);
    if (nq > 1) {
        load_packed<TYPE>(pk, qrow, srow, 1, phalf);
        issue_b(1, 1);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");

    for (uint32_t kq = 0; kq < nq; ++kq) {
        const uint32_t stage = kq % STAGES;
        // stage kq + 1: dequantise from the registers loaded one iteration ago
        if (kq + 1 < nq) store_dequant<TYPE>(pk, smem32 + ((kq + 1) % STAGES) * STAGE_BYTES, prow, phalf);
        // stage kq + 2: start its loads
        if (kq + 2 < nq) {
            load_packed<TYPE>(pk, qrow, srow, kq + 2, phalf);
            issue_b((kq + 2) % STAGES, kq + 2);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 2;" ::: "memory");  // the activation tile of stage kq has landed
        __syncthreads();                                       // ... and everybody's weight stores for it

        const uint32_t a_tiles = smem32 + stage * STAGE_BYTES, b_tiles = a_tiles + 2 * HALF_TILE;
#pragma unroll
        for (int k16 = 0; k16 < 8; ++k16) {
            const uint32_t kh = k16 >> 2, c0 = (k16 & 3) * 2;
            uint32_t a[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(a[i], a_tiles + kh * HALF_TILE + swz(a_row + i * 16, c0 + a_chunk));
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                uint32_t b[4];
                ldmatrix_x4(b, b_tiles + kh * HALF_TILE + swz(b_row + jj * 16, c0 + b_chunk));
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma16816(acc[i][2 * jj], a[i], b[0], b[1]);
                    mma16816(acc[i][2 * jj + 1], a[i], b[2], b[3]);
                }
            }
        }
        __syncthreads();  // stage kq may be overwritten by the stores / copies of iteration kq + 1
    }

    // epilogue: acc[i][j] = rows n (g, g + 8), activation rows m (2t, 2t + 1)
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t n = n0 + wn * 32 + i * 16 + g + (e >> 1) * 8;
                const uint32_t m = m0 + wm * 64 + j * 8 + 2 * t + (e & 1);
                if (n < N && m < M) {
                    const size_t o = (size_t)m * N + n;
                    float v = acc[i][j][e] * post[m];
                    if (ep.bias) v = __fadd_rn(v, ep.bias[n]);
                    if (ep.gelu) v = gelu_tanh(v);
                    if (ep.mul) v = __fmul_rn(v, ep.mul[o]);
                    if (ep.residual) v = __fadd_rn(ep.residual[o], v);
                    y[o] = v;
                }
            }
        }
    }
}

template <int TYPE>
int launch_gemm(const zq_weight* w, const __half* x16, const float* post, float* y, uint32_t M, GemmEpilogue ep,
                cudaStream_t st) {
    auto kern = gemm_f16_kernel<TYPE>;
    const size_t smem = (size_t)STAGES * STAGE_BYTES;
    ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const dim3 grid((w->out_dim + BN - 1) / BN, (M + BM - 1) / BM);
    kern<<<grid, THREADS, smem, st>>>(w->qs, static_cast<const uint8_t*>(w->sc), x16, post, y, w->out_dim,
                                       w->in_dim, M, w->nbp, w->scp, ep);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

}  // namespace

size_t gemm_f16_workspace_bytes(const zq_weight* w, uint32_t m_rows) {
    const size_t xb = ((size_t)m_rows * w->in_dim * sizeof(__half) + 255) & ~(size_t)255;
    const size_t pb = ((size_t)m_rows * sizeof(float) + 255) & ~(size_t)255;
    return xb + pb;
}

int launch_convert_rows_f16(const float* x, __half* x16, float* post, uint32_t m_rows, uint32_t in_dim,
                            cudaStream_t st) {
    convert_rows_f16_kernel<<<m_rows, 256, 0, st>>>(x, x16, post, in_dim);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int launch_gemm_f16(const zq_weight* w, const float* x, float* y, uint32_t m_rows, const zq_epilogue* ep,
                    void* workspace, cudaStream_t st) {
    if (m_rows > 65535u * BM) return ZQ_ERR_LIMIT;
    const size_t xb = ((size_t)m_rows * w->in_dim * sizeof(__half) + 255) & ~(size_t)255;
    __half* x16 = static_cast<__half*>(workspace);
    float* post = reinterpret_cast<float*>(static_cast<char*>(workspace) + xb);
    int rc0 = launch_convert_rows_f16(x, x16, post, m_rows, w->in_dim, st);
    if (rc0 != ZQ_OK) return rc0;
    GemmEpilogue a{nullptr, nullptr, nullptr, 0};
    if (ep) {
        a.bias = ep->d_bias;
        a.gelu = ep->gelu;
        a.mul = ep->d_mul;
        a.residual = ep->d_residual;
    }
    switch (w->type) {
        case ZQ_TYPE_Q4_0: return launch_gemm<ZQ_TYPE_Q4_0>(w, x16, post, y, m_rows, a, st);
        case ZQ_TYPE_Q4_1: return launch_gemm<ZQ_TYPE_Q4_1>(w, x16, post, y, m_rows, a, st);
        case ZQ_TYPE_Q8_0: return launch_gemm<ZQ_TYPE_Q8_0>(w, x16, post, y, m_rows, a, st);
        default: return ZQ_ERR_UNSUPPORTED;
    }
}

}  // namespace zq
