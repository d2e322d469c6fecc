// Transposed quantised matmul: grad_x[M][K] (+)= grad_out[M][N] . W[N][K] — the backward of the
// quantised linear with respect to its activations, weights dequantised on the fly
// (zig-nn src/backend/shaders/nn_training_kernels.metal:1143-1242 `matmul_q*_trans_batched`, called from
// src/diff/mps_runtime.zig:1212-1230 `backward_quant_matmul`; the reference accumulates into grad_x).
//
// The contraction runs over the weight ROWS, so a weight tile is used as stored — row j, elements k
// contiguous — as the "B" operand read with ldmatrix.trans, and the fp16 copy of grad_out (per-row
// power-of-two scale, as for the forward GEMM) is the "A" operand. Per stage a CTA dequantises one quad
// of blocks (128 k) of 128 weight rows into a swizzled fp16 tile and copies a [128 m][128 j] tile of
// grad_out beside it; 8 warps as 4 (m) x 2 (k), warp tile 32 x 64, f32 accumulation on mma.sync.
// Weights and gradients are each rounded once to fp16: about 3e-4 relative L2 against the f32 statement.
//
// A matrix with few 128-column tiles (K = 1152 has nine) would leave most SMs idle, so the weight rows
// can be split over blockIdx.z; the partial tiles then meet in grad_x through red.global.add.f32.
#include "gemm_common.cuh"

namespace zq {
namespace {

using namespace gemm_common;

constexpr int TM = 128;       // grad_out rows per CTA
constexpr int TK = 128;       // output columns per CTA: one quad of blocks
constexpr int TJ = 128;       // weight rows (contraction) per stage
constexpr int STAGES = 3;
constexpr int THREADS = 256;
constexpr uint32_t STAGE_BYTES = 4 * HALF_TILE;  // W tile (k halves 0 / 1), grad_out tile (j halves 0 / 1)

enum StoreMode { STORE = 0, ADD = 1, ATOMIC_ADD = 2 };

__device__ __forceinline__ void red_add_f32(float* p, float v) {
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

template <int TYPE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_trans_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ sc, const __half* __restrict__ g16,
                  const float* __restrict__ post, float* __restrict__ gx, uint32_t N, uint32_t K, uint32_t M,
                  uint32_t nbp, uint32_t scp, uint32_t chunks_per_split, int mode) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QB = Q8 ? 32 : 16;
    constexpr uint32_t SB = Q41 ? 4 : 2;
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t smem32 = (uint32_t)__cvta_generic_to_shared(smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t quad = blockIdx.x, k0 = quad * TK, m0 = blockIdx.y * TM;
    const uint32_t n_chunks = (N + TJ - 1) / TJ;
    const uint32_t c_lo = blockIdx.z * chunks_per_split;
    const uint32_t c_hi = min(c_lo + chunks_per_split, n_chunks);
    if (c_lo >= c_hi) return;
    const uint32_t nst = c_hi - c_lo;  // stages of this CTA

    // producer role: (weight row within the chunk, half) of this CTA's quad
    const uint32_t prow = tid >> 1, phalf = tid & 1;
    PackedQuad<TYPE> pk;
    auto load_w = [&](uint32_t chunk) {
        const uint32_t j = chunk * TJ + prow;
        const uint32_t jr = min(j, N - 1);
        load_packed<TYPE>(pk, qs + (size_t)jr * nbp * QB, sc + (size_t)jr * scp * SB, quad, phalf);
        if (j >= N) pk.s = make_uint4(0, 0, 0, 0);  // rows past the matrix: scale 0 -> the tile row is zero
    };
    // grad_out tile: 128 rows x 16 chunks of 8 halves per stage, 8 chunks per thread; zero past M and N
    auto issue_g = [&](uint32_t stage, uint32_t chunk) {
        const uint32_t tiles = smem32 + stage * STAGE_BYTES + 2 * HALF_TILE;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t idx = tid + i * THREADS;
            const uint32_t r = idx >> 4, c16 = idx & 15;
            const uint32_t m = m0 + r;
            const uint32_t j = chunk * TJ + c16 * 8;
            uint32_t bytes = 0;
            if (m < M && j < N) bytes = min(16u, (N - j) * 2u);
            const __half* src = g16 + (size_t)(bytes ? m : 0) * N + (bytes ? j : 0);
            cp_async16_zfill(tiles + (c16 >> 3) * HALF_TILE + swz(r, c16 & 7), src, bytes);
        }
    };

    // consumer role: warp grid 4 (m) x 2 (k); warp tile 32 x 64
    const uint32_t wm = warp & 3, wk = warp >> 2;
    float acc[2][8][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.0f;

    // A (grad_out) matrices: (rows 0-7 | 8-15) x (j 0-7 | 8-15). B (weights, transposed on load): matrices
    // (j 0-7, k 0-7), (j 8-15, k 0-7), (j 0-7, k 8-15), (j 8-15, k 8-15): lane l supplies row l % 16 of the
    // 16 weight rows and the 16-byte chunk (l / 16) of the pair of 8-column groups.
    const uint32_t a_row = wm * 32 + (lane & 15), a_chunk = lane >> 4;
    const uint32_t b_row = lane & 15, b_chunk = lane >> 4;

    load_w(c_lo);
    issue_g(0, c_lo);
    asm volatile("cp.async.commit_group;" ::: "memory");
    store_dequant<TYPE>(pk, smem32, prow, phalf);
    if (nst > 1) {
        load_w(c_lo + 1);
        issue_g(1, c_lo + 1);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");

    for (uint32_t s = 0; s < nst; ++s) {
        const uint32_t stage = s % STAGES;
        if (s + 1 < nst) store_dequant<TYPE>(pk, smem32 + ((s + 1) % STAGES) * STAGE_BYTES, prow, phalf);
        if (s + 2 < nst) {
            load_w(c_lo + s + 2);
            issue_g((s + 2) % STAGES, c_lo + s + 2);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 2;" ::: "memory");  // the grad_out tile of this stage has landed
        __syncthreads();                                       // ... and everybody's weight stores for it

        const uint32_t w_tiles = smem32 + stage * STAGE_BYTES, g_tiles = w_tiles + 2 * HALF_TILE;
#pragma unroll
        for (int j16 = 0; j16 < 8; ++j16) {
            uint32_t a[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(a[i], g_tiles + (j16 >> 2) * HALF_TILE + swz(a_row + i * 16, (j16 & 3) * 2 + a_chunk));
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                // columns wk * 64 + jj * 16 .. + 15 of the quad: chunk index within the 128-column row
                const uint32_t c = wk * 8 + jj * 2 + b_chunk;
                uint32_t b[4];
                ldmatrix_x4_trans(b, w_tiles + (c >> 3) * HALF_TILE + swz(j16 * 16 + b_row, c & 7));
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    mma16816(acc[i][2 * jj], a[i], b[0], b[1]);
                    mma16816(acc[i][2 * jj + 1], a[i], b[2], b[3]);
                }
            }
        }
        __syncthreads();  // this stage may be overwritten by the stores / copies of the next iteration
    }

    // acc[i][j]: rows m (g, g + 8), columns k (2t, 2t + 1)
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t m = m0 + wm * 32 + i * 16 + g + h * 8;
            if (m >= M) continue;
            const float ps = post[m];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t k = k0 + wk * 64 + j * 8 + 2 * t;
                if (k >= K) continue;  // K is a multiple of 32: k and k + 1 are valid together
                float* o = gx + (size_t)m * K + k;
                const float v0 = acc[i][j][2 * h] * ps, v1 = acc[i][j][2 * h + 1] * ps;
                if (mode == STORE) {
                    *reinterpret_cast<float2*>(o) = make_float2(v0, v1);
                } else if (mode == ADD) {
                    float2 old = *reinterpret_cast<const float2*>(o);
                    old.x += v0;
                    old.y += v1;
                    *reinterpret_cast<float2*>(o) = old;
                } else {
                    red_add_f32(o, v0);
                    red_add_f32(o + 1, v1);
                }
            }
        }
    }
}

template <int TYPE>
int launch_trans(const zq_weight* w, const __half* g16, const float* post, float* gx, uint32_t M, int accumulate,
                 cudaStream_t st) {
    auto kern = gemm_trans_kernel<TYPE>;
    const size_t smem = (size_t)STAGES * STAGE_BYTES;
    ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const uint32_t quads = (w->in_dim + TK - 1) / TK, mt = (M + TM - 1) / TM;
    const uint32_t n_chunks = (w->out_dim + TJ - 1) / TJ;
    // split the weight rows until the grid covers the GPU about twice, keeping at least 4 stages per CTA
    uint32_t splits = 1;
    const uint32_t want = (uint32_t)sm_count() * 2;
    while (quads * mt * splits < want && n_chunks / (splits * 2) >= 4 && splits < 64) splits *= 2;
    const uint32_t per = (n_chunks + splits - 1) / splits;
    splits = (n_chunks + per - 1) / per;
    int mode = accumulate ? ADD : STORE;
    if (splits > 1) {
        mode = ATOMIC_ADD;
        if (!accumulate) ZQ_CUDA(cudaMemsetAsync(gx, 0, (size_t)M * w->in_dim * sizeof(float), st));
    }
    kern<<<dim3(quads, mt, splits), THREADS, smem, st>>>(w->qs, static_cast<const uint8_t*>(w->sc), g16, post, gx,
                                                          w->out_dim, w->in_dim, M, w->nbp, w->scp, per, mode);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

}  // namespace
}  // namespace zq

using namespace zq;

extern "C" size_t zq_matmul_transposed_workspace_bytes(const zq_weight* w, uint32_t m_rows) {
    if (!w) return 0;
    const size_t gb = ((size_t)m_rows * w->out_dim * sizeof(__half) + 255) & ~(size_t)255;
    const size_t pb = ((size_t)m_rows * sizeof(float) + 255) & ~(size_t)255;
    const size_t pair = gemm_trans_pair_takes(w, m_rows) ? gemm_trans_pair_workspace_bytes(w, m_rows) : 0;
    return gb + pb > pair ? gb + pb : pair;
}

extern "C" int zq_matmul_transposed(const zq_weight* w, const float* d_grad_out, float* d_grad_x, uint32_t m_rows,
                                    int accumulate, void* d_workspace, size_t workspace_bytes, zq_stream stream) {
    if (!w) return ZQ_ERR_BAD_ARG;
    if (m_rows == 0) return ZQ_OK;
    if (!d_grad_out || !d_grad_x) return ZQ_ERR_BAD_ARG;
    if (((uintptr_t)d_grad_x & 7) != 0) return ZQ_ERR_BAD_ARG;  // rows are written in 8-byte pairs
    if ((w->out_dim & 7) != 0) return ZQ_ERR_UNSUPPORTED;       // 16-byte copies of the fp16 gradient rows
    if (!d_workspace || ((uintptr_t)d_workspace & 255) ||
        workspace_bytes < zq_matmul_transposed_workspace_bytes(w, m_rows))
        return ZQ_ERR_BAD_ARG;
    if (m_rows > 65535u * TM) return ZQ_ERR_LIMIT;
    cudaStream_t st = as_stream(stream);
    // Many rows on a large matrix: W^T is laid out once as fp16 operand tiles and the product runs on the tcgen05
    // kernel of the forward GEMM (pairs of CTAs). ZQ_ERR_CUDA: the cluster launch was refused, nothing of the
    // product ran: the kernel below takes the call.
    if (gemm_trans_pair_takes(w, m_rows)) {
        const int rc = launch_gemm_trans_pair(w, d_grad_out, d_grad_x, m_rows, accumulate, d_workspace, st);
        if (rc != ZQ_ERR_CUDA) return rc;
        cudaGetLastError();
    }
    const size_t gb = ((size_t)m_rows * w->out_dim * sizeof(__half) + 255) & ~(size_t)255;
    __half* g16 = static_cast<__half*>(d_workspace);
    float* post = reinterpret_cast<float*>(static_cast<char*>(d_workspace) + gb);
    int rc = launch_convert_rows_f16(d_grad_out, g16, post, m_rows, w->out_dim, st);
    if (rc != ZQ_OK) return rc;
    switch (w->type) {
        case ZQ_TYPE_Q4_0: return launch_trans<ZQ_TYPE_Q4_0>(w, g16, post, d_grad_x, m_rows, accumulate, st);
        case ZQ_TYPE_Q4_1: return launch_trans<ZQ_TYPE_Q4_1>(w, g16, post, d_grad_x, m_rows, accumulate, st);
        case ZQ_TYPE_Q8_0: return launch_trans<ZQ_TYPE_Q8_0>(w, g16, post, d_grad_x, m_rows, accumulate, st);
        default: return ZQ_ERR_UNSUPPORTED;
    }
}
