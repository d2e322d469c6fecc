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
#include "zq_internal.h"

namespace zq {
namespace {

constexpr int BN = 128;      // weight rows per CTA (MMA M dimension)
constexpr int BM = 128;      // activation rows per CTA (MMA N dimension)
constexpr int BK = 128;      // K per stage: 4 blocks = one quad
constexpr int STAGES = 3;
constexpr int THREADS = 256;
constexpr uint32_t HALF_TILE = 128 * 128;            // bytes of a [128 rows][64 halves] tile
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

// byte offset of 16-byte chunk `c` (0..7) of row `r` inside a [rows][64 halves] tile
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }

__device__ __forceinline__ uint32_t hsub2_u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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

// ---- weights: one quad (4 blocks) of one row -> 8 chunks of 8 fp16 values ------------------------
// A thread owns (row, half): words 2*half and 2*half + 1 of each of the 4 blocks, i.e. for block j the
// elements [8*half, 8*half + 8) (low nibbles) and [16 + 8*half, 16 + 8*half + 8) (high nibbles).
template <int TYPE>
struct PackedQuad {
    uint4 w0, w1;        // word 2*half / 2*half + 1 of blocks 0..3 (q8_0: words 4*half .. 4*half + 3 in w0..w3)
    uint4 w2, w3;        // q8_0 only
    uint4 s;             // scales: q4_0 / q8_0 use .x, .y (4 x f16); q4_1 all four (4 x (d, m))
};

template <int TYPE>
__device__ __forceinline__ void load_packed(PackedQuad<TYPE>& p, const uint8_t* qrow, const uint8_t* srow,
                                            uint32_t quad, uint32_t half) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    if (Q8) {
        // q8_0 quad = 128 bytes: uint4 #u (u = 0..7) holds word (u / 4) * 4 + (u % 4) ... of blocks 0..3:
        // word w of block j sits at ((w / 4) * 16 + (w % 4) * 4 + j) * 4, so uint4 #w holds word w.
        const uint4* q = reinterpret_cast<const uint4*>(qrow + (size_t)quad * 128) + half * 4;
        p.w0 = __ldg(q); p.w1 = __ldg(q + 1); p.w2 = __ldg(q + 2); p.w3 = __ldg(q + 3);
    } else {
        const uint4* q = reinterpret_cast<const uint4*>(qrow + (size_t)quad * 64) + half * 2;
        p.w0 = __ldg(q); p.w1 = __ldg(q + 1);
    }
    if (Q41) {
        p.s = __ldg(reinterpret_cast<const uint4*>(srow) + quad);
    } else {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(srow) + quad);
        p.s.x = v.x; p.s.y = v.y;
    }
}

__device__ __forceinline__ uint32_t pick4(const uint4& v, int j) {
    return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w;
}

// Four 4-bit values held in the low nibbles of the bytes of `nib` -> two half2 (e0, e1), (e2, e3) of
// value * d (+ m): 0x6400 | n is the fp16 number 1024 + n.
template <int TYPE>
__device__ __forceinline__ void nibbles_to_half(uint32_t nib, uint32_t d2, uint32_t m2, uint32_t& h01,
                                                uint32_t& h23) {
    const uint32_t p01 = __byte_perm(nib, 0x64646464u, 0x5140);
    const uint32_t p23 = __byte_perm(nib, 0x64646464u, 0x5342);
    if (TYPE == ZQ_TYPE_Q4_0) {
        constexpr uint32_t k1032 = 0x64086408u;  // 1024 + 8
        h01 = hmul2_u(hsub2_u(p01, k1032), d2);
        h23 = hmul2_u(hsub2_u(p23, k1032), d2);
    } else {
        constexpr uint32_t k1024 = 0x64006400u;
        h01 = hfma2_u(hsub2_u(p01, k1024), d2, m2);
        h23 = hfma2_u(hsub2_u(p23, k1024), d2, m2);
    }
}
// Four int8 values -> two half2 of q * d.
__device__ __forceinline__ void bytes_to_half(uint32_t q, uint32_t d2, uint32_t& h01, uint32_t& h23) {
    const uint32_t u = q ^ 0x80808080u;  // b + 128 as unsigned bytes
    constexpr uint32_t k1152 = 0x64806480u;  // 1024 + 128
    h01 = hmul2_u(hsub2_u(__byte_perm(u, 0x64646464u, 0x5140), k1152), d2);
    h23 = hmul2_u(hsub2_u(__byte_perm(u, 0x64646464u, 0x5342), k1152), d2);
}

// Dequantise the thread's share of one stage and store it into the A tiles of that stage.
template <int TYPE>
__device__ __forceinline__ void store_dequant(const PackedQuad<TYPE>& p, uint32_t a_tiles, uint32_t row,
                                              uint32_t half) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t d2, m2 = 0;
        if (Q41) {
            const uint32_t dm = pick4(p.s, j);
            d2 = __byte_perm(dm, dm, 0x1010);
            m2 = __byte_perm(dm, dm, 0x3232);
        } else {
            const uint32_t pair = j < 2 ? p.s.x : p.s.y;
            d2 = (j & 1) ? __byte_perm(pair, pair, 0x3232) : __byte_perm(pair, pair, 0x1010);
        }
        // block j covers halves [32 * (j & 1), 32 * (j & 1) + 32) of K-half tile (j >> 1)
        const uint32_t tile = a_tiles + (j >> 1) * HALF_TILE;
        const uint32_t cbase = (j & 1) * 4;
        if (Q8) {
            // elements 16 * half .. 16 * half + 15 of the block: words w0..w3
            uint32_t h[8];
            bytes_to_half(pick4(p.w0, j), d2, h[0], h[1]);
            bytes_to_half(pick4(p.w1, j), d2, h[2], h[3]);
            bytes_to_half(pick4(p.w2, j), d2, h[4], h[5]);
            bytes_to_half(pick4(p.w3, j), d2, h[6], h[7]);
            sts128(tile + swz(row, cbase + half * 2), h[0], h[1], h[2], h[3]);
            sts128(tile + swz(row, cbase + half * 2 + 1), h[4], h[5], h[6], h[7]);
        } else {
            const uint32_t q0 = pick4(p.w0, j), q1 = pick4(p.w1, j);
            uint32_t lo[4], hi[4];
            nibbles_to_half<TYPE>(q0 & 0x0F0F0F0Fu, d2, m2, lo[0], lo[1]);
            nibbles_to_half<TYPE>(q1 & 0x0F0F0F0Fu, d2, m2, lo[2], lo[3]);
            nibbles_to_half<TYPE>((q0 >> 4) & 0x0F0F0F0Fu, d2, m2, hi[0], hi[1]);
            nibbles_to_half<TYPE>((q1 >> 4) & 0x0F0F0F0Fu, d2, m2, hi[2], hi[3]);
            sts128(tile + swz(row, cbase + half), lo[0], lo[1], lo[2], lo[3]);          // elements 8h .. 8h+7
            sts128(tile + swz(row, cbase + 2 + half), hi[0], hi[1], hi[2], hi[3]);      // elements 16+8h ..
        }
    }
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
