// Exact integer GEMM for Q8-quantised activations and many activation rows (batched decode, prefill).
//
// Same arithmetic as the decode kernel in gemv_q8.cu and as zig-nn's CPU path
// (ThreadPool.matmul, src/gguf/thread_pool.zig:96-181 -> src/gguf/simd_dot.zig:71-152): per 32-block an
// exact int8 x int8 -> int32 dot, turned into the f32 term (d * s) * float(idot) [+ (m * s) * float(qsum)],
// and the terms of a row added in block order. Here the block dots of 16 weight rows x 8 activation rows
// come from one mma.sync.m16n8k32 (s8 x s8 -> s32, exact), the weights are read once per 64 activation
// rows instead of once per row, and each (weight row, activation row) pair keeps its running f32 sum in
// a register, so the result is bit-identical to running the decode kernel row by row.
//
// Tile: 128 weight rows (8 warps x 16) x 64 activation rows per CTA; K advances by one quad of blocks
// (128 values). Everything a quad needs travels through a ring of D shared-memory stages filled with
// cp.async, D - 1 quads ahead of the multiplications: the quantised activations (64 rows x 128 bytes, their
// scales and sums; 16-byte halves of a (row, block) entry are swapped for rows with bit 2 set so that the
// fragment loads are free of bank conflicts) and, per lane, the packed weight words and scales of its two
// rows. The small CTA shapes used for matrices with few rows have only a few warps per SM, so the depth of
// this ring — not occupancy — is what hides the memory latency there.
#include "zq_internal.h"

namespace zq {
namespace {

// CTA shape: W warps x 16 weight rows, NT x 8 activation rows. The large shape (8 warps, 64 rows) reads
// the weights once per 64 activation rows; matrices with few rows take smaller CTAs so that the grid
// still covers the GPU.

struct QgEpilogue {
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

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ uint32_t pick4(const uint4& v, int j) {
    return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// Bytes of one ring stage: activations of the CTA, then per warp the packed words (512 bytes per array:
// rows g, rows g + 8, and for q8_0 their second halves) and the scales (rows g, rows g + 8).
template <int TYPE, int W, int NT>
struct QgStage {
    static constexpr uint32_t kXq = 4 * NT * 8 * 32;   // 4 blocks x BM rows x 32 int8
    static constexpr uint32_t kSc = 4 * NT * 8 * 4;    // 4 blocks x BM rows x f32 (and the same for the sums)
    static constexpr uint32_t kAct = kXq + 2 * kSc;
    static constexpr uint32_t kWq = TYPE == ZQ_TYPE_Q8_0 ? 2048 : 1024;
    static constexpr uint32_t kWsHalf = TYPE == ZQ_TYPE_Q4_1 ? 512 : 256;
    static constexpr uint32_t kWarp = kWq + 2 * kWsHalf;
    static constexpr uint32_t kBytes = (kAct + W * kWarp + 127u) & ~127u;
};

template <int TYPE, int W, int NT, int D>
__global__ void __launch_bounds__(W * 32)
gemm_q8_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ sc, const int8_t* __restrict__ xq,
               const float* __restrict__ xscale, const int32_t* __restrict__ xqsum, float* __restrict__ y,
               uint32_t N, uint32_t K, uint32_t M, uint32_t nb, uint32_t scp, QgEpilogue ep) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QB = Q8 ? 32 : 16;
    constexpr uint32_t QUAD = 4 * QB;
    using S = QgStage<TYPE, W, NT>;
    constexpr int QG_BN = W * 16, QG_BM = NT * 8, QG_NT = NT;
    constexpr uint32_t QG_XQ_BYTES = S::kXq, QG_SC_BYTES = S::kSc, QG_STAGE = S::kBytes;
    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t smem32 = (uint32_t)__cvta_generic_to_shared(smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t nbp = (nb + 3u) & ~3u, nq = nbp / 4;
    const uint32_t n0 = blockIdx.x * QG_BN + warp * 16, m0 = blockIdx.y * QG_BM;

    const uint32_t row_a = min(n0 + g, N - 1), row_b = min(n0 + g + 8, N - 1);
    const uint8_t* pa = qs + (size_t)row_a * nbp * QB + 16 * t;
    const uint8_t* pb = qs + (size_t)row_b * nbp * QB + 16 * t;
    const uint8_t* sa = sc + (size_t)row_a * scp * (Q41 ? 4 : 2);
    const uint8_t* sb = sc + (size_t)row_b * scp * (Q41 ? 4 : 2);
    const uint32_t wring = smem32 + S::kAct + warp * S::kWarp;  // this warp's part of stage 0

    // Quad q -> stage. Activations: xq entries [blk][row][32 bytes] (16-byte halves swapped when row & 4),
    // scales [blk][row], sums [blk][row]; rows >= M and blocks >= nb are zero-filled (never used for output).
    // Weights: every lane copies the 16-byte pieces and the scales of its own two rows and reads the same
    // slots back later, so they need no synchronisation beyond cp.async.wait_group.
    auto issue = [&](uint32_t stage, uint32_t q) {
        const uint32_t base = smem32 + stage * QG_STAGE;
        for (uint32_t idx = tid; idx < 8u * QG_BM; idx += W * 32) {  // (blk, row, half)
            const uint32_t b = idx / (2u * QG_BM), r = (idx >> 1) % QG_BM, h = idx & 1u;
            const uint32_t blk = q * 4 + b, m = m0 + r;
            const bool ok = m < M && blk < nb;
            const int8_t* src = xq + (size_t)(ok ? m : 0) * K + (size_t)(ok ? blk : 0) * 32 + h * 16;
            cp_async16_zfill(base + ((b * QG_BM + r) * 2 + (h ^ ((r >> 2) & 1u))) * 16, src, ok ? 16u : 0u);
        }
        for (uint32_t idx = tid; idx < 4u * QG_BM; idx += W * 32) {  // (blk, row)
            const uint32_t b = idx / QG_BM, r = idx % QG_BM;
            const uint32_t blk = q * 4 + b, m = m0 + r;
            const bool ok = m < M && blk < nb;
            const size_t o = (size_t)(ok ? m : 0) * nb + (ok ? blk : 0);
            cp_async4_zfill(base + QG_XQ_BYTES + (b * QG_BM + r) * 4, xscale + o, ok ? 4u : 0u);
            cp_async4_zfill(base + QG_XQ_BYTES + QG_SC_BYTES + (b * QG_BM + r) * 4, xqsum + o, ok ? 4u : 0u);
        }
        const uint32_t wb = wring + stage * QG_STAGE;
        cp_async16(wb + lane * 16, pa + (size_t)q * QUAD);
        cp_async16(wb + 512 + lane * 16, pb + (size_t)q * QUAD);
        if (Q8) {
            cp_async16(wb + 1024 + lane * 16, pa + (size_t)q * QUAD + 64);
            cp_async16(wb + 1536 + lane * 16, pb + (size_t)q * QUAD + 64);
        }
        if (Q41) {
            cp_async16(wb + S::kWq + lane * 16, reinterpret_cast<const uint4*>(sa) + q);
            cp_async16(wb + S::kWq + S::kWsHalf + lane * 16, reinterpret_cast<const uint4*>(sb) + q);
        } else {
            cp_async8(wb + S::kWq + lane * 8, reinterpret_cast<const uint2*>(sa) + q);
            cp_async8(wb + S::kWq + S::kWsHalf + lane * 8, reinterpret_cast<const uint2*>(sb) + q);
        }
    };

    float run[QG_NT][4];
#pragma unroll
    for (int j = 0; j < QG_NT; ++j) run[j][0] = run[j][1] = run[j][2] = run[j][3] = 0.0f;

    // fragment addressing inside a stage: entry (blk, row = 8j + g), word t (and 4 + t), halves swapped by row bit 2
    const uint32_t swap = ((uint32_t)g >> 2) & 1u;
    const uint32_t frag_lo = ((uint32_t)g * 2 + (0u ^ swap)) * 16 + t * 4;   // word t
    const uint32_t frag_hi = ((uint32_t)g * 2 + (1u ^ swap)) * 16 + t * 4;   // word 4 + t

    // the quantised activations come from the kernel before this one
    pdl_launch_dependents();
    pdl_wait();

    // group number n holds quad n (an empty group when the row has no such quad)
#pragma unroll 1
    for (uint32_t i = 0; i + 1 < (uint32_t)D; ++i) {
        if (i < nq) issue(i, i);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    uint32_t stage = 0, p_stage = D - 1;
#pragma unroll 1
    for (uint32_t q = 0; q < nq; ++q) {
        if (q + D - 1 < nq) issue(p_stage, q + D - 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        p_stage = p_stage + 1 == (uint32_t)D ? 0 : p_stage + 1;
        asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory");  // quad q has landed
        __syncthreads();

        const uint32_t base = smem32 + stage * QG_STAGE;
        const uint32_t wb = wring + stage * QG_STAGE;
        const uint4 wa = lds128(wb + lane * 16), wbv = lds128(wb + 512 + lane * 16);
        uint4 wa2 = wa, wb2 = wbv;
        if (Q8) {
            wa2 = lds128(wb + 1024 + lane * 16);
            wb2 = lds128(wb + 1536 + lane * 16);
        }
        float da[4], db[4], ma[4], mb[4];
        if (Q41) {
            const uint4 sa4 = lds128(wb + S::kWq + lane * 16), sb4 = lds128(wb + S::kWq + S::kWsHalf + lane * 16);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t ua = pick4(sa4, b), ub = pick4(sb4, b);
                const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&ua));
                const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&ub));
                da[b] = fa.x; ma[b] = fa.y;
                db[b] = fb.x; mb[b] = fb.y;
            }
        } else {
            const uint2 sa2 = lds64(wb + S::kWq + lane * 8), sb2 = lds64(wb + S::kWq + S::kWsHalf + lane * 8);
            const float2 a01 = __half22float2(*reinterpret_cast<const __half2*>(&sa2.x));
            const float2 a23 = __half22float2(*reinterpret_cast<const __half2*>(&sa2.y));
            const float2 b01 = __half22float2(*reinterpret_cast<const __half2*>(&sb2.x));
            const float2 b23 = __half22float2(*reinterpret_cast<const __half2*>(&sb2.y));
            da[0] = a01.x; da[1] = a01.y; da[2] = a23.x; da[3] = a23.y;
            db[0] = b01.x; db[1] = b01.y; db[2] = b23.x; db[3] = b23.y;
#pragma unroll
            for (int b = 0; b < 4; ++b) ma[b] = mb[b] = 0.0f;
        }
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            if (q * 4 + b >= nb) break;  // row padding: no term is added for blocks that do not exist
            uint32_t a0, a1, a2, a3;
            if (Q8) {
                a0 = pick4(wa, b); a1 = pick4(wbv, b); a2 = pick4(wa2, b); a3 = pick4(wb2, b);
            } else {
                const uint32_t ua = pick4(wa, b), ub = pick4(wbv, b);
                a0 = ua & 0x0F0F0F0Fu; a1 = ub & 0x0F0F0F0Fu;
                a2 = (ua >> 4) & 0x0F0F0F0Fu; a3 = (ub >> 4) & 0x0F0F0F0Fu;
            }
            const uint32_t xb = base + b * (QG_BM * 32), sbase = base + QG_XQ_BYTES + b * (QG_BM * 4);
#pragma unroll
            for (int j = 0; j < QG_NT; ++j) {
                const uint32_t b0 = lds32(xb + j * 256 + frag_lo), b1 = lds32(xb + j * 256 + frag_hi);
                int d[4];
                mma_s8(d, a0, a1, a2, a3, b0, b1);
                // columns of this lane: activation rows 8j + 2t and 8j + 2t + 1
                const uint32_t so = sbase + (j * 8 + 2 * t) * 4;
                float s0, s1;
                asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(s0), "=f"(s1) : "r"(so));
                int qs0 = 0, qs1 = 0;
                if (!Q8) asm volatile("ld.shared.v2.s32 {%0,%1}, [%2];" : "=r"(qs0), "=r"(qs1) : "r"(so + QG_SC_BYTES));
                if (TYPE == ZQ_TYPE_Q4_0) {  // sum((n - 8) * q) = sum(n * q) - 8 * sum(q), exact
                    d[0] -= 8 * qs0; d[1] -= 8 * qs1; d[2] -= 8 * qs0; d[3] -= 8 * qs1;
                }
                float t0 = __fmul_rn(__fmul_rn(da[b], s0), (float)d[0]);
                float t1 = __fmul_rn(__fmul_rn(da[b], s1), (float)d[1]);
                float t2 = __fmul_rn(__fmul_rn(db[b], s0), (float)d[2]);
                float t3 = __fmul_rn(__fmul_rn(db[b], s1), (float)d[3]);
                if (Q41) {
                    t0 = __fadd_rn(t0, __fmul_rn(__fmul_rn(ma[b], s0), (float)qs0));
                    t1 = __fadd_rn(t1, __fmul_rn(__fmul_rn(ma[b], s1), (float)qs1));
                    t2 = __fadd_rn(t2, __fmul_rn(__fmul_rn(mb[b], s0), (float)qs0));
                    t3 = __fadd_rn(t3, __fmul_rn(__fmul_rn(mb[b], s1), (float)qs1));
                }
                run[j][0] = __fadd_rn(run[j][0], t0);
                run[j][1] = __fadd_rn(run[j][1], t1);
                run[j][2] = __fadd_rn(run[j][2], t2);
                run[j][3] = __fadd_rn(run[j][3], t3);
            }
        }
        __syncthreads();  // this stage is overwritten by the copies issued in the next iteration
        stage = stage + 1 == (uint32_t)D ? 0 : stage + 1;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");

#pragma unroll
    for (int j = 0; j < QG_NT; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t n = n0 + g + (e >> 1) * 8;
            const uint32_t m = m0 + j * 8 + 2 * t + (e & 1);
            if (n < N && m < M) {
                const size_t o = (size_t)m * N + n;
                float v = run[j][e];
                if (ep.bias) v = __fadd_rn(v, ep.bias[n]);
                if (ep.gelu) v = gelu_tanh(v);
                if (ep.mul) v = __fmul_rn(v, ep.mul[o]);
                if (ep.residual) v = __fadd_rn(ep.residual[o], v);
                y[o] = v;
            }
        }
    }
}

template <int TYPE, int W, int NT, int D>
int launch_cfg(const zq_weight* w, const int8_t* xq, const float* xs, const int32_t* xsum, float* y, uint32_t M,
               QgEpilogue ep, cudaStream_t st) {
    const dim3 grid((w->out_dim + W * 16 - 1) / (W * 16), (M + NT * 8 - 1) / (NT * 8));
    if (grid.y > 65535u) return ZQ_ERR_LIMIT;
    const size_t smem = (size_t)D * QgStage<TYPE, W, NT>::kBytes;
    auto kern = gemm_q8_kernel<TYPE, W, NT, D>;
    if (smem > 48 * 1024)
        ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    ZQ_CUDA(launch_pdl(kern, grid, dim3(W * 32), smem, st, w->qs, static_cast<const uint8_t*>(w->sc), xq, xs, xsum,
                       y, w->out_dim, w->in_dim, M, w->nb, w->scp, ep));
    return ZQ_OK;
}

// CTA shape by measurement on the Gemma-3 layer shapes (64 and 128 activation rows): a warp owns 16 weight
// rows x NT column tiles of 8 activation rows. Few column tiles per warp mean more warps (the running sums
// are a serial chain over K per output, so only more, smaller warp tiles shorten a launch that cannot fill
// the GPU) but also more passes over the weights through L2; so: the largest NT that still gives about
// 1000 warps, never so small that a weight is read more than 8 times, and the smallest such NT when no
// choice reaches 1000 warps. (6912->1152 at 128 rows: 35 us with NT = 2, 41 us with NT = 1, 60 us with
// one-warp CTAs; 1152->13824 at 64 rows: 21 us with NT = 4, 25 us with NT = 8.)
template <int TYPE>
int launch_one(const zq_weight* w, const int8_t* xq, const float* xs, const int32_t* xsum, float* y, uint32_t M,
               QgEpilogue ep, cudaStream_t st) {
    const uint64_t rt = (w->out_dim + 15) / 16, mt8 = (M + 7) / 8;
    uint32_t nt_cap = 1, nt_min = 1;
    while (nt_cap < 8 && nt_cap < mt8) nt_cap *= 2;
    while (nt_min < nt_cap && (mt8 + nt_min - 1) / nt_min > 8) nt_min *= 2;
    uint32_t nt = nt_min;
    for (uint32_t c = nt_cap; c >= nt_min; c /= 2)
        if (rt * ((mt8 + c - 1) / c) >= 1000) {
            nt = c;
            break;
        }
    switch (nt) {
        case 8: return launch_cfg<TYPE, 8, 8, 3>(w, xq, xs, xsum, y, M, ep, st);
        case 4: return launch_cfg<TYPE, 4, 4, 4>(w, xq, xs, xsum, y, M, ep, st);
        case 2: return launch_cfg<TYPE, 4, 2, 6>(w, xq, xs, xsum, y, M, ep, st);
        default: return launch_cfg<TYPE, 4, 1, 8>(w, xq, xs, xsum, y, M, ep, st);
    }
}

}  // namespace

int launch_gemm_q8(const zq_weight* w, const int8_t* xq, const float* xscale, const int32_t* xsum, float* y,
                   uint32_t m_rows, const zq_epilogue* ep, cudaStream_t st) {
    QgEpilogue a{nullptr, nullptr, nullptr, 0};
    if (ep) {
        a.bias = ep->d_bias;
        a.gelu = ep->gelu;
        a.mul = ep->d_mul;
        a.residual = ep->d_residual;
    }
    switch (w->type) {
        case ZQ_TYPE_Q4_0: return launch_one<ZQ_TYPE_Q4_0>(w, xq, xscale, xsum, y, m_rows, a, st);
        case ZQ_TYPE_Q4_1: return launch_one<ZQ_TYPE_Q4_1>(w, xq, xscale, xsum, y, m_rows, a, st);
        case ZQ_TYPE_Q8_0: return launch_one<ZQ_TYPE_Q8_0>(w, xq, xscale, xsum, y, m_rows, a, st);
        default: return ZQ_ERR_UNSUPPORTED;
    }
}

}  // namespace zq
