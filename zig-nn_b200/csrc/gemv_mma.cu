// f32-activation decode GEMV on the tensor cores (m_rows <= 16).
//
// The CUDA-core kernel in gemv.cu spends about four instructions per weight on turning nibbles
// into floats, which caps it near 40 % of HBM bandwidth. Here the integer weights (n-8, n, or the
// int8 value — all exact in fp16) go into mma.sync.m16n8k16 A fragments with two instructions per
// pair, and each f32 activation x is split into fp16 parts hi = fp16(x), lo = fp16(x - hi) that sit
// in two B columns. Products are exact, accumulation is f32, and hi + lo carries 22 bits of x, so
// results agree with the f32 CPU path (zig-nn src/gguf/dequant.zig:133-309) to about 1e-7.
//
// Tile: a warp owns 16 consecutive weight rows and walks the blocks of a K slice. For one block
// (32 weights per row) it issues two MMAs — low nibbles (elements 0..15), high nibbles (16..31) —
// into a fresh accumulator, then adds accumulator * d[row][block] into the running sums: the
// per-block scale is applied in f32, as the reference does.
//
// Fragment ownership (g = lane / 4, t = lane % 4): the thread loads quant word t of the block for
// rows g and g + 8. Word t holds elements 4t..4t+3 (low nibbles) and 16+4t..16+4t+3 (high nibbles),
// which is exactly the K footprint an m16n8k16 A fragment wants from lane (g, t), so no data moves
// between lanes. K slots are assigned as (2t, 2t+1, 2t+8, 2t+9) <- elements (4t, 4t+2, 4t+1, 4t+3);
// the activation fragments in shared memory are laid out with the same permutation.
#include "zq_internal.h"

namespace zq {
namespace {

constexpr int kMaxCols = 4;  // column sets of 8 MMA columns = 4 activation rows (hi, lo) each

struct EpilogueArgs {
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

__device__ __forceinline__ float apply_epilogue(float v, const EpilogueArgs& ep, size_t j, size_t mj) {
    if (ep.bias) v = __fadd_rn(v, ep.bias[j]);
    if (ep.gelu) v = gelu_tanh(v);
    if (ep.mul) v = __fmul_rn(v, ep.mul[mj]);
    if (ep.residual) v = __fadd_rn(ep.residual[mj], v);
    return v;
}

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                        const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]),
          "f"(c[3]));
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// One 4-bit quant word -> fp16 pairs. lo = (e0, e2), (e1, e3) of the low nibbles, hi likewise.
// (q & 0x000F000F) | 0x6400_6400 reads as (1024 + n, 1024 + n'); the 0x00F0 mask gives 1024 + 16 n.
// OFF = 8 (q4_0: n - 8) or 0 (q4_1: n). All results are exact.
template <int OFF>
__device__ __forceinline__ void unpack_q4(uint32_t q, uint32_t& lo02, uint32_t& lo13, uint32_t& hi02,
                                          uint32_t& hi13) {
    constexpr uint32_t kMagic = 0x64006400u;
    constexpr uint32_t kSubLo = OFF == 8 ? 0x64086408u : 0x64006400u;   // 1024 + OFF
    constexpr uint32_t kSixteenth = 0x2C002C00u;                        // 1/16
    constexpr uint32_t kSubHi = OFF == 8 ? 0xD480D480u : 0xD400D400u;   // -(64 + OFF)
    const uint32_t s = q >> 8;
    lo02 = hsub2_u32((q & 0x000F000Fu) | kMagic, kSubLo);
    hi02 = hfma2_u32((q & 0x00F000F0u) | kMagic, kSixteenth, kSubHi);
    lo13 = hsub2_u32((s & 0x000F000Fu) | kMagic, kSubLo);
    hi13 = hfma2_u32((s & 0x00F000F0u) | kMagic, kSixteenth, kSubHi);
}

// One int8 quant word (elements e0..e3) -> fp16 pairs (e0, e2), (e1, e3), exact.
__device__ __forceinline__ void unpack_q8(uint32_t q, uint32_t& p02, uint32_t& p13) {
    const uint32_t u = q ^ 0x80808080u;                 // b + 128 as unsigned bytes
    constexpr uint32_t kSub = 0x64806480u;              // 1024 + 128
    p02 = hsub2_u32(__byte_perm(u, 0x64646464u, 0x4240), kSub);
    p13 = hsub2_u32(__byte_perm(u, 0x64646464u, 0x4341), kSub);
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Shared-memory image of the activations for one K chunk:
//   frag[block][set][lane][4 x u32]: B fragments {MMA-low b0, b1, MMA-high b0, b1} of lane (g, t) for
//     column g of the set = activation row 4*set + g/2, part g%2 (0 = hi, 1 = lo);
//   xsum[block][16]: f32 sum of each activation row's 32 values (q4_1 only).
// `pre` holds the per-row power-of-two prescale that keeps |x| inside fp16 range.
template <bool WITH_SUM>
__device__ void stage_activations(const float* __restrict__ x, uint32_t M, uint32_t K, uint32_t blk0,
                                  uint32_t nblk, int ns, const float* pre, uint4* frag, float* xsum) {
    const uint32_t total = nblk * (uint32_t)ns * 32u;
    for (uint32_t i = threadIdx.x; i < total; i += blockDim.x) {
        const uint32_t lane = i & 31u, set = (i >> 5) % (uint32_t)ns, blk = (i >> 5) / (uint32_t)ns;
        const uint32_t g = lane >> 2, t = lane & 3u;
        const uint32_t m = 4u * set + (g >> 1);
        const bool lo_part = g & 1u;
        float v[8];
        if (m < M) {
            const float* p = x + (size_t)m * K + (size_t)(blk0 + blk) * 32u;
            const float4 a = *reinterpret_cast<const float4*>(p + 4u * t);
            const float4 b = *reinterpret_cast<const float4*>(p + 16u + 4u * t);
            const float s = pre[m];
            v[0] = a.x * s; v[1] = a.y * s; v[2] = a.z * s; v[3] = a.w * s;
            v[4] = b.x * s; v[5] = b.y * s; v[6] = b.z * s; v[7] = b.w * s;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.0f;
        }
        if (WITH_SUM) {
            // every lane of the quad (same g) adds its 8 values; lanes with g even publish the row sum
            float s8 = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
            s8 += __shfl_xor_sync(0xFFFFFFFFu, s8, 1);
            s8 += __shfl_xor_sync(0xFFFFFFFFu, s8, 2);
            if (!lo_part && t == 0 && m < 16) xsum[blk * 16u + m] = s8;
        }
        float w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float hi = __half2float(__float2half_rn(v[j]));
            w[j] = lo_part ? (v[j] - hi) : hi;  // x - hi is exact in f32
        }
        uint4 out;
        out.x = pack_half2(w[0], w[2]);
        out.y = pack_half2(w[1], w[3]);
        out.z = pack_half2(w[4], w[6]);
        out.w = pack_half2(w[5], w[7]);
        frag[i] = out;
    }
}

// Grid-stride over tiles of 16 rows x WR warps; the KS warps that share a row tile split the blocks
// of each K chunk and are summed in a fixed order through shared memory.
template <int TYPE, int NS, int U>
__global__ void __launch_bounds__(256, NS == 1 ? 4 : 2)
gemv_mma_kernel(const uint8_t* __restrict__ qs, const void* __restrict__ sc, const float* __restrict__ x,
                float* __restrict__ y, uint32_t N, uint32_t K, uint32_t nb, uint32_t M, uint32_t kc,
                uint32_t WR, uint32_t KS, EpilogueArgs ep) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr int QB = Q8 ? 32 : 16;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint4* frag = reinterpret_cast<uint4*>(smem_raw);                       // kc * NS * 32
    float* xsum = reinterpret_cast<float*>(frag + (size_t)kc * NS * 32);    // kc * 16 (q4_1)
    float* red = xsum + (Q41 ? (size_t)kc * 16 : 0);                        // KS>1: WR*KS*NS*4*32 (+Q41 *2*32)
    __shared__ float pre[16], post[16];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t wr = warp % WR, ks = warp / WR;

    // per activation row: power-of-two prescale so that |x| * pre < 2^15 (fp16 range), undone at the end
    for (uint32_t m = warp; m < M; m += blockDim.x >> 5) {
        float amax = 0.0f;
        for (uint32_t i = lane; i < K; i += 32) amax = fmaxf(amax, fabsf(x[(size_t)m * K + i]));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
        if (lane == 0) {
            int e = 0;
            if (amax >= 32768.0f && amax < INFINITY) e = ilogbf(amax) - 14;
            pre[m] = ldexpf(1.0f, -e);
            post[m] = ldexpf(1.0f, e);
        }
    }
    __syncthreads();

    const uint32_t n_chunks = (nb + kc - 1) / kc;
    const uint32_t rows_per_cta = WR * 16;
    bool staged = false;

    for (uint64_t tile = blockIdx.x; tile * rows_per_cta < N; tile += gridDim.x) {
        const uint32_t row_a = min((uint32_t)(tile * rows_per_cta) + wr * 16 + g, N - 1);
        const uint32_t row_b = min((uint32_t)(tile * rows_per_cta) + wr * 16 + g + 8, N - 1);
        const uint8_t* qa = qs + (size_t)row_a * nb * QB + 4 * t;
        const uint8_t* qb = qs + (size_t)row_b * nb * QB + 4 * t;
        float acc[NS][4];
        float accm[NS][2];
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            acc[s][0] = acc[s][1] = acc[s][2] = acc[s][3] = 0.0f;
            accm[s][0] = accm[s][1] = 0.0f;
        }

        for (uint32_t c = 0; c < n_chunks; ++c) {
            const uint32_t c0 = c * kc, cn = min(kc, nb - c0);
            if (n_chunks > 1 || !staged) {
                if (n_chunks > 1) __syncthreads();  // everyone is done with the previous chunk
                stage_activations<Q41>(x, M, K, c0, cn, NS, pre, frag, xsum);
                __syncthreads();
                staged = true;
            }
            // this warp's share of the chunk
            const uint32_t per = (cn + KS - 1) / KS;
            const uint32_t b_lo = min(ks * per, cn), b_hi = min(b_lo + per, cn);
            for (uint32_t bb = b_lo; bb < b_hi; bb += U) {
                uint32_t wa[U][Q8 ? 2 : 1], wb[U][Q8 ? 2 : 1];
                float da[U], db[U], ma[U], mb[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const uint32_t b = c0 + min(bb + u, b_hi - 1);  // clamp; clamped copies get scale 0 below
                    const bool live = bb + u < b_hi;
                    wa[u][0] = __ldg(reinterpret_cast<const uint32_t*>(qa + (size_t)b * QB));
                    wb[u][0] = __ldg(reinterpret_cast<const uint32_t*>(qb + (size_t)b * QB));
                    if (Q8) {
                        wa[u][Q8 ? 1 : 0] = __ldg(reinterpret_cast<const uint32_t*>(qa + (size_t)b * QB + 16));
                        wb[u][Q8 ? 1 : 0] = __ldg(reinterpret_cast<const uint32_t*>(qb + (size_t)b * QB + 16));
                    }
                    if (Q41) {
                        const __half2 sa = __ldg(reinterpret_cast<const __half2*>(sc) + (size_t)row_a * nb + b);
                        const __half2 sb = __ldg(reinterpret_cast<const __half2*>(sc) + (size_t)row_b * nb + b);
                        da[u] = live ? __low2float(sa) : 0.0f;
                        ma[u] = live ? __high2float(sa) : 0.0f;
                        db[u] = live ? __low2float(sb) : 0.0f;
                        mb[u] = live ? __high2float(sb) : 0.0f;
                    } else {
                        const __half sa = __ldg(reinterpret_cast<const __half*>(sc) + (size_t)row_a * nb + b);
                        const __half sb = __ldg(reinterpret_cast<const __half*>(sc) + (size_t)row_b * nb + b);
                        da[u] = live ? __half2float(sa) : 0.0f;
                        db[u] = live ? __half2float(sb) : 0.0f;
                        ma[u] = mb[u] = 0.0f;
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const uint32_t bl = min(bb + u, b_hi - 1);  // block index inside the chunk
                    uint32_t a_lo[4], a_hi[4];
                    if (Q8) {
                        unpack_q8(wa[u][0], a_lo[0], a_lo[2]);
                        unpack_q8(wb[u][0], a_lo[1], a_lo[3]);
                        unpack_q8(wa[u][Q8 ? 1 : 0], a_hi[0], a_hi[2]);
                        unpack_q8(wb[u][Q8 ? 1 : 0], a_hi[1], a_hi[3]);
                    } else {
                        unpack_q4<Q41 ? 0 : 8>(wa[u][0], a_lo[0], a_lo[2], a_hi[0], a_hi[2]);
                        unpack_q4<Q41 ? 0 : 8>(wb[u][0], a_lo[1], a_lo[3], a_hi[1], a_hi[3]);
                    }
#pragma unroll
                    for (int s = 0; s < NS; ++s) {
                        const uint4 bf = frag[((size_t)bl * NS + s) * 32 + lane];
                        const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        float d1[4], d2[4];
                        mma_f16(d1, a_lo, bf.x, bf.y, zero);
                        mma_f16(d2, a_hi, bf.z, bf.w, d1);
                        acc[s][0] = fmaf(d2[0], da[u], acc[s][0]);
                        acc[s][1] = fmaf(d2[1], da[u], acc[s][1]);
                        acc[s][2] = fmaf(d2[2], db[u], acc[s][2]);
                        acc[s][3] = fmaf(d2[3], db[u], acc[s][3]);
                        if (Q41) {
                            const float xs_m = xsum[bl * 16 + 4 * s + t];
                            accm[s][0] = fmaf(ma[u], xs_m, accm[s][0]);
                            accm[s][1] = fmaf(mb[u], xs_m, accm[s][1]);
                        }
                    }
                }
            }
        }

        // hi + lo columns -> one value per (row, activation row); lane (g, t) of set s owns
        // activation row 4s + t for weight rows g and g + 8.
        float out_a[NS], out_b[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            out_a[s] = acc[s][0] + acc[s][1] + accm[s][0];
            out_b[s] = acc[s][2] + acc[s][3] + accm[s][1];
        }
        if (KS > 1) {
            __syncthreads();  // staging buffer of the last chunk is no longer read (red is separate)
            float* mine = red + ((size_t)(wr * KS + ks) * NS * 2) * 32;
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                mine[(s * 2 + 0) * 32 + lane] = out_a[s];
                mine[(s * 2 + 1) * 32 + lane] = out_b[s];
            }
            __syncthreads();
            if (ks == 0) {
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    float sa = 0.0f, sb = 0.0f;
                    for (uint32_t k2 = 0; k2 < KS; ++k2) {
                        const float* other = red + ((size_t)(wr * KS + k2) * NS * 2) * 32;
                        sa += other[(s * 2 + 0) * 32 + lane];
                        sb += other[(s * 2 + 1) * 32 + lane];
                    }
                    out_a[s] = sa;
                    out_b[s] = sb;
                }
            }
        }
        if (ks == 0) {
            const uint32_t r0 = (uint32_t)(tile * rows_per_cta) + wr * 16 + g;
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                const uint32_t m = 4 * s + t;
                if (m < M) {
                    const float ps = post[m];
                    if (r0 < N)
                        y[(size_t)m * N + r0] = apply_epilogue(out_a[s] * ps, ep, r0, (size_t)m * N + r0);
                    if (r0 + 8 < N)
                        y[(size_t)m * N + r0 + 8] =
                            apply_epilogue(out_b[s] * ps, ep, r0 + 8, (size_t)m * N + r0 + 8);
                }
            }
        }
        if (KS > 1) __syncthreads();  // red is reused by the next tile
    }
}

struct Plan {
    uint32_t WR, KS, kc, grid;
    size_t smem;
};

// Chooses the CTA shape: enough warps in flight on every SM, K split across warps only when there
// are too few row tiles to do that with one warp per tile.
Plan make_plan(const zq_weight* w, int ns, bool q41) {
    Plan p;
    const uint32_t tiles = (w->out_dim + 15) / 16;
    const uint32_t sms = (uint32_t)sm_count();
    const uint32_t want_warps = sms * 16;
    uint32_t ks = 1;
    while (ks < 8 && tiles * ks < want_warps && w->nb / (ks * 2) >= 4) ks *= 2;
    // 8 warps per CTA, fewer when that would leave SMs without a CTA
    uint32_t warps = 8;
    while (warps > ks && (tiles + warps / ks - 1) / (warps / ks) < sms) warps /= 2;
    uint32_t wr = warps / ks;
    if (wr == 0) wr = 1;
    p.WR = wr;
    p.KS = ks;
    const size_t per_block = (size_t)ns * 32 * 16 + (q41 ? 64 : 0);
    const size_t red = ks > 1 ? (size_t)wr * ks * ns * 2 * 32 * 4 : 0;
    const size_t budget = 64 * 1024;  // keeps several CTAs resident per SM
    uint32_t kc = w->nb;
    if ((size_t)kc * per_block + red > budget) kc = (uint32_t)((budget - red) / per_block);
    if (kc < 1) kc = 1;
    p.kc = kc;
    p.smem = (size_t)kc * per_block + red;
    const uint32_t cta_tiles = (tiles + wr - 1) / wr;
    const uint32_t cap = sms * 4;
    p.grid = cta_tiles < cap ? cta_tiles : cap;
    return p;
}

template <int TYPE, int NS>
int launch_one(const zq_weight* w, const float* x, float* y, uint32_t M, EpilogueArgs ep, cudaStream_t st) {
    const Plan p = make_plan(w, NS, TYPE == ZQ_TYPE_Q4_1);
    auto kern = gemv_mma_kernel<TYPE, NS, 4>;
    if (p.smem > 48 * 1024)
        ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem));
    kern<<<p.grid, p.WR * p.KS * 32, p.smem, st>>>(w->qs, w->sc, x, y, w->out_dim, w->in_dim, w->nb, M, p.kc,
                                                    p.WR, p.KS, ep);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

template <int TYPE>
int launch_ns(const zq_weight* w, const float* x, float* y, uint32_t M, EpilogueArgs ep, cudaStream_t st) {
    switch ((M + 3) / 4) {
        case 1: return launch_one<TYPE, 1>(w, x, y, M, ep, st);
        case 2: return launch_one<TYPE, 2>(w, x, y, M, ep, st);
        case 3: return launch_one<TYPE, 3>(w, x, y, M, ep, st);
        default: return launch_one<TYPE, 4>(w, x, y, M, ep, st);
    }
}

}  // namespace

// y[m][j] for m < m_rows <= 16. Epilogue pointers `mul` / `residual` are indexed [m][j].
int launch_gemv_mma_f32(const zq_weight* w, const float* x, float* y, uint32_t m_rows,
                        const zq_epilogue* ep, cudaStream_t st) {
    if (m_rows == 0) return ZQ_OK;
    if (m_rows > 4 * kMaxCols) return ZQ_ERR_BAD_ARG;
    if (((uintptr_t)x & 15) != 0) return ZQ_ERR_BAD_ARG;  // activation rows are read as float4
    EpilogueArgs a{nullptr, nullptr, nullptr, 0};
    if (ep) {
        a.bias = ep->d_bias;
        a.gelu = ep->gelu;
        a.mul = ep->d_mul;
        a.residual = ep->d_residual;
    }
    switch (w->type) {
        case ZQ_TYPE_Q4_0: return launch_ns<ZQ_TYPE_Q4_0>(w, x, y, m_rows, a, st);
        case ZQ_TYPE_Q4_1: return launch_ns<ZQ_TYPE_Q4_1>(w, x, y, m_rows, a, st);
        case ZQ_TYPE_Q8_0: return launch_ns<ZQ_TYPE_Q8_0>(w, x, y, m_rows, a, st);
        default: return ZQ_ERR_UNSUPPORTED;
    }
}

}  // namespace zq
