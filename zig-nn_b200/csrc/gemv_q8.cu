// Q8-activation decode GEMV: int8 activations (quantize_row_q8), exact int32 block dots with dp4a,
// block terms (d*s)*float(idot) [+ (m*s)*float(qsum)] added in block order — the arithmetic of
// zig-nn's ThreadPool.matmul (src/gguf/thread_pool.zig:96-181 -> src/gguf/simd_dot.zig:71-152), so the
// outputs are bit-identical to that CPU path.
//
// Mapping (g = lane / 4, t = lane % 4). A warp owns 16 rows; lane (g, t) works on rows g and g + 8.
// The device layout interleaves each group of 4 blocks (a quad) so that word t of the 4 blocks is 16
// contiguous bytes: one 128-bit load gives the lane 8 weights of each of the 4 blocks. The lane forms
// 4 partial integer dots; a 3-shuffle transpose-reduce inside the 4 lanes leaves the complete dot of
// block 4q + t in lane t. That lane applies the block's scales and stores the f32 term to shared
// memory. When every block of a row has its term, one lane adds them in block order. Because only
// the terms (not partial sums) cross warps, K can be split over warps without changing a single bit.
#include "zq_internal.h"

namespace zq {
namespace {

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

__device__ __forceinline__ float apply_epilogue(float v, const EpilogueArgs& ep, size_t j) {
    if (ep.bias) v = __fadd_rn(v, ep.bias[j]);
    if (ep.gelu) v = gelu_tanh(v);
    if (ep.mul) v = __fmul_rn(v, ep.mul[j]);
    if (ep.residual) v = __fadd_rn(ep.residual[j], v);
    return v;
}

__device__ __forceinline__ uint32_t pick(const uint4& v, int j) {
    return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w;
}

// Four partial dots p[j] (block j of the quad) held by each of the 4 lanes of a quad ->
// the sum over the 4 lanes of p[t], delivered to lane t. Integer adds: exact in any order.
__device__ __forceinline__ int quad_transpose_reduce(const int (&p)[4], int t) {
    const bool upper = t & 2;
    // lanes 0,1 keep blocks 0,1 and hand over 2,3; lanes 2,3 the other way round
    const int keep0 = upper ? p[2] : p[0], keep1 = upper ? p[3] : p[1];
    const int send0 = upper ? p[0] : p[2], send1 = upper ? p[1] : p[3];
    const int a0 = keep0 + __shfl_xor_sync(0xFFFFFFFFu, send0, 2);
    const int a1 = keep1 + __shfl_xor_sync(0xFFFFFFFFu, send1, 2);
    const bool odd = t & 1;
    const int keep = odd ? a1 : a0, send = odd ? a0 : a1;
    return keep + __shfl_xor_sync(0xFFFFFFFFu, send, 1);
}

// smem: xl[nq][4] uint4 | xh[nq][4] uint4 | xs[nbp] f32 | xsum[nbp] i32 | terms[WR][16][pitch] f32
template <int TYPE>
__global__ void __launch_bounds__(512)
gemv_q8_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ sc, const int8_t* __restrict__ xq,
               const float* __restrict__ xscale, const int32_t* __restrict__ xqsum, float* __restrict__ y,
               uint32_t N, uint32_t nb, uint32_t scp, uint32_t WR, uint32_t KS, int prefetch, EpilogueArgs ep) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QB = Q8 ? 32 : 16;
    constexpr uint32_t QUAD = 4 * QB;

    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint32_t nbp = (nb + 3u) & ~3u, nq = nbp / 4;
    const uint32_t pitch = nbp + 1;  // odd pitch: the 16 rows of a tile fall in different banks
    uint4* xl = reinterpret_cast<uint4*>(smem_raw);
    uint4* xh = xl + (size_t)nq * 4;
    float* xs = reinterpret_cast<float*>(xh + (size_t)nq * 4);
    int32_t* xsum = reinterpret_cast<int32_t*>(xs + nbp);
    float* terms = reinterpret_cast<float*>(xsum + nbp);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t wr = warp % WR, ks = warp / WR;

    // The weights do not depend on the kernel that produces the activations: let the next kernel be
    // scheduled, ask L2 for this CTA's rows, and only then wait for the activations.
    pdl_launch_dependents();
    if (prefetch) {
        const uint32_t rows_cta = WR * 16;
        const size_t row_bytes = (size_t)nbp * QB, sc_row_bytes = (size_t)scp * (Q41 ? 4 : 2);
        constexpr uint32_t kChunk = 8192;
        for (uint64_t tile = blockIdx.x; tile * rows_cta < N; tile += gridDim.x) {
            const uint32_t row0 = (uint32_t)(tile * rows_cta);
            const uint32_t rows = min(rows_cta, N - row0);
            const size_t qbytes = rows * row_bytes, sbytes = rows * sc_row_bytes;
            const uint8_t* qp = qs + (size_t)row0 * row_bytes;
            const uint8_t* sp = sc + (size_t)row0 * sc_row_bytes;
            for (size_t off = (size_t)tid * kChunk; off < qbytes; off += (size_t)blockDim.x * kChunk)
                prefetch_l2_bulk(qp + off, (uint32_t)min((size_t)kChunk, qbytes - off));
            for (size_t off = (size_t)tid * kChunk; off < sbytes; off += (size_t)blockDim.x * kChunk)
                prefetch_l2_bulk(sp + off, (uint32_t)min((size_t)kChunk, sbytes - off));
        }
    }
    pdl_wait();

    // Activation image: word w of block b goes to xl/xh[b/4][w%4] component b%4 (xl: w < 4, xh: w >= 4),
    // the same interleave as the weights. Blocks past nb (row padding) are zero with scale 1.
    {
        const uint32_t* xw = reinterpret_cast<const uint32_t*>(xq);
        uint32_t* xl32 = reinterpret_cast<uint32_t*>(xl);
        uint32_t* xh32 = reinterpret_cast<uint32_t*>(xh);
        for (uint32_t i = tid; i < nbp * 8; i += blockDim.x) {
            const uint32_t b = i >> 3, w = i & 7u;
            const uint32_t v = b < nb ? xw[i] : 0u;
            uint32_t* dst = w < 4 ? xl32 : xh32;
            dst[((b >> 2) * 4 + (w & 3u)) * 4 + (b & 3u)] = v;
        }
        for (uint32_t b = tid; b < nbp; b += blockDim.x) {
            xs[b] = b < nb ? xscale[b] : 1.0f;
            xsum[b] = b < nb ? xqsum[b] : 0;
        }
    }
    __syncthreads();

    const uint32_t per = (nq + KS - 1) / KS;
    const uint32_t q_lo = min(ks * per, nq), q_hi = min(q_lo + per, nq);
    const uint32_t rows_per_cta = WR * 16;
    float* my_terms = terms + (size_t)wr * 16 * pitch;

    for (uint64_t tile = blockIdx.x; tile * rows_per_cta < N; tile += gridDim.x) {
        const uint32_t r0 = (uint32_t)(tile * rows_per_cta) + wr * 16;
        const uint32_t row_a = min(r0 + g, N - 1), row_b = min(r0 + g + 8, N - 1);
        const uint8_t* pa = qs + (size_t)row_a * nbp * QB + 16 * t;
        const uint8_t* pb = qs + (size_t)row_b * nbp * QB + 16 * t;
        const uint8_t* sa = sc + (size_t)row_a * scp * (Q41 ? 4 : 2);
        const uint8_t* sb = sc + (size_t)row_b * scp * (Q41 ? 4 : 2);

#pragma unroll 4
        for (uint32_t q = q_lo; q < q_hi; ++q) {
            const uint4 wa = __ldg(reinterpret_cast<const uint4*>(pa + (size_t)q * QUAD));
            const uint4 wb = __ldg(reinterpret_cast<const uint4*>(pb + (size_t)q * QUAD));
            uint4 wa2 = wa, wb2 = wb;
            if (Q8) {
                wa2 = __ldg(reinterpret_cast<const uint4*>(pa + (size_t)q * QUAD + 64));
                wb2 = __ldg(reinterpret_cast<const uint4*>(pb + (size_t)q * QUAD + 64));
            }
            const uint32_t blk = q * 4 + t;  // the block whose complete dot ends up in this lane
            float da, db, ma = 0.0f, mb = 0.0f;
            if (Q41) {
                const __half2 ha = __ldg(reinterpret_cast<const __half2*>(sa) + blk);
                const __half2 hb = __ldg(reinterpret_cast<const __half2*>(sb) + blk);
                da = __low2float(ha); ma = __high2float(ha);
                db = __low2float(hb); mb = __high2float(hb);
            } else {
                da = __half2float(__ldg(reinterpret_cast<const __half*>(sa) + blk));
                db = __half2float(__ldg(reinterpret_cast<const __half*>(sb) + blk));
            }
            const uint4 xlo = xl[q * 4 + t], xhi = xh[q * 4 + t];
            int pa4[4], pb4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int x0 = (int)pick(xlo, j), x1 = (int)pick(xhi, j);
                if (Q8) {
                    pa4[j] = __dp4a((int)pick(wa2, j), x1, __dp4a((int)pick(wa, j), x0, 0));
                    pb4[j] = __dp4a((int)pick(wb2, j), x1, __dp4a((int)pick(wb, j), x0, 0));
                } else {
                    const uint32_t ua = pick(wa, j), ub = pick(wb, j);
                    pa4[j] = __dp4a((int)((ua >> 4) & 0x0F0F0F0Fu), x1, __dp4a((int)(ua & 0x0F0F0F0Fu), x0, 0));
                    pb4[j] = __dp4a((int)((ub >> 4) & 0x0F0F0F0Fu), x1, __dp4a((int)(ub & 0x0F0F0F0Fu), x0, 0));
                }
            }
            int ia = quad_transpose_reduce(pa4, t), ib = quad_transpose_reduce(pb4, t);
            const float s = xs[blk];
            const int qsum = xsum[blk];
            float ta, tb;
            if (TYPE == ZQ_TYPE_Q4_0) {
                ia -= 8 * qsum;  // sum((n-8)*q) = sum(n*q) - 8*sum(q), exact
                ib -= 8 * qsum;
            }
            ta = __fmul_rn(__fmul_rn(da, s), (float)ia);
            tb = __fmul_rn(__fmul_rn(db, s), (float)ib);
            if (Q41) {
                ta = __fadd_rn(ta, __fmul_rn(__fmul_rn(ma, s), (float)qsum));
                tb = __fadd_rn(tb, __fmul_rn(__fmul_rn(mb, s), (float)qsum));
            }
            my_terms[g * pitch + blk] = ta;
            my_terms[(g + 8) * pitch + blk] = tb;
        }
        if (KS > 1) __syncthreads(); else __syncwarp();

        // one lane per row adds the row's terms in block order, as the CPU loop does
        if (ks == 0 && lane < 16) {
            const float* tr = my_terms + lane * pitch;
            float run = 0.0f;
            uint32_t b = 0;
            for (; b + 4 <= nb; b += 4) {
                const float t0 = tr[b], t1 = tr[b + 1], t2 = tr[b + 2], t3 = tr[b + 3];
                run = __fadd_rn(run, t0); run = __fadd_rn(run, t1);
                run = __fadd_rn(run, t2); run = __fadd_rn(run, t3);
            }
            for (; b < nb; ++b) run = __fadd_rn(run, tr[b]);
            const uint32_t row = r0 + lane;
            if (row < N) y[row] = apply_epilogue(run, ep, row);
        }
        if (KS > 1) __syncthreads(); else __syncwarp();  // terms are rewritten by the next tile
    }
}

// ---- whole rows per warp, for matrices with many row tiles ------------------------------------------
// Same arithmetic, another data path: a warp owns 16 rows and all their blocks, its quant words stream
// through a per-lane cp.async ring (data in flight sits in shared memory; a warp has only six load
// scoreboards, so register prefetch cannot go deep), and the scales of a 16-row tile — contiguous in
// memory — are copied once per tile into a per-warp buffer. The kernel above is latency-bound on the
// 170-320 MB vocabulary head (two quads of loads in flight per lane); this one keeps D - 1 quads in
// flight per lane.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint32_t v;
    asm volatile("{\n\t.reg .u16 h;\n\tld.shared.u16 h, [%1];\n\tcvt.u32.u16 %0, h;\n\t}" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

constexpr int kRowsWarps = 8;
constexpr int kRowsDepth = 4;

// smem: xl[nq][4] uint4 | xh[nq][4] uint4 | xs[nbp] f32 | xsum[nbp] i32 | terms[W][16][pitch] f32 |
//       scale tiles [W][2][16 rows][scp * SB] | ring [W][D][stage]
template <int TYPE>
__global__ void __launch_bounds__(kRowsWarps * 32, 2)
gemv_q8_rows_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ sc, const int8_t* __restrict__ xq,
                    const float* __restrict__ xscale, const int32_t* __restrict__ xqsum, float* __restrict__ y,
                    uint32_t N, uint32_t nb, uint32_t scp, uint32_t sc_off, uint32_t ring_off, EpilogueArgs ep) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QB = Q8 ? 32 : 16;
    constexpr uint32_t QUAD = 4 * QB;
    constexpr uint32_t SB = Q41 ? 4 : 2;
    constexpr int D = kRowsDepth;
    constexpr uint32_t kStage = Q8 ? 2048 : 1024;
    constexpr uint32_t rows_per_cta = kRowsWarps * 16;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t nbp = (nb + 3u) & ~3u, nq = nbp / 4;
    const uint32_t pitch = nbp + 1;
    uint4* xl = reinterpret_cast<uint4*>(smem_raw);
    uint4* xh = xl + (size_t)nq * 4;
    float* xs = reinterpret_cast<float*>(xh + (size_t)nq * 4);
    int32_t* xsum = reinterpret_cast<int32_t*>(xs + nbp);
    float* terms = reinterpret_cast<float*>(xsum + nbp);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    float* my_terms = terms + (size_t)warp * 16 * pitch;

    pdl_launch_dependents();

    const uint32_t sc_row_bytes = scp * SB;
    const uint32_t sc_tile_bytes = 16 * sc_row_bytes;
    const uint32_t sbuf32 = (uint32_t)__cvta_generic_to_shared(smem_raw + sc_off) + warp * 2 * sc_tile_bytes;
    const uint32_t ring32 = (uint32_t)__cvta_generic_to_shared(smem_raw + ring_off) + warp * D * kStage + lane * 16;

    // ---- producer: the quads of this warp's tiles, in order, D - 1 ahead of the consumer; group n holds
    //      quad n of the warp's sequence (plus, with the last quad of a tile, the next tile's scales) ----
    uint64_t p_tile = blockIdx.x;
    uint32_t p_q = 0, p_par = 0, p_slot = 0;
    const uint8_t *p_pa = qs, *p_pb = qs;
    auto producer_set_tile = [&]() {
        if (p_tile * rows_per_cta < N) {
            const uint32_t r0 = (uint32_t)(p_tile * rows_per_cta) + warp * 16;
            const uint32_t r = r0 + g;
            const uint32_t row_a = min(r, N - 1), row_b = min(r + 8, N - 1);
            p_pa = qs + (size_t)row_a * nbp * QB + 16 * t;
            p_pb = qs + (size_t)row_b * nbp * QB + 16 * t;
            if (r0 < N) {
                const uint32_t bytes = min(16u, N - r0) * sc_row_bytes;
                const uint8_t* src = sc + (size_t)r0 * sc_row_bytes;
                const uint32_t dst = sbuf32 + p_par * sc_tile_bytes;
                for (uint32_t o = lane * 16; o < bytes; o += 32 * 16) cp_async16(dst + o, src + o);
            }
            p_par ^= 1u;
        }
    };
    auto producer_step = [&]() {
        if (p_tile * rows_per_cta < N) {
            const uint32_t stage = ring32 + p_slot * kStage;
            cp_async16(stage, p_pa);
            cp_async16(stage + 512, p_pb);
            if (Q8) {
                cp_async16(stage + 1024, p_pa + 64);
                cp_async16(stage + 1536, p_pb + 64);
            }
            p_slot = p_slot + 1 == (uint32_t)D ? 0 : p_slot + 1;
            if (++p_q == nq) {
                p_q = 0;
                p_tile += gridDim.x;
                producer_set_tile();
            } else {
                p_pa += QUAD; p_pb += QUAD;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    producer_set_tile();
#pragma unroll 1
    for (int i = 0; i < D - 1; ++i) producer_step();
    uint32_t c_slot = 0;

    // The weights do not depend on the kernel that produces the activations; the activations do.
    pdl_wait();
    {
        const uint32_t* xw = reinterpret_cast<const uint32_t*>(xq);
        uint32_t* xl32 = reinterpret_cast<uint32_t*>(xl);
        uint32_t* xh32 = reinterpret_cast<uint32_t*>(xh);
        for (uint32_t i = tid; i < nbp * 8; i += blockDim.x) {
            const uint32_t b = i >> 3, w = i & 7u;
            const uint32_t v = b < nb ? xw[i] : 0u;
            uint32_t* dst = w < 4 ? xl32 : xh32;
            dst[((b >> 2) * 4 + (w & 3u)) * 4 + (b & 3u)] = v;
        }
        for (uint32_t b = tid; b < nbp; b += blockDim.x) {
            xs[b] = b < nb ? xscale[b] : 1.0f;
            xsum[b] = b < nb ? xqsum[b] : 0;
        }
    }
    __syncthreads();

    uint64_t c_tile = blockIdx.x;
    uint32_t c_q = 0, c_par = 0;
    const uint32_t sc_lane = g * sc_row_bytes + t * SB;
    uint32_t saddr = sbuf32 + sc_lane;

#pragma unroll 1
    while (c_tile * rows_per_cta < N) {
        producer_step();
        asm volatile("cp.async.wait_group %0;" ::"n"(D - 1) : "memory");
        __syncwarp();
        const uint32_t stage = ring32 + c_slot * kStage;
        const uint4 wa = lds128(stage), wb = lds128(stage + 512);
        uint4 wa2 = wa, wb2 = wb;
        if (Q8) {
            wa2 = lds128(stage + 1024);
            wb2 = lds128(stage + 1536);
        }
        c_slot = c_slot + 1 == (uint32_t)D ? 0 : c_slot + 1;

        const uint32_t q = c_q, blk = q * 4 + t;  // the block whose complete dot ends up in this lane
        float da, db, ma = 0.0f, mb = 0.0f;
        if (Q41) {
            const uint32_t ua = lds_u32(saddr), ub = lds_u32(saddr + 8 * sc_row_bytes);
            const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&ua));
            const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&ub));
            da = fa.x; ma = fa.y;
            db = fb.x; mb = fb.y;
        } else {
            da = __half2float(__ushort_as_half((unsigned short)lds_u16(saddr)));
            db = __half2float(__ushort_as_half((unsigned short)lds_u16(saddr + 8 * sc_row_bytes)));
        }
        const uint4 xlo = xl[q * 4 + t], xhi = xh[q * 4 + t];
        int pa4[4], pb4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int x0 = (int)pick(xlo, j), x1 = (int)pick(xhi, j);
            if (Q8) {
                pa4[j] = __dp4a((int)pick(wa2, j), x1, __dp4a((int)pick(wa, j), x0, 0));
                pb4[j] = __dp4a((int)pick(wb2, j), x1, __dp4a((int)pick(wb, j), x0, 0));
            } else {
                const uint32_t ua = pick(wa, j), ub = pick(wb, j);
                pa4[j] = __dp4a((int)((ua >> 4) & 0x0F0F0F0Fu), x1, __dp4a((int)(ua & 0x0F0F0F0Fu), x0, 0));
                pb4[j] = __dp4a((int)((ub >> 4) & 0x0F0F0F0Fu), x1, __dp4a((int)(ub & 0x0F0F0F0Fu), x0, 0));
            }
        }
        int ia = quad_transpose_reduce(pa4, t), ib = quad_transpose_reduce(pb4, t);
        const float s = xs[blk];
        const int qsum = xsum[blk];
        if (TYPE == ZQ_TYPE_Q4_0) {
            ia -= 8 * qsum;
            ib -= 8 * qsum;
        }
        float ta = __fmul_rn(__fmul_rn(da, s), (float)ia);
        float tb = __fmul_rn(__fmul_rn(db, s), (float)ib);
        if (Q41) {
            ta = __fadd_rn(ta, __fmul_rn(__fmul_rn(ma, s), (float)qsum));
            tb = __fadd_rn(tb, __fmul_rn(__fmul_rn(mb, s), (float)qsum));
        }
        my_terms[g * pitch + blk] = ta;
        my_terms[(g + 8) * pitch + blk] = tb;
        saddr += 4 * SB;

        if (++c_q == nq) {
            __syncwarp();
            // one lane per row adds the row's terms in block order, as the CPU loop does
            if (lane < 16) {
                const float* tr = my_terms + lane * pitch;
                float run = 0.0f;
                uint32_t b = 0;
                for (; b + 4 <= nb; b += 4) {
                    const float t0 = tr[b], t1 = tr[b + 1], t2 = tr[b + 2], t3 = tr[b + 3];
                    run = __fadd_rn(run, t0); run = __fadd_rn(run, t1);
                    run = __fadd_rn(run, t2); run = __fadd_rn(run, t3);
                }
                for (; b < nb; ++b) run = __fadd_rn(run, tr[b]);
                const uint32_t row = (uint32_t)(c_tile * rows_per_cta) + warp * 16 + lane;
                if (row < N) y[row] = apply_epilogue(run, ep, row);
            }
            __syncwarp();  // terms are rewritten by the next tile
            c_q = 0;
            c_tile += gridDim.x;
            c_par ^= 1u;
            saddr = sbuf32 + c_par * sc_tile_bytes + sc_lane;
        }
    }
}

template <int TYPE>
int launch_rows(const zq_weight* w, const int8_t* xq, const float* xs, const int32_t* xsum, float* y,
                EpilogueArgs ep, cudaStream_t st) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    const uint32_t sms = (uint32_t)sm_count();
    const uint32_t nq = w->nbp / 4;
    if (nq < (uint32_t)kRowsDepth) return ZQ_ERR_LIMIT;  // the producer must stay within one tile of the consumer
    size_t smem = (size_t)nq * 4 * 16 * 2 + (size_t)w->nbp * 8;
    smem += (size_t)kRowsWarps * 16 * (w->nbp + 1) * sizeof(float);
    smem = (smem + 127) & ~(size_t)127;
    const uint32_t sc_off = (uint32_t)smem;
    smem += (size_t)kRowsWarps * 2 * 16 * w->scp * (Q41 ? 4 : 2);
    smem = (smem + 127) & ~(size_t)127;
    const uint32_t ring_off = (uint32_t)smem;
    smem += (size_t)kRowsWarps * kRowsDepth * (Q8 ? 2048 : 1024);
    if (smem > (size_t)(227 * 1024) / 2 - 1024) return ZQ_ERR_LIMIT;  // two CTAs per SM
    auto kern = gemv_q8_rows_kernel<TYPE>;
    if (smem > 48 * 1024)
        ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const uint32_t cta_tiles = (w->out_dim + kRowsWarps * 16 - 1) / (kRowsWarps * 16);
    const uint32_t cap = sms * 2;
    ZQ_CUDA(launch_pdl(kern, dim3(cta_tiles < cap ? cta_tiles : cap), dim3(kRowsWarps * 32), smem, st, w->qs,
                       static_cast<const uint8_t*>(w->sc), xq, xs, xsum, y, w->out_dim, w->nb, w->scp, sc_off,
                       ring_off, ep));
    return ZQ_OK;
}

template <int TYPE>
int launch_one(const zq_weight* w, const int8_t* xq, const float* xs, const int32_t* xsum, float* y,
               EpilogueArgs ep, cudaStream_t st) {
    const uint32_t tiles = (w->out_dim + 15) / 16;
    const uint32_t sms = (uint32_t)sm_count();
    const uint32_t nq = w->nbp / 4;
    if (tiles >= sms * 2 * kRowsWarps) {  // enough row tiles for whole rows per warp: the ring kernel
        const int rc = launch_rows<TYPE>(w, xq, xs, xsum, y, ep, st);
        if (rc != ZQ_ERR_LIMIT) return rc;
    }
    // Small matrices are latency-bound: split K over up to 16 warps so that every load of a row tile is
    // in flight at once; large ones keep whole rows per warp.
    uint32_t ks = 1;
    while (ks < 16 && tiles * ks < sms * 16 && nq >= ks * 2) ks *= 2;
    uint32_t warps = ks > 8 ? ks : 8;
    while (warps > ks && (tiles + warps / ks - 1) / (warps / ks) < sms) warps /= 2;
    uint32_t wr = warps / ks ? warps / ks : 1;
    const size_t fixed = (size_t)nq * 4 * 16 * 2 + (size_t)w->nbp * 8;
    auto smem_for = [&](uint32_t r) { return fixed + (size_t)r * 16 * (w->nbp + 1) * sizeof(float); };
    while (wr > 1 && smem_for(wr) > 96 * 1024) wr /= 2;
    const size_t smem = smem_for(wr);
    if (smem > 200 * 1024) return ZQ_ERR_LIMIT;
    auto kern = gemv_q8_kernel<TYPE>;
    if (smem > 48 * 1024)
        ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const uint32_t cta_tiles = (tiles + wr - 1) / wr;
    uint32_t per_sm = (uint32_t)((200 * 1024) / (smem + 1024));
    if (per_sm > 4) per_sm = 4;
    if (per_sm < 1) per_sm = 1;
    const uint32_t cap = sms * per_sm;
    // prefetching pays when the whole matrix can sit in L2 next to its neighbours in the step
    const int prefetch = w->bytes <= (size_t)48 << 20;
    ZQ_CUDA(launch_pdl(kern, dim3(cta_tiles < cap ? cta_tiles : cap), dim3(wr * ks * 32), smem, st, w->qs,
                       static_cast<const uint8_t*>(w->sc), xq, xs, xsum, y, w->out_dim, w->nb, w->scp, wr, ks,
                       prefetch, ep));
    return ZQ_OK;
}

}  // namespace

int launch_gemv_q8(const zq_weight* w, const int8_t* xq, const float* xscale, const int32_t* xsum,
                   float* y, uint32_t m_rows, const zq_epilogue* ep, cudaStream_t st) {
    for (uint32_t m = 0; m < m_rows; ++m) {
        const size_t yo = (size_t)m * w->out_dim, bo = (size_t)m * w->nb;
        EpilogueArgs a{nullptr, nullptr, nullptr, 0};
        if (ep) {
            a.bias = ep->d_bias;
            a.gelu = ep->gelu;
            a.mul = ep->d_mul ? ep->d_mul + yo : nullptr;
            a.residual = ep->d_residual ? ep->d_residual + yo : nullptr;
        }
        const int8_t* q = xq + (size_t)m * w->in_dim;
        int rc;
        switch (w->type) {
            case ZQ_TYPE_Q4_0: rc = launch_one<ZQ_TYPE_Q4_0>(w, q, xscale + bo, xsum + bo, y + yo, a, st); break;
            case ZQ_TYPE_Q4_1: rc = launch_one<ZQ_TYPE_Q4_1>(w, q, xscale + bo, xsum + bo, y + yo, a, st); break;
            case ZQ_TYPE_Q8_0: rc = launch_one<ZQ_TYPE_Q8_0>(w, q, xscale + bo, xsum + bo, y + yo, a, st); break;
            default: return ZQ_ERR_UNSUPPORTED;
        }
        if (rc != ZQ_OK) return rc;
    }
    return ZQ_OK;
}

}  // namespace zq
