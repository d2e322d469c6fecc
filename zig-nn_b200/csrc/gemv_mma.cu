// f32-activation decode GEMV on the tensor cores (m_rows <= 16).
//
// The integer weights (n-8, n, or the
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
// Fragment ownership (g = lane / 4, t = lane % 4): the thread needs quant word t of every block of
// rows g and g + 8. Word t holds elements 4t..4t+3 (low nibbles) and 16+4t..16+4t+3 (high nibbles),
// which is exactly the K footprint an m16n8k16 A fragment wants from lane (g, t), so no data moves
// between lanes. The device layout interleaves each group of 4 blocks so that those words are 16
// contiguous bytes: one 128-bit load per row brings the thread's share of 4 blocks, and the 4 lanes
// of a quad read 64 contiguous bytes. K slots are assigned as (2t, 2t+1, 2t+8, 2t+9) <- elements
// (4t, 4t+2, 4t+1, 4t+3); the activation fragments in shared memory use the same permutation.
#include "zq_internal.h"

namespace zq {
namespace {

// Per-call options: the output epilogue and, for one activation row, an optional LayerNorm applied to
// the row before the product (ln_gamma != nullptr; two-pass mean / variance as gpt2.zig:541-596).
struct EpilogueArgs {
    const float* bias;
    const float* mul;
    const float* residual;
    int gelu;
    const float* ln_gamma;
    const float* ln_beta;
    float ln_eps;
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
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]),
          "f"(c[3]));
}

__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// One 4-bit quant word -> fp16 pairs (e0, e2), (e1, e3) of the low nibbles and of the high nibbles,
// with no arithmetic at all: a nibble left in the low mantissa bits of an fp16 with exponent field 0
// is the subnormal n * 2^-24 (low nibbles) or n * 2^-20 (high nibbles, bits 4..7). The tensor core
// multiplies subnormals exactly; the high-nibble MMA gets activations pre-divided by 16, so both MMAs
// accumulate sum(n * x) * 2^-24, and the factor 2^24 is applied once to the finished row. The "- 8"
// of q4_0 becomes -8 * d * sum(x) per block, the same form as q4_1's m * sum(x).
__device__ __forceinline__ void unpack_q4(uint32_t q, uint32_t& lo02, uint32_t& lo13, uint32_t& hi02,
                                          uint32_t& hi13) {
    const uint32_t s = q >> 8;
    lo02 = q & 0x000F000Fu;
    hi02 = q & 0x00F000F0u;
    lo13 = s & 0x000F000Fu;
    hi13 = s & 0x00F000F0u;
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

// Shared-memory image of the activations, built once per CTA:
//   frag[block][col][t] (uint4): B registers {low-MMA b0, b1, high-MMA b0, b1} that lane (g, t) feeds
//     for MMA column `col` = 2 * activation row + part (0 = hi, 1 = lo); only the 2*M real columns
//     are stored (lanes of the other columns feed zeros); blocks >= nb (row padding) are zero;
//   xsum[block][M]: f32 sum of each activation row's 32 values (4-bit types).
// `pre[m]` is a power-of-two prescale that brings the row's largest |x| just under 2^14 (undone in the
// epilogue), so that the fp16 parts use the normal range whatever the scale of the activations.
template <bool WITH_SUM, bool HI_DIV16>
__device__ void stage_activations(const float* __restrict__ x, uint32_t M, uint32_t K, uint32_t nb,
                                  uint32_t nbp, const float* pre, uint4* frag, float* xsum) {
    const uint32_t ncols = 2 * M;
    const uint32_t total = nbp * ncols * 4;
    const uint32_t total_up = (total + 31u) & ~31u;  // whole warps run the shuffles below
    constexpr int U = 4;  // entries per thread and round: their loads are all issued before any is used
    for (uint32_t i0 = threadIdx.x; i0 < total_up; i0 += blockDim.x * U) {
        float4 a[U], b[U];
        float s[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t i = i0 + u * blockDim.x;
            const uint32_t ii = i < total ? i : 0;
            const uint32_t t = ii & 3u, col = (ii >> 2) % ncols, blk = (ii >> 2) / ncols;
            const uint32_t m = col >> 1;
            a[u] = b[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            s[u] = 0.0f;
            if (i < total_up && blk < nb) {
                const float* p = x + (size_t)m * K + (size_t)blk * 32u;
                a[u] = *reinterpret_cast<const float4*>(p + 4u * t);
                b[u] = *reinterpret_cast<const float4*>(p + 16u + 4u * t);
                s[u] = pre[m];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t i = i0 + u * blockDim.x;
            if (i >= total_up) break;  // uniform per warp: blockDim.x and total_up are multiples of 32
            const bool active = i < total;
            const uint32_t ii = active ? i : 0;
            const uint32_t t = ii & 3u, col = (ii >> 2) % ncols, blk = (ii >> 2) / ncols;
            const uint32_t m = col >> 1;
            const bool lo_part = col & 1u;
            float v[8];
            v[0] = a[u].x * s[u]; v[1] = a[u].y * s[u]; v[2] = a[u].z * s[u]; v[3] = a[u].w * s[u];
            v[4] = b[u].x * s[u]; v[5] = b[u].y * s[u]; v[6] = b[u].z * s[u]; v[7] = b[u].w * s[u];
            if (WITH_SUM) {
                float s8 = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
                s8 += __shfl_xor_sync(0xFFFFFFFFu, s8, 1);
                s8 += __shfl_xor_sync(0xFFFFFFFFu, s8, 2);
                if (active && !lo_part && t == 0) xsum[blk * M + m] = s8;
            }
            float w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float hi = __half2float(__float2half_rn(v[j]));
                w[j] = lo_part ? (v[j] - hi) : hi;  // x - hi is exact in f32
            }
            if (HI_DIV16) {  // exact: a power of two (tiny parts may round in the subnormal range)
#pragma unroll
                for (int j = 4; j < 8; ++j) w[j] *= 0.0625f;
            }
            if (active)
                frag[i] = make_uint4(pack_half2(w[0], w[2]), pack_half2(w[1], w[3]), pack_half2(w[4], w[6]),
                                     pack_half2(w[5], w[7]));
        }
    }
}

// The quant words and scales one lane needs for one quad (4 blocks) of rows g and g + 8.
template <bool Q8, bool Q41>
struct QuadRegs {
    uint4 a_lo, b_lo;  // word t of blocks 0..3, rows g / g+8
    uint4 a_hi, b_hi;  // q8_0 only: word 4+t
    uint4 sa, sb;      // scales: q4_0/q8_0 use .x,.y (4 x f16); q4_1 all four (4 x (d, m))
};

// ---- per-lane cp.async ring -------------------------------------------------------------------------
// Every lane copies the 16-byte quant pieces and the scales it will need for one quad into its own
// slots of a shared-memory stage and, a few stages later, reads the same slots back. Nothing is
// shared between lanes, so cp.async.wait_group is the only synchronisation, and the data in flight
// sits in shared memory instead of registers.
template <bool Q8, bool Q41>
struct Ring {
    static constexpr uint32_t kQuantArrays = Q8 ? 4 : 2;              // a, b (, a_hi, b_hi): 512 bytes each
    static constexpr uint32_t kScaleOff = kQuantArrays * 512;
    static constexpr uint32_t kScaleArray = Q41 ? 512 : 256;          // 16 or 8 bytes per lane
    static constexpr uint32_t kStage = kScaleOff + 2 * kScaleArray;
    static constexpr int kDepth = 4;  // quads in flight per lane: 3 x (32..64) bytes
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// stage: shared address of the stage for this warp; pointers already offset to this lane's 16 bytes.
template <bool Q8, bool Q41>
__device__ __forceinline__ void ring_issue(uint32_t stage, int lane, const uint8_t* pa, const uint8_t* pb,
                                           const uint8_t* psa, const uint8_t* psb) {
    using R = Ring<Q8, Q41>;
    cp_async16(stage + lane * 16, pa);
    cp_async16(stage + 512 + lane * 16, pb);
    if (Q8) {
        cp_async16(stage + 1024 + lane * 16, pa + 64);
        cp_async16(stage + 1536 + lane * 16, pb + 64);
    }
    if (Q41) {
        cp_async16(stage + R::kScaleOff + lane * 16, psa);
        cp_async16(stage + R::kScaleOff + 512 + lane * 16, psb);
    } else {
        cp_async8(stage + R::kScaleOff + lane * 8, psa);
        cp_async8(stage + R::kScaleOff + 256 + lane * 8, psb);
    }
}

// Direct global -> register load of one quad (alternative to the ring).
template <bool Q8, bool Q41>
__device__ __forceinline__ void load_quad_regs(QuadRegs<Q8, Q41>& r, const uint8_t* pa, const uint8_t* pb,
                                               const uint8_t* psa, const uint8_t* psb) {
    r.a_lo = __ldg(reinterpret_cast<const uint4*>(pa));
    r.b_lo = __ldg(reinterpret_cast<const uint4*>(pb));
    if (Q8) {
        r.a_hi = __ldg(reinterpret_cast<const uint4*>(pa + 64));
        r.b_hi = __ldg(reinterpret_cast<const uint4*>(pb + 64));
    }
    if (Q41) {
        r.sa = __ldg(reinterpret_cast<const uint4*>(psa));
        r.sb = __ldg(reinterpret_cast<const uint4*>(psb));
    } else {
        const uint2 va = __ldg(reinterpret_cast<const uint2*>(psa));
        const uint2 vb = __ldg(reinterpret_cast<const uint2*>(psb));
        r.sa.x = va.x; r.sa.y = va.y;
        r.sb.x = vb.x; r.sb.y = vb.y;
    }
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
template <bool Q8, bool Q41>
__device__ __forceinline__ void ring_read(QuadRegs<Q8, Q41>& r, uint32_t stage, int lane) {
    using R = Ring<Q8, Q41>;
    r.a_lo = lds128(stage + lane * 16);
    r.b_lo = lds128(stage + 512 + lane * 16);
    if (Q8) {
        r.a_hi = lds128(stage + 1024 + lane * 16);
        r.b_hi = lds128(stage + 1536 + lane * 16);
    }
    if (Q41) {
        r.sa = lds128(stage + R::kScaleOff + lane * 16);
        r.sb = lds128(stage + R::kScaleOff + 512 + lane * 16);
    } else {
        const uint2 va = lds64(stage + R::kScaleOff + lane * 8), vb = lds64(stage + R::kScaleOff + 256 + lane * 8);
        r.sa.x = va.x; r.sa.y = va.y;
        r.sb.x = vb.x; r.sb.y = vb.y;
    }
}
// Predicated forms: lanes whose stride is 0 own no column / activation row and read zeros without
// touching shared memory (a warp-wide 128-bit load costs a wavefront per quarter warp that is active).
__device__ __forceinline__ uint4 lds128_if(uint32_t addr, uint32_t pred) {
    uint4 v = make_uint4(0, 0, 0, 0);
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.u32 p, %5, 0;\n\t"
        "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "r"(addr), "r"(pred));
    return v;
}
__device__ __forceinline__ float lds_f32_if(uint32_t addr, uint32_t pred) {
    float v = 0.0f;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.u32 p, %2, 0;\n\t"
        "@p ld.shared.f32 %0, [%1];\n\t}"
        : "+f"(v)
        : "r"(addr), "r"(pred));
    return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t pick(const uint4& v, int j) {
    return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w;
}

__device__ __forceinline__ void unpack_half2(uint32_t v, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
    lo = f.x;
    hi = f.y;
}

// One quad (4 blocks) of rows g and g + 8 against every activation column set.
// faddr[c] / fstride[c]: 32-bit shared address of this lane's B fragment for the quad's first block in
// column set c, and its per-block stride in bytes; lanes whose MMA column carries no activation point
// at a zero slot with stride 0, so the load needs no predicate. xaddr: shared address of
// xsum[first block][4c' + t] terms (q4_1), xstride its per-block stride.
template <int TYPE, int NS>
__device__ __forceinline__ void compute_quad(const QuadRegs<TYPE == ZQ_TYPE_Q8_0, TYPE == ZQ_TYPE_Q4_1>& r,
                                             const uint32_t (&faddr)[NS], const uint32_t (&fstride)[NS],
                                             const uint32_t (&xaddr)[NS], const uint32_t (&xstride)[NS],
                                             float (&acc)[NS][4], float (&accm)[NS][2]) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    const float zero[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float da[4], db[4], ma[4], mb[4];
    if (Q41) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            unpack_half2(pick(r.sa, j), da[j], ma[j]);
            unpack_half2(pick(r.sb, j), db[j], mb[j]);
        }
    } else {
        unpack_half2(r.sa.x, da[0], da[1]);
        unpack_half2(r.sa.y, da[2], da[3]);
        unpack_half2(r.sb.x, db[0], db[1]);
        unpack_half2(r.sb.y, db[2], db[3]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t a_lo[4], a_hi[4];
        if (Q8) {
            unpack_q8(pick(r.a_lo, j), a_lo[0], a_lo[2]);
            unpack_q8(pick(r.b_lo, j), a_lo[1], a_lo[3]);
            unpack_q8(pick(r.a_hi, j), a_hi[0], a_hi[2]);
            unpack_q8(pick(r.b_hi, j), a_hi[1], a_hi[3]);
        } else {
            unpack_q4(pick(r.a_lo, j), a_lo[0], a_lo[2], a_hi[0], a_hi[2]);
            unpack_q4(pick(r.b_lo, j), a_lo[1], a_lo[3], a_hi[1], a_hi[3]);
        }
#pragma unroll
        for (int c = 0; c < NS; ++c) {
            const uint4 bf = lds128_if(faddr[c] + j * fstride[c], fstride[c]);
            float d1[4], d2[4];
            mma_f16(d1, a_lo, bf.x, bf.y, zero);
            mma_f16(d2, a_hi, bf.z, bf.w, d1);
            acc[c][0] = fmaf(d2[0], da[j], acc[c][0]);
            acc[c][1] = fmaf(d2[1], da[j], acc[c][1]);
            acc[c][2] = fmaf(d2[2], db[j], acc[c][2]);
            acc[c][3] = fmaf(d2[3], db[j], acc[c][3]);
            if (!Q8) {  // q4_1: m * sum(x); q4_0: d * sum(x), times -8 at the end
                const float xs_m = lds_f32_if(xaddr[c] + j * xstride[c], xstride[c]);
                accm[c][0] = fmaf(Q41 ? ma[j] : da[j], xs_m, accm[c][0]);
                accm[c][1] = fmaf(Q41 ? mb[j] : db[j], xs_m, accm[c][1]);
            }
        }
    }
}

// Grid-stride over tiles of 16 rows x WR warps; the KS warps that share a row tile split the quads
// of a row and are summed in a fixed order through shared memory.
constexpr int kCtasPerSm = 2;  // more resident warps did not help: the kernel is bound by instruction work

template <int TYPE, int NS, bool USE_RING>
__global__ void __launch_bounds__(256, kCtasPerSm)
gemv_mma_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ sc, const float* __restrict__ x,
                float* __restrict__ y, uint32_t N, uint32_t K, uint32_t nb, uint32_t scp, uint32_t M,
                uint32_t WR, uint32_t KS, uint32_t ring_off, EpilogueArgs ep) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QB = Q8 ? 32 : 16;
    constexpr uint32_t SB = Q41 ? 4 : 2;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float pre[16], post[16];
    __shared__ unsigned int amax_bits[16];

    const uint32_t nbp = (nb + 3u) & ~3u, ncols = 2 * M;
    uint4* frag = reinterpret_cast<uint4*>(smem_raw);                       // nbp * ncols * 4, then one zero slot
    float* xsum = reinterpret_cast<float*>(frag + (size_t)nbp * ncols * 4 + 1);
    float* red = xsum + (!Q8 ? (size_t)nbp * M : 0);  // KS > 1: WR*KS*NS*2*32 floats
    // per-warp cp.async ring, 128-byte aligned, behind everything else (offset passed by the host)
    unsigned char* ring = smem_raw + ring_off;

    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t wr = warp % WR, ks = warp / WR;
    // Warps past WR * KS only help to build the activation image; they own no quads (q_lo == q_hi below)
    // and no output, but keep every barrier of the tile loop.
    const bool helper = (uint32_t)warp >= WR * KS;

    const uint32_t nq = nbp / 4;
    const uint32_t per = (nq + KS - 1) / KS;
    const uint32_t q_lo = min(ks * per, nq), q_hi = min(q_lo + per, nq);
    const uint32_t rows_per_cta = WR * 16;

    // ---- weight stream: producer cursor runs kDepth-1 quads ahead of the consumer, across tiles;
    //      the first copies are issued before the activations are staged so that both overlap ----
    using R = Ring<Q8, Q41>;
    constexpr int D = R::kDepth;
    constexpr uint32_t QUAD = Q8 ? 128 : 64;  // quant bytes of one quad of blocks
    constexpr uint32_t SQ = 4 * SB;           // scale bytes of one quad
    const uint32_t ring32 = (uint32_t)__cvta_generic_to_shared(ring) + warp * D * R::kStage;
    const uint32_t nqw = q_hi - q_lo;  // quads per tile for this warp

    uint64_t p_tile = blockIdx.x;  // producer cursor
    uint32_t p_q = 0, p_slot = 0;
    const uint8_t *p_pa = qs, *p_pb = qs, *p_psa = sc, *p_psb = sc;
    auto producer_set_tile = [&]() {
        const uint32_t r = (uint32_t)(p_tile * rows_per_cta) + wr * 16 + g;
        const uint32_t row_a = min(r, N - 1), row_b = min(r + 8, N - 1);
        p_pa = qs + (size_t)row_a * nbp * QB + 16 * t + (size_t)q_lo * QUAD;
        p_pb = qs + (size_t)row_b * nbp * QB + 16 * t + (size_t)q_lo * QUAD;
        p_psa = sc + (size_t)row_a * scp * SB + (size_t)q_lo * SQ;
        p_psb = sc + (size_t)row_b * scp * SB + (size_t)q_lo * SQ;
    };
    // issues the copies of the next quad (if any is left) and always closes a group, so that group
    // number n holds quad number n of this warp's sequence
    QuadRegs<Q8, Q41> nxt;  // !USE_RING: the quad in flight lives in registers instead
    auto producer_step = [&]() {
        if (nqw != 0 && p_tile * rows_per_cta < N) {
            if (USE_RING) {
                ring_issue<Q8, Q41>(ring32 + p_slot * R::kStage, lane, p_pa, p_pb, p_psa, p_psb);
                p_slot = p_slot + 1 == (uint32_t)D ? 0 : p_slot + 1;
            } else {
                load_quad_regs<Q8, Q41>(nxt, p_pa, p_pb, p_psa, p_psb);
            }
            if (++p_q == nqw) {
                p_q = 0;
                p_tile += gridDim.x;
                producer_set_tile();
            } else {
                p_pa += QUAD; p_pb += QUAD; p_psa += SQ; p_psb += SQ;
            }
        }
        if (USE_RING) cp_async_commit();
    };
    producer_set_tile();
#pragma unroll 1
    for (int i = 0; i < (USE_RING ? D - 1 : 1); ++i) producer_step();
    uint32_t c_slot = 0;

    // Everything above touched only the weights. The activations may come from the kernel before this one.
    pdl_wait();

    // ---- optional LayerNorm of the (single) activation row into shared memory ----
    if (ep.ln_gamma != nullptr) {
        __shared__ float lnred[34];
        float* xln = reinterpret_cast<float*>(smem_raw + ring_off) - ((K + 31u) & ~31u);  // just below the ring
        const int nw = blockDim.x >> 5;
        float sum = 0.0f;
        for (uint32_t i = tid; i < K; i += blockDim.x) sum += x[i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
        if (lane == 0) lnred[warp] = sum;
        __syncthreads();
        if (tid == 0) {
            float t2 = 0.0f;
            for (int w2 = 0; w2 < nw; ++w2) t2 += lnred[w2];
            lnred[32] = t2 / (float)K;
        }
        __syncthreads();
        const float mean = lnred[32];
        float var = 0.0f;
        for (uint32_t i = tid; i < K; i += blockDim.x) {
            const float d = x[i] - mean;
            var = fmaf(d, d, var);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) var += __shfl_xor_sync(0xFFFFFFFFu, var, off);
        __syncthreads();
        if (lane == 0) lnred[warp] = var;
        __syncthreads();
        if (tid == 0) {
            float t2 = 0.0f;
            for (int w2 = 0; w2 < nw; ++w2) t2 += lnred[w2];
            lnred[33] = 1.0f / sqrtf(t2 / (float)K + ep.ln_eps);
        }
        __syncthreads();
        const float inv_std = lnred[33];
        for (uint32_t i = tid; i < K; i += blockDim.x)
            xln[i] = __fadd_rn(__fmul_rn(__fmul_rn(x[i] - mean, inv_std), ep.ln_gamma[i]), ep.ln_beta[i]);
        __syncthreads();
        x = xln;
    }

    // ---- activations: range prescale, then the fp16 hi/lo fragment image ----
    // one warp per activation row, eight 128-bit loads in flight per lane
    for (uint32_t m = warp; m < M; m += blockDim.x >> 5) {
        float amax = 0.0f;
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)m * K);
        const uint32_t n4 = K / 4;
        for (uint32_t i0 = lane; i0 < n4; i0 += 32 * 8) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                v[u] = i0 + 32 * u < n4 ? xr[i0 + 32 * u] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v[u].x), fabsf(v[u].y))), fmaxf(fabsf(v[u].z), fabsf(v[u].w)));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
        if (lane == 0) amax_bits[m] = __float_as_uint(amax);
    }
    __syncthreads();
    if (tid < (int)M) {
        const float amax = __uint_as_float(amax_bits[tid]);
        const int e = row_scale_exponent(amax);
        pre[tid] = ldexpf(1.0f, -e);
        post[tid] = ldexpf(1.0f, e);
    }
    __syncthreads();
    stage_activations<!Q8, !Q8>(x, M, K, nb, nbp, pre, frag, xsum);
    if (tid == 0) frag[(size_t)nbp * ncols * 4] = make_uint4(0, 0, 0, 0);
    __syncthreads();

    // Per-lane shared addresses of the activation image (block 0) and strides per block. Columns /
    // activation rows that do not exist read a zero slot with stride 0.
    const uint32_t zero_slot = (uint32_t)__cvta_generic_to_shared(frag + (size_t)nbp * ncols * 4);
    uint32_t fbase[NS], fstride[NS], xbase[NS], xstride[NS];
#pragma unroll
    for (int c = 0; c < NS; ++c) {
        const uint32_t col = 8 * c + g;
        const bool real = col < ncols;
        fbase[c] = real ? (uint32_t)__cvta_generic_to_shared(frag + (size_t)col * 4 + t) : zero_slot;
        fstride[c] = real ? ncols * 64 : 0;
        const uint32_t m = 4 * c + t;
        const bool xreal = !Q8 && m < M;
        xbase[c] = xreal ? (uint32_t)__cvta_generic_to_shared(xsum + m) : zero_slot;
        xstride[c] = xreal ? M * 4 : 0;
    }

    for (uint64_t tile = blockIdx.x; tile * rows_per_cta < N; tile += gridDim.x) {
        const uint32_t r0 = (uint32_t)(tile * rows_per_cta) + wr * 16 + g;
        uint32_t faddr[NS], xaddr[NS];
#pragma unroll
        for (int c = 0; c < NS; ++c) {
            faddr[c] = fbase[c] + q_lo * 4 * fstride[c];
            xaddr[c] = xbase[c] + q_lo * 4 * xstride[c];
        }
        float acc[NS][4], accm[NS][2];
#pragma unroll
        for (int c = 0; c < NS; ++c) {
            acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.0f;
            accm[c][0] = accm[c][1] = 0.0f;
        }
#pragma unroll 1
        for (uint32_t i = 0; i < nqw; ++i) {
            QuadRegs<Q8, Q41> r;
            if (USE_RING) {
                producer_step();
                cp_async_wait<D - 1>();  // all but the newest D-1 groups have landed: this quad is in the ring
                ring_read<Q8, Q41>(r, ring32 + c_slot * R::kStage, lane);
                c_slot = c_slot + 1 == (uint32_t)D ? 0 : c_slot + 1;
            } else {
                r = nxt;
                producer_step();
            }
            compute_quad<TYPE, NS>(r, faddr, fstride, xaddr, xstride, acc, accm);
#pragma unroll
            for (int c = 0; c < NS; ++c) {
                faddr[c] += 4 * fstride[c];
                xaddr[c] += 4 * xstride[c];
            }
        }

        // hi + lo columns -> one value per (row, activation row); lane (g, t) of set c owns
        // activation row 4c + t for weight rows g and g + 8.
        float out_a[NS], out_b[NS];
#pragma unroll
        for (int c = 0; c < NS; ++c) {
            if (Q8) {
                out_a[c] = acc[c][0] + acc[c][1];
                out_b[c] = acc[c][2] + acc[c][3];
            } else {  // sums are in units of 2^-24; the block offsets/minimums were collected in accm
                const float k = Q41 ? 1.0f : -8.0f;
                out_a[c] = fmaf(acc[c][0] + acc[c][1], 16777216.0f, k * accm[c][0]);
                out_b[c] = fmaf(acc[c][2] + acc[c][3], 16777216.0f, k * accm[c][1]);
            }
        }
        if (KS > 1) {
            if (!helper) {
                float* mine = red + ((size_t)(wr * KS + ks) * NS * 2) * 32;
#pragma unroll
                for (int c = 0; c < NS; ++c) {
                    mine[(c * 2 + 0) * 32 + lane] = out_a[c];
                    mine[(c * 2 + 1) * 32 + lane] = out_b[c];
                }
            }
            __syncthreads();
            if (ks == 0) {
#pragma unroll
                for (int c = 0; c < NS; ++c) {
                    float va = 0.0f, vb = 0.0f;
                    for (uint32_t k2 = 0; k2 < KS; ++k2) {
                        const float* other = red + ((size_t)(wr * KS + k2) * NS * 2) * 32;
                        va += other[(c * 2 + 0) * 32 + lane];
                        vb += other[(c * 2 + 1) * 32 + lane];
                    }
                    out_a[c] = va;
                    out_b[c] = vb;
                }
            }
        }
        if (ks == 0) {
#pragma unroll
            for (int c = 0; c < NS; ++c) {
                const uint32_t m = 4 * c + t;
                if (m < M) {
                    const float ps = post[m];
                    if (r0 < N) y[(size_t)m * N + r0] = apply_epilogue(out_a[c] * ps, ep, r0, (size_t)m * N + r0);
                    if (r0 + 8 < N)
                        y[(size_t)m * N + r0 + 8] = apply_epilogue(out_b[c] * ps, ep, r0 + 8, (size_t)m * N + r0 + 8);
                }
            }
        }
        if (KS > 1) __syncthreads();  // `red` is reused by the next tile
    }
}

// ---- single activation row (decode): the 8 MMA columns hold 4 blocks x (hi, lo) ------------------
//
// With one activation row only two of the eight MMA columns would carry data. This kernel instead
// gives column pair (2j, 2j+1) the hi / lo activation parts of block j of the quad and zeros
// elsewhere, and chains the 8 MMAs of a quad (4 blocks x low / high nibbles) into ONE accumulator:
// column pair j then holds sum(n * x) of block j alone. Lane (g, t) owns columns 2t, 2t+1 of rows g and
// g + 8, i.e. the finished sums of block 4q + t — so it needs one scale per row and quad (not four),
// one multiply-add per row and quad, and one real activation-fragment load per quad (it feeds column
// g, which is non-zero only for block g / 2). q4_0's "- 8" enters as the accumulator's initial value
// -8 * sum(x_block) in the hi column, so no second accumulator exists. Per quad and lane: the nibble
// unpack (40 logic ops), 8 MMAs, 4 predicated shared loads, 2 global 128-bit loads, 2 scale loads.
// Rows are not split across warps (used when there are enough row tiles to fill the GPU).
__device__ __forceinline__ void lds128_keep(uint4& v, uint32_t addr, uint32_t pred) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.u32 p, %5, 0;\n\t"
        "@p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n\t}"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "r"(addr), "r"(pred));
}


// Row-sharded use: besides its own result buffer the kernel stores every output row into the same
// place of each peer's buffer (plain stores to peer-mapped memory over NVLink), so the all-gather of the
// slices happens while the weights are still streaming. When the last CTA of the grid is done it adds 1
// to this rank's counter on every peer and waits — bounded — until every peer's counter here has
// reached the round number. world <= 1: an ordinary GEMV into `y`.
//
// Tagged form (pa.tagged): what travels to a peer is a 64-bit word per output row, the round number above the
// float's bits, stored into the peer's inbox; a word says by itself whether it belongs to this round, so no
// fence, counter or flag follows the stores. When a CTA has finished its own rows it turns to the inbox of
// this GPU: the grid's threads share the other ranks' rows, poll each pair of words (bounded) until both
// carry this round's number and store the floats into this rank's result row. Two inboxes alternate: a peer
// can be at most one round ahead (it needs this rank's words of a round to finish that round), and then it
// writes into the other one.
//
// Arg-max form (ARGMAX): for greedy decoding only the index of the first largest logit is needed
// (gpt2.zig:980-990: strict `>`, so the lowest index among equals). Every lane keeps the best of its rows, a CTA
// reduces its lanes and writes (value, row) into its slot; the grid's last CTA reduces the slots, sends this
// rank's (value, row) as two tagged words to every peer, polls (bounded) for theirs and takes the best in rank
// order, which is row order: 16 bytes per peer instead of the row.
constexpr int kPeerMax = 8;
constexpr uint32_t kPeerSpinLimit = 1u << 21;               // polls of a local flag before giving up (about a second)
constexpr unsigned int kErrFusedGatherTimeout = 0x46474154u;  // 'FGAT'
struct PeerArgs {
    float* y[2][kPeerMax];       // [round parity][rank]: result buffers, entry `rank` is this GPU's own
    uint32_t* flags[kPeerMax];   // [rank]: that rank's counters, one uint32 per source rank
    uint32_t* sync;              // this GPU: [0] completed rounds, [1] CTAs that have finished the current one
    unsigned int* err;           // the library's device-error word
    uint32_t world, rank, row_off;
    uint32_t spin_limit;         // polls of a local flag before giving up
    unsigned long long* inbox[2][kPeerMax];  // tagged form: [round parity][rank] that rank's inbox, world * per words
    uint32_t tagged, per;        // tagged form; rows owned by every rank (even)
    // arg-max form (the ARGMAX instantiation; world = 1 too): what leaves the kernel is the index and value of the
    // row's first largest element over all ranks. cta_best: one slot per CTA of this GPU; inbox: 2 words per rank.
    unsigned long long* cta_best;
    int32_t* out_index;
    float* out_value;
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Quads in flight per lane. They travel through a per-lane cp.async ring in shared memory: register
// prefetch cannot go deep (a warp has six load scoreboards, and later loads share them with earlier
// ones). Measured on the 1152 -> 262144 head: depths 3..7 are within 2% of each other once the scales
// no longer travel through the ring; one CTA per SM (8 warps) is 25% slower than two, three are 5% slower.
constexpr int kRows1Depth = 4;

template <bool Q8>
struct QuadWords {
    uint4 a, b;    // word t of blocks 0..3 of rows g / g + 8
    uint4 a2, b2;  // q8_0: word 4 + t
};

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

// (value, row) candidates: the larger value wins, the lower row among equals
__device__ __forceinline__ void take_better(float& v, uint32_t& r, float ov, uint32_t orow) {
    if (ov > v || (ov == v && orow < r)) {
        v = ov;
        r = orow;
    }
}

template <int TYPE, int D, int CTAS, int W, bool ARGMAX>
__global__ void __launch_bounds__(W * 32, CTAS)
gemv_mma1_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ sc, const float* __restrict__ x,
                 float* __restrict__ y, uint32_t N, uint32_t K, uint32_t nb, uint32_t scp, uint32_t sc_off,
                 uint32_t ring_off, EpilogueArgs ep, PeerArgs pa) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QB = Q8 ? 32 : 16;
    constexpr uint32_t SB = Q41 ? 4 : 2;
    constexpr uint32_t QUAD = 4 * QB;  // quant bytes of one quad of blocks

    extern __shared__ __align__(128) unsigned char smem_raw[];

    const uint32_t nbp = (nb + 3u) & ~3u, nq = nbp / 4;
    uint4* frag = reinterpret_cast<uint4*>(smem_raw);  // [block][hi, lo][t]
    float* xsum = reinterpret_cast<float*>(frag + (size_t)nbp * 8);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr uint32_t rows_per_cta = W * 16;

    // Let the next kernel on the stream be scheduled as CTAs of this one retire: its weight stream can
    // start while this kernel's last tiles drain. Everything up to the wait below touches only weights.
    pdl_launch_dependents();
    const bool sharded = pa.world > 1;

    // Scales of a whole 16-row tile (contiguous in memory) are copied to this warp's shared buffer when
    // the producer enters the tile; two buffers, because the producer is less than one tile ahead.
    const uint32_t sc_row_bytes = scp * SB;
    const uint32_t sc_tile_bytes = 16 * sc_row_bytes;  // a multiple of 256
    const uint32_t sbuf32 = (uint32_t)__cvta_generic_to_shared(smem_raw + sc_off) + warp * 2 * sc_tile_bytes;

    // ---- producer: the quads of this warp's tiles, in order, D - 1 ahead of the consumer. Each step
    //      closes one cp.async group: group n holds quad n of the warp's sequence (plus, when quad n is
    //      the last of its tile, the next tile's scales) ----
    constexpr uint32_t kStage = Q8 ? 2048 : 1024;  // a, b (, a2, b2): 512 bytes each
    const uint32_t ring32 = (uint32_t)__cvta_generic_to_shared(smem_raw + ring_off) + warp * D * kStage + lane * 16;
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
        cp_async_commit();
    };
    producer_set_tile();
#pragma unroll 1
    for (int i = 0; i < D - 1; ++i) producer_step();
    uint32_t c_slot = 0;

    // The activations, the result buffer and (sharded) the round counter may belong to the kernel before
    // this one: wait for it to complete. Sharded: every CTA then reads the round before any CTA can finish
    // it (the counter moves only when all CTAs have arrived at the end of the kernel).
    pdl_wait();
    const uint32_t round = (sharded || ARGMAX) ? pa.sync[0] + 1 : 0;
    if (sharded && !ARGMAX) y = pa.y[round & 1u][pa.rank] + pa.row_off;
    float best_v = -INFINITY;       // ARGMAX: the best of this lane's rows (they come in ascending order)
    uint32_t best_r = 0xFFFFFFFFu;

    // ---- activations: range prescale, then the fp16 hi / lo fragment image. Every warp finds the row's
    //      largest magnitude by itself (the row is a few KB and stays in L1): no block-wide exchange ----
    float pre_l[1], ps;
    {
        float amax = 0.0f;
        const float4* xr = reinterpret_cast<const float4*>(x);
        const uint32_t n4 = K / 4;
        for (uint32_t i0 = lane; i0 < n4; i0 += 32 * 8) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                v[u] = i0 + 32 * u < n4 ? xr[i0 + 32 * u] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v[u].x), fabsf(v[u].y))), fmaxf(fabsf(v[u].z), fabsf(v[u].w)));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
        const int e = row_scale_exponent(amax);
        pre_l[0] = ldexpf(1.0f, -e);
        ps = ldexpf(1.0f, e);
    }
    stage_activations<!Q8, !Q8>(x, 1, K, nb, nbp, pre_l, frag, xsum);
    __syncthreads();

    // This lane feeds MMA column g: part (g & 1) of block (g >> 1) of each quad.
    const uint32_t myj = g >> 1;
    const uint32_t frag0 = (uint32_t)__cvta_generic_to_shared(frag + ((size_t)myj * 2 + (g & 1)) * 4 + t);
    const uint32_t xsum0 = (uint32_t)__cvta_generic_to_shared(xsum + t);
    const uint32_t pj0 = myj == 0, pj1 = myj == 1, pj2 = myj == 2, pj3 = myj == 3;
    uint4 bj0 = make_uint4(0, 0, 0, 0), bj1 = bj0, bj2 = bj0, bj3 = bj0;  // stay zero unless this lane's block

    uint64_t c_tile = blockIdx.x;
    uint32_t c_q = 0, c_par = 0;
    uint32_t faddr = frag0, xaddr = xsum0;
    // scales of block 4q + t, rows g and g + 8, in the current tile's buffer
    const uint32_t sc_lane = g * sc_row_bytes + t * SB;
    uint32_t saddr = sbuf32 + sc_lane;
    float acc_a = 0.0f, acc_b = 0.0f, accm_a = 0.0f, accm_b = 0.0f;

    auto consume = [&](const QuadWords<Q8>& d) {
        lds128_keep(bj0, faddr, pj0);  // one of the four executes: faddr already points at this lane's block
        lds128_keep(bj1, faddr, pj1);
        lds128_keep(bj2, faddr, pj2);
        lds128_keep(bj3, faddr, pj3);
        float xs = 0.0f;
        if (!Q8) xs = lds_f32(xaddr);
        float da, db, ma = 0.0f, mb = 0.0f;
        if (Q41) {
            unpack_half2(lds_u32(saddr), da, ma);
            unpack_half2(lds_u32(saddr + 8 * sc_row_bytes), db, mb);
        } else {
            da = __half2float(__ushort_as_half((unsigned short)lds_u16(saddr)));
            db = __half2float(__ushort_as_half((unsigned short)lds_u16(saddr + 8 * sc_row_bytes)));
        }
        float dacc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (TYPE == ZQ_TYPE_Q4_0) {
            // (n - 8) * x summed = sum(n * x) - 8 * sum(x); the MMAs work in units of 2^-24
            dacc[0] = dacc[2] = xs * (-8.0f / 16777216.0f);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4& bf = j == 0 ? bj0 : j == 1 ? bj1 : j == 2 ? bj2 : bj3;
            uint32_t a_lo[4], a_hi[4];
            if (Q8) {
                unpack_q8(pick(d.a, j), a_lo[0], a_lo[2]);
                unpack_q8(pick(d.b, j), a_lo[1], a_lo[3]);
                unpack_q8(pick(d.a2, j), a_hi[0], a_hi[2]);
                unpack_q8(pick(d.b2, j), a_hi[1], a_hi[3]);
            } else {
                unpack_q4(pick(d.a, j), a_lo[0], a_lo[2], a_hi[0], a_hi[2]);
                unpack_q4(pick(d.b, j), a_lo[1], a_lo[3], a_hi[1], a_hi[3]);
            }
            mma_f16(dacc, a_lo, bf.x, bf.y, dacc);
            mma_f16(dacc, a_hi, bf.z, bf.w, dacc);
        }
        if (Q41) {
            accm_a = fmaf(ma, xs, accm_a);
            accm_b = fmaf(mb, xs, accm_b);
        }
        acc_a = fmaf(dacc[0] + dacc[1], da, acc_a);
        acc_b = fmaf(dacc[2] + dacc[3], db, acc_b);
        faddr += 512;  // 4 blocks x (hi, lo) x 4 lanes x 16 bytes
        xaddr += 16;
        saddr += 4 * SB;
        if (++c_q == nq) {
            // blocks of the row are spread over the 4 lanes of the quad: add them up
            float va = acc_a, vb = acc_b;
            if (!Q8) {
                va *= 16777216.0f;
                vb *= 16777216.0f;
            }
            if (Q41) {
                va += accm_a;
                vb += accm_b;
            }
            va += __shfl_xor_sync(0xFFFFFFFFu, va, 1);
            vb += __shfl_xor_sync(0xFFFFFFFFu, vb, 1);
            va += __shfl_xor_sync(0xFFFFFFFFu, va, 2);
            vb += __shfl_xor_sync(0xFFFFFFFFu, vb, 2);
            // all four lanes of a quad hold both sums: lane t = 0 stores row g, lane t = 1 row g + 8, so one
            // store instruction writes the tile's 16 outputs as 64 contiguous bytes
            const uint32_t row = (uint32_t)(c_tile * rows_per_cta) + warp * 16 + g + (t == 1 ? 8u : 0u);
            if (t < 2 && row < N) {
                const float o = apply_epilogue((t == 1 ? vb : va) * ps, ep, row, row);
                if (ARGMAX) {
                    if (y) y[row] = o;
                    if (o > best_v) {
                        best_v = o;
                        best_r = row;
                    }
                } else {
                    y[row] = o;
                }
                if (ARGMAX) {
                } else if (sharded && pa.tagged) {
                    const unsigned long long word = ((unsigned long long)round << 32) | __float_as_uint(o);
                    for (uint32_t p = 0; p < pa.world; ++p)
                        if (p != pa.rank)
                            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(pa.inbox[round & 1u][p] + pa.row_off + row),
                                         "l"(word)
                                         : "memory");
                } else if (sharded) {
                    for (uint32_t p = 0; p < pa.world; ++p)
                        if (p != pa.rank) pa.y[round & 1u][p][pa.row_off + row] = o;
                }
            }
            c_q = 0;
            c_tile += gridDim.x;
            c_par ^= 1u;
            faddr = frag0;
            xaddr = xsum0;
            saddr = sbuf32 + c_par * sc_tile_bytes + sc_lane;
            acc_a = acc_b = accm_a = accm_b = 0.0f;
        }
    };

#pragma unroll 1
    while (c_tile * rows_per_cta < N) {
        producer_step();
        cp_async_wait<D - 1>();  // all but the newest D - 1 groups have landed: this quad (and, at the
        __syncwarp();            // start of a tile, its scales, copied by all lanes) is in shared memory
        const uint32_t stage = ring32 + c_slot * kStage;
        QuadWords<Q8> r;
        r.a = lds128(stage);
        r.b = lds128(stage + 512);
        if (Q8) {
            r.a2 = lds128(stage + 1024);
            r.b2 = lds128(stage + 1536);
        }
        c_slot = c_slot + 1 == (uint32_t)D ? 0 : c_slot + 1;
        consume(r);
    }

    if (ARGMAX) {
        __shared__ float s_v[W];
        __shared__ uint32_t s_r[W];
        __shared__ int s_last;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1)
            take_better(best_v, best_r, __shfl_xor_sync(0xFFFFFFFFu, best_v, off), __shfl_xor_sync(0xFFFFFFFFu, best_r, off));
        if (lane == 0) {
            s_v[warp] = best_v;
            s_r[warp] = best_r;
        }
        __syncthreads();
        if (tid == 0) {
            float v = s_v[0];
            uint32_t r = s_r[0];
            for (int i = 1; i < W; ++i) take_better(v, r, s_v[i], s_r[i]);
            pa.cta_best[blockIdx.x] = ((unsigned long long)__float_as_uint(v) << 32) | r;
            __threadfence();
            s_last = atomicAdd(pa.sync + 1, 1u) == gridDim.x - 1;
        }
        __syncthreads();
        if (s_last) {  // every CTA's slot is written: this CTA reduces them
            __threadfence();
            float v = -INFINITY;
            uint32_t r = 0xFFFFFFFFu;
            for (uint32_t i = tid; i < gridDim.x; i += W * 32) {
                const unsigned long long s = __ldcg(pa.cta_best + i);
                take_better(v, r, __uint_as_float((uint32_t)(s >> 32)), (uint32_t)s);
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1)
                take_better(v, r, __shfl_xor_sync(0xFFFFFFFFu, v, off), __shfl_xor_sync(0xFFFFFFFFu, r, off));
            __syncthreads();  // s_v / s_r of the first reduction have been read
            if (lane == 0) {
                s_v[warp] = v;
                s_r[warp] = r;
            }
            __syncthreads();
            if (warp == 0) {
                v = s_v[0], r = s_r[0];
                for (int i = 1; i < W; ++i) take_better(v, r, s_v[i], s_r[i]);
                r = r == 0xFFFFFFFFu ? 0u : r + pa.row_off;  // nothing compared greater than -inf: index 0, as the reference
                if (sharded) {
                    // lane q talks to rank q: this rank's two words to q's inbox, q's two words from this rank's inbox
                    const uint32_t q = (uint32_t)lane;
                    float qv = v;
                    uint32_t qr = r;
                    if (q < pa.world && q != pa.rank) {
                        unsigned long long* to = pa.inbox[round & 1u][q] + 2u * pa.rank;
                        const unsigned long long tag = (unsigned long long)round << 32;
                        asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};" ::"l"(to), "l"(tag | __float_as_uint(v)), "l"(tag | r)
                                     : "memory");
                        const unsigned long long* from = pa.inbox[round & 1u][pa.rank] + 2u * q;
                        unsigned long long a = 0, b = 0;
                        bool ok = false;
                        for (uint32_t n = 0; n < pa.spin_limit; ++n) {
                            asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(from) : "memory");
                            if ((uint32_t)(a >> 32) == round && (uint32_t)(b >> 32) == round) {
                                ok = true;
                                break;
                            }
                        }
                        if (!ok) atomicExch(pa.err, kErrFusedGatherTimeout);
                        qv = __uint_as_float((uint32_t)a);
                        qr = (uint32_t)b;
                    }
                    // ranks in ascending order own ascending rows: strict `>` keeps the first largest
                    v = __shfl_sync(0xFFFFFFFFu, qv, 0);
                    r = __shfl_sync(0xFFFFFFFFu, qr, 0);
                    for (uint32_t p = 1; p < pa.world; ++p) {
                        const float pv = __shfl_sync(0xFFFFFFFFu, qv, p);
                        const uint32_t pr = __shfl_sync(0xFFFFFFFFu, qr, p);
                        if (pv > v) {
                            v = pv;
                            r = pr;
                        }
                    }
                }
                if (lane == 0) {
                    *pa.out_index = (int32_t)r;
                    if (pa.out_value) *pa.out_value = v;
                    pa.sync[1] = 0;
                    __threadfence();
                    pa.sync[0] = round;
                }
            }
        }
    } else if (sharded && pa.tagged) {
        // the other ranks' rows, two words per thread and pass
        const unsigned long long* in = pa.inbox[round & 1u][pa.rank];
        float* yfull = pa.y[round & 1u][pa.rank];
        const uint32_t n_other = pa.per * (pa.world - 1u);
        bool dead = false;
        for (uint32_t i = 2u * (blockIdx.x * blockDim.x + tid); i < n_other; i += 2u * gridDim.x * blockDim.x) {
            const uint32_t pi = i / pa.per;
            const uint32_t at = i + (pi >= pa.rank ? pa.per : 0u);  // skip this rank's own rows
            unsigned long long a = 0, b = 0;
            bool ok = false;
            for (uint32_t n = 0; n < pa.spin_limit && !dead; ++n) {
                asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(in + at) : "memory");
                if ((uint32_t)(a >> 32) == round && (uint32_t)(b >> 32) == round) {
                    ok = true;
                    break;
                }
            }
            if (!ok && !dead) {  // one report per thread, and no further waiting by it
                dead = true;
                atomicExch(pa.err, kErrFusedGatherTimeout);
            }
            *reinterpret_cast<float2*>(yfull + at) = make_float2(__uint_as_float((uint32_t)a), __uint_as_float((uint32_t)b));
        }
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            const uint32_t ticket = atomicAdd(pa.sync + 1, 1u);
            if (ticket == gridDim.x - 1) {  // every CTA has stored its rows and its share of the inbox
                pa.sync[1] = 0;
                __threadfence();
                pa.sync[0] = round;
            }
        }
    } else if (sharded) {
        __syncthreads();  // the CTA's peer stores happen before thread 0's fence (fences are cumulative)
        if (tid == 0) {
            // Device-scope fence per CTA (a system-scope fence here costs about 10 us per launch, measured);
            // the last CTA's system-scope fence is cumulative over everything that happened before the
            // arrivals it has observed, i.e. over every CTA's peer stores.
            __threadfence();
            const uint32_t ticket = atomicAdd(pa.sync + 1, 1u);
            if (ticket == gridDim.x - 1) {  // every CTA has stored, fenced and arrived
                __threadfence_system();
                for (uint32_t p = 0; p < pa.world; ++p)
                    if (p != pa.rank)  // fire-and-forget add on the peer: no round trip
                        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(pa.flags[p] + pa.rank), "r"(1u)
                                     : "memory");
                for (uint32_t p = 0; p < pa.world; ++p) {
                    if (p == pa.rank) continue;
                    bool ok = false;
                    for (uint32_t i = 0; i < pa.spin_limit; ++i) {
                        if ((int32_t)(ld_acquire_sys_u32(pa.flags[pa.rank] + p) - round) >= 0) {
                            ok = true;
                            break;
                        }
                    }
                    if (!ok) atomicExch(pa.err, kErrFusedGatherTimeout);
                }
                pa.sync[1] = 0;
                __threadfence();
                pa.sync[0] = round;  // later kernels on this stream see the completed round
            }
        }
    }
}

template <int TYPE, int D, int CTAS, int W, bool ARGMAX>
int launch_rows1_cfg(const zq_weight* w, const float* x, float* y, EpilogueArgs ep, const PeerArgs& pa,
                     cudaStream_t st) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    const uint32_t sms = (uint32_t)sm_count();
    if (w->nbp / 4 < (uint32_t)D) return ZQ_ERR_LIMIT;  // the producer must stay within one tile of the consumer
    size_t smem = (size_t)w->nbp * 128;
    if (!Q8) smem += (size_t)w->nbp * sizeof(float);
    smem = (smem + 127) & ~(size_t)127;
    const uint32_t sc_off = (uint32_t)smem;
    smem += (size_t)W * 2 * 16 * w->scp * (Q41 ? 4 : 2);
    smem = (smem + 127) & ~(size_t)127;
    const uint32_t ring_off = (uint32_t)smem;
    smem += (size_t)W * D * (Q8 ? 2048 : 1024);
    if (smem > (size_t)(227 * 1024) / CTAS - 1024) return ZQ_ERR_LIMIT;  // CTAS CTAs per SM must fit
    auto kern = gemv_mma1_kernel<TYPE, D, CTAS, W, ARGMAX>;
    if (smem > 48 * 1024)
        ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const uint32_t cta_tiles = (w->out_dim + W * 16 - 1) / (W * 16);
    const uint32_t cap = sms * CTAS;
    ZQ_CUDA(launch_pdl(kern, dim3(cta_tiles < cap ? cta_tiles : cap), dim3(W * 32), smem, st, w->qs,
                       static_cast<const uint8_t*>(w->sc), x, y, w->out_dim, w->in_dim, w->nb, w->scp, sc_off,
                       ring_off, ep, pa));
    return ZQ_OK;
}

// Whole rows per warp need enough row tiles to occupy the GPU. With fewer tiles the CTAs get smaller (so
// that every SM still has several) and the ring deeper (fewer warps must keep as many bytes in flight).
template <int TYPE, bool ARGMAX>
int launch_rows1(const zq_weight* w, const float* x, float* y, EpilogueArgs ep, const PeerArgs& pa,
                 cudaStream_t st) {
    const uint32_t tiles = (w->out_dim + 15) / 16, sms = (uint32_t)sm_count();
    constexpr int S = TYPE == ZQ_TYPE_Q8_0 ? 2 : 1;  // q8_0 stages are twice as large
    int rc = ZQ_ERR_LIMIT;
    if (tiles >= sms * 2 * 8) rc = launch_rows1_cfg<TYPE, kRows1Depth, kCtasPerSm, 8, ARGMAX>(w, x, y, ep, pa, st);
    if (rc == ZQ_ERR_LIMIT && tiles >= sms * 2 * 4) rc = launch_rows1_cfg<TYPE, 8 / S, 4, 4, ARGMAX>(w, x, y, ep, pa, st);
    if (rc == ZQ_ERR_LIMIT && tiles >= sms * 4) rc = launch_rows1_cfg<TYPE, 16 / S, 4, 2, ARGMAX>(w, x, y, ep, pa, st);
    return rc;
}

int launch_rows1_any(const zq_weight* w, const float* x, float* y, EpilogueArgs ep, const PeerArgs& pa,
                     cudaStream_t st, bool argmax = false) {
    if (argmax) {
        switch (w->type) {
            case ZQ_TYPE_Q4_0: return launch_rows1<ZQ_TYPE_Q4_0, true>(w, x, y, ep, pa, st);
            case ZQ_TYPE_Q4_1: return launch_rows1<ZQ_TYPE_Q4_1, true>(w, x, y, ep, pa, st);
            case ZQ_TYPE_Q8_0: return launch_rows1<ZQ_TYPE_Q8_0, true>(w, x, y, ep, pa, st);
            default: return ZQ_ERR_UNSUPPORTED;
        }
    }
    switch (w->type) {
        case ZQ_TYPE_Q4_0: return launch_rows1<ZQ_TYPE_Q4_0, false>(w, x, y, ep, pa, st);
        case ZQ_TYPE_Q4_1: return launch_rows1<ZQ_TYPE_Q4_1, false>(w, x, y, ep, pa, st);
        case ZQ_TYPE_Q8_0: return launch_rows1<ZQ_TYPE_Q8_0, false>(w, x, y, ep, pa, st);
        default: return ZQ_ERR_UNSUPPORTED;
    }
}

struct Plan {
    uint32_t WR, KS, grid, ring_off, warps;
    size_t smem;
    bool fits;
};

// CTA shape: enough warps in flight on every SM; K is split across warps only when there are too
// few row tiles to do that with one warp per tile.
Plan make_plan(const zq_weight* w, uint32_t M, int ns, bool use_ring, bool with_ln) {
    Plan p{};
    const bool q41 = w->type == ZQ_TYPE_Q4_1;
    const uint32_t tiles = (w->out_dim + 15) / 16;
    const uint32_t sms = (uint32_t)sm_count();
    const uint32_t nq = w->nbp / 4;
    uint32_t ks = 1;
    while (ks < 8 && tiles * ks < sms * 16 && nq / (ks * 2) >= 2) ks *= 2;
    uint32_t warps = 8;  // per CTA; fewer when that would leave SMs without a CTA
    while (warps > ks && (tiles + warps / ks - 1) / (warps / ks) < sms) warps /= 2;
    p.WR = warps / ks ? warps / ks : 1;
    p.KS = ks;
    // The activation image has nbp * 2M * 4 entries of 16 bytes; with several activation rows and few
    // computing warps, extra warps share the work of building it (about four entries per thread).
    const uint32_t entries = w->nbp * 2 * M * 4;
    uint32_t total_warps = (entries + 127) / 128;
    if (total_warps > 8) total_warps = 8;
    p.warps = total_warps > p.WR * ks ? total_warps : p.WR * ks;
    size_t smem = (size_t)w->nbp * 2 * M * 64 + 16;  // activation image + zero slot
    if (w->type != ZQ_TYPE_Q8_0) smem += (size_t)w->nbp * M * sizeof(float);
    if (ks > 1) smem += (size_t)p.WR * ks * ns * 2 * 32 * sizeof(float);
    smem = (smem + 127) & ~(size_t)127;
    if (with_ln) smem += (size_t)((w->in_dim + 31u) & ~31u) * sizeof(float);  // the normalised row, just below the ring
    p.ring_off = (uint32_t)smem;
    const bool q8 = w->type == ZQ_TYPE_Q8_0;
    const size_t stage = q8 ? Ring<true, false>::kStage : q41 ? Ring<false, true>::kStage : Ring<false, false>::kStage;
    const size_t depth = q8 ? Ring<true, false>::kDepth : Ring<false, false>::kDepth;
    if (use_ring) smem += (size_t)p.WR * ks * depth * stage;
    p.smem = smem;
    p.fits = smem <= 200 * 1024;
    const uint32_t cta_tiles = (tiles + p.WR - 1) / p.WR;
    uint32_t per_sm = (uint32_t)((224 * 1024) / (smem + 1024));
    if (per_sm > (uint32_t)kCtasPerSm) per_sm = kCtasPerSm;  // register budget set by the launch bounds
    if (per_sm < 1) per_sm = 1;
    const uint32_t cap = sms * per_sm;
    p.grid = cta_tiles < cap ? cta_tiles : cap;
    return p;
}

template <int TYPE, int NS, bool USE_RING>
int launch_kernel(const zq_weight* w, const float* x, float* y, uint32_t M, EpilogueArgs ep, cudaStream_t st) {
    const Plan p = make_plan(w, M, NS, USE_RING, ep.ln_gamma != nullptr);
    if (!p.fits) return ZQ_ERR_LIMIT;
    auto kern = gemv_mma_kernel<TYPE, NS, USE_RING>;
    if (p.smem > 48 * 1024)
        ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem));
    ZQ_CUDA(launch_pdl(kern, dim3(p.grid), dim3(p.warps * 32), p.smem, st, w->qs,
                       static_cast<const uint8_t*>(w->sc), x, y, w->out_dim, w->in_dim, w->nb, w->scp, M, p.WR, p.KS,
                       p.ring_off, ep));
    return ZQ_OK;
}

// The shared-memory ring pays off on long streams of q4_0 / q8_0 rows (measured on the 170-320 MB
// vocabulary head); q4_1 (wider scale copies) and weights of a few tens of MB run faster with the
// next quad held in registers and more CTAs per SM.
template <int TYPE, int NS>
int launch_one(const zq_weight* w, const float* x, float* y, uint32_t M, EpilogueArgs ep, cudaStream_t st) {
    const size_t quant_bytes = (size_t)w->out_dim * w->nbp * w->qb;
    if (TYPE != ZQ_TYPE_Q4_1 && quant_bytes >= ((size_t)64 << 20))
        return launch_kernel<TYPE, NS, true>(w, x, y, M, ep, st);
    return launch_kernel<TYPE, NS, false>(w, x, y, M, ep, st);
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
// Returns ZQ_ERR_LIMIT when the activation image does not fit in shared memory.
int launch_gemv_mma_f32(const zq_weight* w, const float* x, float* y, uint32_t m_rows,
                        const zq_epilogue* ep, cudaStream_t st) {
    return launch_gemv_mma_ln_f32(w, x, y, m_rows, ep, nullptr, nullptr, 0.0f, st);
}

// ln_gamma != nullptr (one activation row only): y = W . LayerNorm(x), the norm computed in the prologue.
int launch_gemv_mma_ln_f32(const zq_weight* w, const float* x, float* y, uint32_t m_rows, const zq_epilogue* ep,
                           const float* ln_gamma, const float* ln_beta, float ln_eps, cudaStream_t st) {
    if (m_rows == 0) return ZQ_OK;
    if (m_rows > 16) return ZQ_ERR_BAD_ARG;
    if (ln_gamma && (m_rows != 1 || !ln_beta)) return ZQ_ERR_BAD_ARG;
    if (((uintptr_t)x & 15) != 0) return ZQ_ERR_BAD_ARG;  // activation rows are read as float4
    EpilogueArgs a{nullptr, nullptr, nullptr, 0, ln_gamma, ln_beta, ln_eps};
    if (ep) {
        a.bias = ep->d_bias;
        a.gelu = ep->gelu;
        a.mul = ep->d_mul;
        a.residual = ep->d_residual;
    }
    // One activation row and enough 16-row tiles to give every resident warp its own rows: the
    // block-per-column kernel. Otherwise the general kernel (activation rows in columns, K split).
    if (m_rows == 1 && !ln_gamma && (w->out_dim + 15) / 16 >= (uint32_t)sm_count() * 4) {
        PeerArgs none{};
        const int rc = launch_rows1_any(w, x, y, a, none, st);
        if (rc != ZQ_ERR_LIMIT) return rc;
    }
    switch (w->type) {
        case ZQ_TYPE_Q4_0: return launch_ns<ZQ_TYPE_Q4_0>(w, x, y, m_rows, a, st);
        case ZQ_TYPE_Q4_1: return launch_ns<ZQ_TYPE_Q4_1>(w, x, y, m_rows, a, st);
        case ZQ_TYPE_Q8_0: return launch_ns<ZQ_TYPE_Q8_0>(w, x, y, m_rows, a, st);
        default: return ZQ_ERR_UNSUPPORTED;
    }
}


// Any number of activation rows: passes of up to 16 rows over the weights, the pass height halved until
// the activation image of a pass fits in shared memory. ZQ_ERR_LIMIT when not even one row fits.
int launch_gemv_mma_passes_f32(const zq_weight* w, const float* x, float* y, uint32_t m_rows,
                               const zq_epilogue* epilogue, cudaStream_t st) {
    uint32_t pass = 16;
    while (pass > 1 && pass / 2 >= m_rows) pass /= 2;
    const bool ring = w->type != ZQ_TYPE_Q4_1 && (size_t)w->out_dim * w->nbp * w->qb >= ((size_t)64 << 20);
    while (pass >= 1 && !make_plan(w, pass, (int)((pass + 3) / 4), ring, false).fits) pass /= 2;
    if (pass == 0) return ZQ_ERR_LIMIT;
    for (uint32_t m0 = 0; m0 < m_rows; m0 += pass) {
        const uint32_t mc = m_rows - m0 < pass ? m_rows - m0 : pass;
        zq_epilogue ep{nullptr, 0, nullptr, nullptr};
        if (epilogue) {
            ep = *epilogue;
            if (ep.d_mul) ep.d_mul += (size_t)m0 * w->out_dim;
            if (ep.d_residual) ep.d_residual += (size_t)m0 * w->out_dim;
        }
        const int rc = launch_gemv_mma_f32(w, x + (size_t)m0 * w->in_dim, y + (size_t)m0 * w->out_dim, mc,
                                           epilogue ? &ep : nullptr, st);
        if (rc != ZQ_OK) return rc;
    }
    return ZQ_OK;
}

static EpilogueArgs gather_epilogue(const zq_epilogue* ep) {
    EpilogueArgs a{nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0.0f};
    if (ep) {
        a.bias = ep->d_bias;
        a.gelu = ep->gelu;
        a.mul = ep->d_mul;
        a.residual = ep->d_residual;
    }
    return a;
}

// The tagged form: inboxes of 64-bit words on every rank instead of result buffers and counters.
int launch_gemv_gather_tagged_f32(const zq_weight* w, const float* x, const zq_epilogue* ep,
                                  unsigned long long* const* inbox_odd, unsigned long long* const* inbox_even,
                                  float* y_odd, float* y_even, uint32_t world, uint32_t rank, uint32_t* d_sync,
                                  cudaStream_t st) {
    if (world < 2 || world > (uint32_t)kPeerMax || rank >= world) return ZQ_ERR_BAD_ARG;
    if (((uintptr_t)x & 15) != 0 || ((uintptr_t)y_odd & 7) != 0 || ((uintptr_t)y_even & 7) != 0) return ZQ_ERR_BAD_ARG;
    if ((w->out_dim & 1u) != 0) return ZQ_ERR_UNSUPPORTED;  // words are read in pairs
    if ((w->out_dim + 15) / 16 < (uint32_t)sm_count() * 4) return ZQ_ERR_UNSUPPORTED;
    const EpilogueArgs a = gather_epilogue(ep);
    PeerArgs pa{};
    for (uint32_t r = 0; r < world; ++r) {
        if (!inbox_odd[r] || !inbox_even[r]) return ZQ_ERR_PEER;  // a peer's inbox was never mapped
        if ((((uintptr_t)inbox_odd[r] | (uintptr_t)inbox_even[r]) & 15) != 0) return ZQ_ERR_BAD_ARG;
        pa.inbox[1][r] = inbox_odd[r];
        pa.inbox[0][r] = inbox_even[r];
    }
    pa.y[1][rank] = y_odd;
    pa.y[0][rank] = y_even;
    pa.sync = d_sync;
    int rc = device_error_word(&pa.err);
    if (rc != ZQ_OK) return rc;
    pa.world = world;
    pa.rank = rank;
    pa.row_off = rank * w->out_dim;
    pa.per = w->out_dim;
    pa.tagged = 1;
    pa.spin_limit = wait_limit() ? wait_limit() : kPeerSpinLimit;
    rc = launch_rows1_any(w, x, nullptr, a, pa, st);
    return rc == ZQ_ERR_LIMIT ? ZQ_ERR_UNSUPPORTED : rc;
}

// One activation row, row-sharded weight: GEMV with the all-gather of the output slices in its epilogue.
// ZQ_ERR_UNSUPPORTED when the shard is too small for the whole-rows kernel (the caller then runs the
// plain GEMV followed by the separate exchange).
// The arg-max form. world = 1: no inboxes, the index over this GPU's rows. d_sync: 2 words as above, then one
// 64-bit slot per CTA (kArgmaxSyncWords uint32 in all).
int launch_gemv_argmax_f32(const zq_weight* w, const float* x, const zq_epilogue* ep, float* y_local,
                           unsigned long long* const* inbox_odd, unsigned long long* const* inbox_even,
                           int32_t* out_index, float* out_value, uint32_t world, uint32_t rank, uint32_t* d_sync,
                           cudaStream_t st) {
    if (world < 1 || world > (uint32_t)kPeerMax || rank >= world || !out_index || !d_sync) return ZQ_ERR_BAD_ARG;
    if (((uintptr_t)x & 15) != 0 || ((uintptr_t)d_sync & 7) != 0) return ZQ_ERR_BAD_ARG;
    if ((w->out_dim + 15) / 16 < (uint32_t)sm_count() * 4) return ZQ_ERR_UNSUPPORTED;
    if ((uint64_t)w->out_dim * world > 0xFFFFFFFEull) return ZQ_ERR_LIMIT;
    const EpilogueArgs a = gather_epilogue(ep);
    PeerArgs pa{};
    if (world > 1) {
        if (!inbox_odd || !inbox_even) return ZQ_ERR_BAD_ARG;
        for (uint32_t r = 0; r < world; ++r) {
            if (!inbox_odd[r] || !inbox_even[r]) return ZQ_ERR_PEER;
            if ((((uintptr_t)inbox_odd[r] | (uintptr_t)inbox_even[r]) & 15) != 0) return ZQ_ERR_BAD_ARG;
            pa.inbox[1][r] = inbox_odd[r];
            pa.inbox[0][r] = inbox_even[r];
        }
    }
    pa.sync = d_sync;
    pa.cta_best = reinterpret_cast<unsigned long long*>(d_sync + 2);
    pa.out_index = out_index;
    pa.out_value = out_value;
    int rc = device_error_word(&pa.err);
    if (rc != ZQ_OK) return rc;
    pa.world = world;
    pa.rank = rank;
    pa.row_off = rank * w->out_dim;
    pa.per = w->out_dim;
    pa.tagged = 2;
    pa.spin_limit = wait_limit() ? wait_limit() : kPeerSpinLimit;
    rc = launch_rows1_any(w, x, y_local, a, pa, st, true);
    return rc == ZQ_ERR_LIMIT ? ZQ_ERR_UNSUPPORTED : rc;
}

int launch_gemv_gather_f32(const zq_weight* w, const float* x, const zq_epilogue* ep, float* const* y_odd,
                           float* const* y_even, uint32_t* const* flags, uint32_t world, uint32_t rank,
                           uint32_t row_off, uint32_t* d_sync, cudaStream_t st) {
    if (world < 2 || world > (uint32_t)kPeerMax || rank >= world) return ZQ_ERR_BAD_ARG;
    if (((uintptr_t)x & 15) != 0) return ZQ_ERR_BAD_ARG;
    if ((w->out_dim + 15) / 16 < (uint32_t)sm_count() * 4) return ZQ_ERR_UNSUPPORTED;
    const EpilogueArgs a = gather_epilogue(ep);
    PeerArgs pa{};
    for (uint32_t r = 0; r < world; ++r) {
        if (!y_odd[r] || !y_even[r] || !flags[r]) return ZQ_ERR_PEER;  // a peer's buffer was never mapped
        pa.y[1][r] = y_odd[r];
        pa.y[0][r] = y_even[r];
        pa.flags[r] = flags[r];
    }
    pa.sync = d_sync;
    int rc = device_error_word(&pa.err);
    if (rc != ZQ_OK) return rc;
    pa.world = world;
    pa.rank = rank;
    pa.row_off = row_off;
    pa.spin_limit = wait_limit() ? wait_limit() : kPeerSpinLimit;
    rc = launch_rows1_any(w, x, nullptr, a, pa, st);
    return rc == ZQ_ERR_LIMIT ? ZQ_ERR_UNSUPPORTED : rc;
}

}  // namespace zq
