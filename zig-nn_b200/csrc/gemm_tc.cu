// Batched quantised matmul on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// Same arithmetic as gemm.cu (weights dequantised once to fp16, activations fp16 with a per-row
// power-of-two scale, f32 accumulation; zig-nn src/gguf/dequant.zig:133-309 is the CPU statement), but
// the product runs as tcgen05.mma with both operands in shared memory and the accumulator in tensor
// memory:
//
//   A operand  = 128 weight rows x 64 K (fp16, K-major, 128-byte swizzle), written by the dequantising
//                warps straight from the packed GGUF words;
//   B operand  = up to 256 activation rows x 64 K (fp16, K-major, same swizzle). The conversion kernel
//                writes the fp16 activations segment-major ([K / 64][rows][64], chunks already swizzled,
//                rows padded with zeros to whole tiles), so a stage's tile is one contiguous block that a
//                single bulk copy (cp.async.bulk, completion counted on the stage's mbarrier) brings in;
//   D          = 128 lanes x N columns of f32 in tensor memory (one lane per weight row).
//
// A CTA owns one or two tiles of 128 weight rows (two accumulators side by side in tensor memory, the
// activation tile of a stage shared by both; chosen per call, see launch_tc).
// Roles: warps 0-15 produce stages (dequantise) and later drain the accumulator; one thread of
// warp 16 issues the MMAs. Stages are handed over through mbarriers: full[s] (one arrival per producer warp),
// empty[s] (tcgen05.commit when the MMAs that read the stage are done), acc (last commit). Every wait
// is bounded; on a timeout the kernel records it in the library's device-error word, stops using
// the pipeline, still releases tensor memory and returns (outputs are then undefined; zq_device_error
// reports it).
#include "zq_internal.h"

namespace zq {
namespace {

constexpr int TC_BN = 128;          // weight rows per CTA  (UMMA M)
constexpr int TC_BM = 256;          // activation rows per CTA, at most (UMMA N)
constexpr int TC_BK = 64;           // K per stage: one 128-byte swizzle atom of fp16
constexpr int TC_MAX_STAGES = 4;
constexpr int TC_PRODUCERS = 512;   // threads of warps 0-15
constexpr int TC_THREADS = TC_PRODUCERS + 32;
constexpr uint32_t TC_A_BYTES = TC_BN * 128;   // 16 KB per tile of 128 weight rows
constexpr uint32_t TC_B_BYTES = TC_BM * 128;   // 32 KB
// RT tiles of 128 weight rows share one activation tile per stage (RT accumulators in tensor memory):
// RT = 1: 48 KB stages, 4 of them; RT = 2: 64 KB stages, 3 of them, twice the MMA work per hand-over.
template <int RT>
struct TcShape {
    static constexpr uint32_t kStageBytes = RT * TC_A_BYTES + TC_B_BYTES;
    static constexpr int kStages = RT == 1 ? 4 : 3;
};
constexpr uint32_t kSpinLimit = 1u << 24;      // iterations of a try_wait loop before giving up (about a second)
constexpr unsigned int kErrGemmTimeout = 0x47454D4Du;  // 'GEMM'

struct TcEpilogue {
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

// ---- mbarrier / tcgen05 wrappers -----------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// global -> shared bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned); the bytes are
// counted on `bar` as they land
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait. Returns false after kSpinLimit polls or when another thread has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned int* err_word) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(err_word, kErrGemmTimeout);
    return false;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 32 consecutive columns of f32: register i of lane l = D[lane_base + l][col + i]
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major tile of rows x 64 fp16, 128-byte swizzle, 8-row groups 1024
// bytes apart (stride-dimension offset); the leading-dimension offset is unused for this layout.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);        // start address, 16-byte units
    d |= (uint64_t)1 << 16;                          // leading-dimension byte offset (ignored), 16-byte units
    d |= (uint64_t)(1024u >> 4) << 32;               // stride-dimension byte offset
    d |= (uint64_t)1 << 46;                          // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                          // swizzle mode: 128 bytes
    return d;
}
// Instruction descriptor, kind::f16: D = f32, A = B = fp16, both K-major, M x N tile.
__host__ __device__ constexpr uint32_t idesc_f16(uint32_t m, uint32_t n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---- activations: f32 rows -> fp16, segment-major and pre-swizzled -------------------------------
// xt[(seg * m_pad + m) * 64 + ((c ^ (m & 7)) * 8) + e] = fp16(x[m][seg * 64 + c * 8 + e] * 2^-e_m), zero for
// m >= M or k >= K; post[m] = 2^e_m. One CTA per padded row.
__global__ void __launch_bounds__(256)
convert_rows_tiled_kernel(const float* __restrict__ x, __half* __restrict__ xt, float* __restrict__ post,
                          uint32_t M, uint32_t K, uint32_t m_pad, uint32_t n_seg) {
    __shared__ float red[8];
    __shared__ float s_pre;
    const uint32_t m = blockIdx.x;
    const bool real = m < M;
    const float* row = x + (size_t)(real ? m : 0) * K;
    float amax = 0.0f;
    if (real)
        for (uint32_t i = threadIdx.x; i < K; i += blockDim.x) amax = fmaxf(amax, fabsf(row[i]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float a = red[0];
        for (int w = 1; w < 8; ++w) a = fmaxf(a, red[w]);
        const int e = row_scale_exponent(a);
        s_pre = ldexpf(1.0f, -e);
        if (real) post[m] = ldexpf(1.0f, e);
    }
    __syncthreads();
    const float pre = s_pre;
    const uint32_t kp = n_seg * 64;  // padded K
    for (uint32_t k = threadIdx.x; k < kp; k += blockDim.x) {
        const uint32_t seg = k >> 6, c = (k >> 3) & 7u, e = k & 7u;
        const float v = (real && k < K) ? row[k] * pre : 0.0f;
        xt[((size_t)seg * m_pad + m) * 64 + ((c ^ (m & 7u)) << 3) + e] = __float2half_rn(v);
    }
}

// ---- weight dequantisation (same mapping as gemm.cu: a thread owns (row, half) of a quad) ---------
template <int TYPE>
struct PackedQuad {
    uint4 w0, w1, w2, w3;  // q4: w0, w1 = words 2*half, 2*half + 1; q8_0: words 4*half .. 4*half + 3 (of blocks 0..3)
    uint4 s;
};

template <int TYPE>
__device__ __forceinline__ void load_packed(PackedQuad<TYPE>& p, const uint8_t* qrow, const uint8_t* srow,
                                            uint32_t quad, uint32_t half) {
    if (TYPE == ZQ_TYPE_Q8_0) {
        const uint4* q = reinterpret_cast<const uint4*>(qrow + (size_t)quad * 128) + half * 4;
        p.w0 = __ldg(q); p.w1 = __ldg(q + 1); p.w2 = __ldg(q + 2); p.w3 = __ldg(q + 3);
    } else {
        const uint4* q = reinterpret_cast<const uint4*>(qrow + (size_t)quad * 64) + half * 2;
        p.w0 = __ldg(q); p.w1 = __ldg(q + 1);
    }
    if (TYPE == ZQ_TYPE_Q4_1) {
        p.s = __ldg(reinterpret_cast<const uint4*>(srow) + quad);
    } else {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(srow) + quad);
        p.s.x = v.x; p.s.y = v.y;
    }
}

__device__ __forceinline__ uint32_t pick4(const uint4& v, int j) {
    return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w;
}

template <int TYPE>
__device__ __forceinline__ void nibbles_to_half(uint32_t nib, uint32_t d2, uint32_t m2, uint32_t& h01,
                                                uint32_t& h23) {
    const uint32_t p01 = __byte_perm(nib, 0x64646464u, 0x5140);
    const uint32_t p23 = __byte_perm(nib, 0x64646464u, 0x5342);
    if (TYPE == ZQ_TYPE_Q4_0) {
        constexpr uint32_t k1032 = 0x64086408u;
        h01 = hmul2_u(hsub2_u(p01, k1032), d2);
        h23 = hmul2_u(hsub2_u(p23, k1032), d2);
    } else {
        constexpr uint32_t k1024 = 0x64006400u;
        h01 = hfma2_u(hsub2_u(p01, k1024), d2, m2);
        h23 = hfma2_u(hsub2_u(p23, k1024), d2, m2);
    }
}
__device__ __forceinline__ void bytes_to_half(uint32_t q, uint32_t d2, uint32_t& h01, uint32_t& h23) {
    const uint32_t u = q ^ 0x80808080u;
    constexpr uint32_t k1152 = 0x64806480u;
    h01 = hmul2_u(hsub2_u(__byte_perm(u, 0x64646464u, 0x5140), k1152), d2);
    h23 = hmul2_u(hsub2_u(__byte_perm(u, 0x64646464u, 0x5342), k1152), d2);
}

// Block j of the quad (j = JBASE + jj: the stage holds blocks JBASE and JBASE + 1) -> its 32 K-columns of the
// 64-K A tile. A thread owns (row, half, jj).
template <int TYPE, int JBASE>
__device__ __forceinline__ void store_dequant(const PackedQuad<TYPE>& p, uint32_t tile, uint32_t row, uint32_t half,
                                              uint32_t jj) {
    // select block j's words and scale without dynamic register indexing
    const uint32_t q0 = jj ? pick4(p.w0, JBASE + 1) : pick4(p.w0, JBASE);
    const uint32_t q1 = jj ? pick4(p.w1, JBASE + 1) : pick4(p.w1, JBASE);
    uint32_t d2, m2 = 0;
    if (TYPE == ZQ_TYPE_Q4_1) {
        const uint32_t dm = jj ? pick4(p.s, JBASE + 1) : pick4(p.s, JBASE);
        d2 = __byte_perm(dm, dm, 0x1010);
        m2 = __byte_perm(dm, dm, 0x3232);
    } else {
        const uint32_t pair = JBASE < 2 ? p.s.x : p.s.y;  // blocks (0, 1) or (2, 3)
        d2 = jj ? __byte_perm(pair, pair, 0x3232) : __byte_perm(pair, pair, 0x1010);
    }
    const uint32_t cbase = jj * 4;
    if (TYPE == ZQ_TYPE_Q8_0) {
        const uint32_t q2 = jj ? pick4(p.w2, JBASE + 1) : pick4(p.w2, JBASE);
        const uint32_t q3 = jj ? pick4(p.w3, JBASE + 1) : pick4(p.w3, JBASE);
        uint32_t h[8];
        bytes_to_half(q0, d2, h[0], h[1]);
        bytes_to_half(q1, d2, h[2], h[3]);
        bytes_to_half(q2, d2, h[4], h[5]);
        bytes_to_half(q3, d2, h[6], h[7]);
        sts128(tile + swz(row, cbase + half * 2), h[0], h[1], h[2], h[3]);
        sts128(tile + swz(row, cbase + half * 2 + 1), h[4], h[5], h[6], h[7]);
    } else {
        uint32_t lo[4], hi[4];
        nibbles_to_half<TYPE>(q0 & 0x0F0F0F0Fu, d2, m2, lo[0], lo[1]);
        nibbles_to_half<TYPE>(q1 & 0x0F0F0F0Fu, d2, m2, lo[2], lo[3]);
        nibbles_to_half<TYPE>((q0 >> 4) & 0x0F0F0F0Fu, d2, m2, hi[0], hi[1]);
        nibbles_to_half<TYPE>((q1 >> 4) & 0x0F0F0F0Fu, d2, m2, hi[2], hi[3]);
        sts128(tile + swz(row, cbase + half), lo[0], lo[1], lo[2], lo[3]);
        sts128(tile + swz(row, cbase + 2 + half), hi[0], hi[1], hi[2], hi[3]);
    }
}

template <int TYPE, int RT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const uint8_t* __restrict__ qs, const uint8_t* __restrict__ sc, const __half* __restrict__ xt,
               const float* __restrict__ post, float* __restrict__ y, uint32_t N, uint32_t K, uint32_t M,
               uint32_t m_pad, uint32_t nbp, uint32_t scp, uint32_t n_mma, uint32_t tmem_cols,
               unsigned int* err_word, TcEpilogue ep) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QB = Q8 ? 32 : 16;
    constexpr uint32_t SB = Q41 ? 4 : 2;
    constexpr uint32_t TC_STAGES = TcShape<RT>::kStages, TC_STAGE_BYTES = TcShape<RT>::kStageBytes;
    const uint32_t acc_cols = tmem_cols / RT;  // columns of one accumulator (a power of two >= n_mma)
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ __align__(8) unsigned long long bars[2 * TC_MAX_STAGES + 1];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    // operand tiles must start on a 1024-byte boundary (swizzle atoms); the launch adds the slack
    const uint32_t smem32 = ((uint32_t)__cvta_generic_to_shared(smem) + 1023u) & ~1023u;
    const uint32_t bar32 = (uint32_t)__cvta_generic_to_shared(bars);
    auto full_bar = [&](uint32_t s) { return bar32 + s * 8; };
    auto empty_bar = [&](uint32_t s) { return bar32 + (TC_STAGES + s) * 8; };
    const uint32_t acc_bar = bar32 + 2 * TC_STAGES * 8;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t n0 = blockIdx.x * (RT * TC_BN), m0 = blockIdx.y * n_mma;
    const uint32_t n_stages = nbp / 2;  // 64-K stages (the row padding to whole quads is zero weights)

    if (tid == 0) {
        for (uint32_t s = 0; s < TC_STAGES; ++s) {
            mbar_init(full_bar(s), TC_PRODUCERS / 32);  // one arrival per producer warp
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_PRODUCERS / 32) {  // the MMA warp owns the tensor-memory allocation
        const uint32_t slot = (uint32_t)__cvta_generic_to_shared(&tmem_base_slot);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_p = &abort_flag;

    if (warp < TC_PRODUCERS / 32) {
        // ================= producers =================
        const uint32_t prow = tid >> 2, phalf = (tid >> 1) & 1, pjj = tid & 1;
        const uint8_t* qrow[RT];
        const uint8_t* srow[RT];
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            const uint32_t wrow = min(n0 + r * TC_BN + prow, N - 1);
            qrow[r] = qs + (size_t)wrow * nbp * QB;
            srow[r] = sc + (size_t)wrow * scp * SB;
        }
        // packed words of the current quad and of the next one (loaded a whole quad ahead of their use)
        PackedQuad<TYPE> pk[RT], pk_next[RT];
        const uint32_t n_quads = nbp / 4;
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            load_packed<TYPE>(pk[r], qrow[r], srow[r], 0, phalf);
            if (n_quads > 1) load_packed<TYPE>(pk_next[r], qrow[r], srow[r], 1, phalf);
        }
        bool alive = true;
        for (uint32_t s = 0; s < n_stages && alive; ++s) {
            const uint32_t slot = s % TC_STAGES, round = s / TC_STAGES;
            if (round > 0) alive = mbar_wait(empty_bar(slot), (round - 1) & 1u, abort_p, err_word);
            if (!alive) break;
            const uint32_t a_tile = smem32 + slot * TC_STAGE_BYTES, b_tile = a_tile + RT * TC_A_BYTES;
            if ((tid & 31) == 0 && warp < 8) {
                // the stage's activation tile: n_mma rows x 128 bytes, contiguous in the converted image; eight
                // threads (one per warp) copy an eighth each so that several transfers are in flight
                const uint32_t bytes = n_mma * 16u;  // n_mma is a multiple of 64: a multiple of 1024 bytes
                const uint32_t off = warp * bytes;
                mbar_expect_tx(full_bar(slot), bytes);
                bulk_copy_g2s(b_tile + off, reinterpret_cast<const unsigned char*>(xt + ((size_t)s * m_pad + m0) * 64) + off,
                              bytes, full_bar(slot));
            }
#pragma unroll
            for (int r = 0; r < RT; ++r) {
                if ((s & 1u) == 0) {
                    store_dequant<TYPE, 0>(pk[r], a_tile + r * TC_A_BYTES, prow, phalf, pjj);
                } else {
                    store_dequant<TYPE, 2>(pk[r], a_tile + r * TC_A_BYTES, prow, phalf, pjj);
                    pk[r] = pk_next[r];
                    const uint32_t q_ahead = ((s + 1) >> 1) + 1;
                    if (q_ahead < n_quads) load_packed<TYPE>(pk_next[r], qrow[r], srow[r], q_ahead, phalf);
                }
            }
            fence_proxy_async();  // generic-proxy writes (st.shared) -> visible to the tensor core
            __syncwarp();         // every lane's stores and fence precede the warp's single arrival
            if (lane == 0) mbar_arrive(full_bar(slot));  // 16 arrivals per stage instead of 512 serialised ones
        }

        // ================= epilogue: drain tensor memory =================
        if (alive) alive = mbar_wait(acc_bar, 0, abort_p, err_word);
        tc_fence_after();
        if (alive) {
            // warp w reads lanes 32 * (w % 4) ..; the column chunks of 32 go round the four warp groups
            const uint32_t lane_base = (warp & 3) * 32;
#pragma unroll 1
            for (int r = 0; r < RT; ++r) {
                const uint32_t n = n0 + r * TC_BN + lane_base + lane;
                for (uint32_t c = (warp >> 2) * 32; c < n_mma; c += (TC_PRODUCERS / 128) * 32) {
                    uint32_t v32[32];
                    tc_ld32(tmem_base + (lane_base << 16) + r * acc_cols + c, v32);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const uint32_t m = m0 + c + i;
                        if (n < N && m < M) {
                            const size_t o = (size_t)m * N + n;
                            float v = __uint_as_float(v32[i]) * post[m];
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
        tc_fence_before();
    } else {
        // ================= MMA issuer =================
        if (lane == 0) {
            const uint32_t idesc = idesc_f16(TC_BN, n_mma);
            bool alive = true;
            for (uint32_t s = 0; s < n_stages && alive; ++s) {
                const uint32_t slot = s % TC_STAGES, round = s / TC_STAGES;
                alive = mbar_wait(full_bar(slot), round & 1u, abort_p, err_word);
                if (!alive) break;
                tc_fence_after();
                const uint32_t a_tile = smem32 + slot * TC_STAGE_BYTES, b_tile = a_tile + RT * TC_A_BYTES;
                const uint64_t b_desc = smem_desc_sw128(b_tile);
#pragma unroll
                for (uint32_t k16 = 0; k16 < TC_BK / 16; ++k16) {
                    // 16 fp16 = 32 bytes further along K inside the swizzle atom: +2 in 16-byte units
#pragma unroll
                    for (int r = 0; r < RT; ++r)
                        tc_mma_f16(tmem_base + r * acc_cols, smem_desc_sw128(a_tile + r * TC_A_BYTES) + 2 * k16,
                                   b_desc + 2 * k16, idesc, (s | k16) != 0 ? 1u : 0u);
                }
                tc_commit(empty_bar(slot));  // arrives when the MMAs issued so far have read their operands
            }
            if (alive) tc_commit(acc_bar);
            else *abort_p = 1;
        }
        __syncwarp();
    }

    __syncthreads();
    if (warp == TC_PRODUCERS / 32) {
        // If the pipeline was abandoned, MMAs may still be in flight: give the last commit a bounded chance.
        if (abort_flag && lane == 0) {
            tc_commit(acc_bar);
            for (uint32_t i = 0; i < kSpinLimit; ++i)
                if (mbar_try_wait(acc_bar, 0)) break;
        }
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// rows per CTA tile and padded row count for m_rows activation rows
inline void tc_tiling(uint32_t m_rows, uint32_t* n_mma, uint32_t* m_pad) {
    *n_mma = m_rows >= (uint32_t)TC_BM ? (uint32_t)TC_BM : ((m_rows + 63u) / 64u) * 64u;
    *m_pad = ((m_rows + *n_mma - 1) / *n_mma) * *n_mma;
}

template <int TYPE, int RT>
int launch_tc_rt(const zq_weight* w, const __half* xt, const float* post, float* y, uint32_t M, TcEpilogue ep,
                 cudaStream_t st) {
    auto kern = gemm_tc_kernel<TYPE, RT>;
    const size_t smem = (size_t)TcShape<RT>::kStages * TcShape<RT>::kStageBytes + 1024;  // + alignment slack
    ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // activation rows per CTA: a multiple of 64 (the epilogue splits the columns in two halves of 32s)
    uint32_t n_mma, m_pad;
    tc_tiling(M, &n_mma, &m_pad);
    uint32_t acc_cols = 64;
    while (acc_cols < n_mma) acc_cols *= 2;
    const uint32_t tmem_cols = acc_cols * RT;  // RT accumulators side by side
    const dim3 grid((w->out_dim + RT * TC_BN - 1) / (RT * TC_BN), m_pad / n_mma);
    unsigned int* err_word = nullptr;
    int rc = device_error_word(&err_word);
    if (rc != ZQ_OK) return rc;
    kern<<<grid, TC_THREADS, smem, st>>>(w->qs, static_cast<const uint8_t*>(w->sc), xt, post, y, w->out_dim,
                                          w->in_dim, M, m_pad, w->nbp, w->scp, n_mma, tmem_cols, err_word, ep);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

template <int TYPE>
int launch_tc(const zq_weight* w, const __half* xt, const float* post, float* y, uint32_t M, TcEpilogue ep,
              cudaStream_t st) {
    // Two 128-row tiles per CTA double the MMA work per stage hand-over (the loop that bounds this kernel);
    // they pay off when the paired tiles still cover about two thirds of the SMs (measured at 2048 rows:
    // 4096->14336 691 -> 738, 14336->4096 659 -> 776, head 518 -> 625 TFLOP/s; with 54-56 paired tiles the
    // single-tile form is 1.4x faster).
    uint32_t n_mma, m_pad;
    tc_tiling(M, &n_mma, &m_pad);
    const uint64_t paired = (uint64_t)((w->out_dim + 2 * TC_BN - 1) / (2 * TC_BN)) * (m_pad / n_mma);
    if (paired >= 100) return launch_tc_rt<TYPE, 2>(w, xt, post, y, M, ep, st);
    return launch_tc_rt<TYPE, 1>(w, xt, post, y, M, ep, st);
}

}  // namespace

size_t gemm_tc_workspace_bytes(const zq_weight* w, uint32_t m_rows) {
    uint32_t n_mma, m_pad;
    tc_tiling(m_rows, &n_mma, &m_pad);
    const size_t xb = ((size_t)(w->nbp / 2) * m_pad * 64 * sizeof(__half) + 255) & ~(size_t)255;
    const size_t pb = ((size_t)m_rows * sizeof(float) + 255) & ~(size_t)255;
    return xb + pb;
}

int launch_gemm_tc(const zq_weight* w, const float* x, float* y, uint32_t m_rows, const zq_epilogue* ep,
                   void* workspace, cudaStream_t st) {
    if (m_rows > 65535u * TC_BM) return ZQ_ERR_LIMIT;
    uint32_t n_mma, m_pad;
    tc_tiling(m_rows, &n_mma, &m_pad);
    const uint32_t n_seg = w->nbp / 2;
    const size_t xb = ((size_t)n_seg * m_pad * 64 * sizeof(__half) + 255) & ~(size_t)255;
    __half* xt = static_cast<__half*>(workspace);
    float* post = reinterpret_cast<float*>(static_cast<char*>(workspace) + xb);
    convert_rows_tiled_kernel<<<m_pad, 256, 0, st>>>(x, xt, post, m_rows, w->in_dim, m_pad, n_seg);
    ZQ_LAUNCH_CHECK();
    TcEpilogue a{nullptr, nullptr, nullptr, 0};
    if (ep) {
        a.bias = ep->d_bias;
        a.gelu = ep->gelu;
        a.mul = ep->d_mul;
        a.residual = ep->d_residual;
    }
    switch (w->type) {
        case ZQ_TYPE_Q4_0: return launch_tc<ZQ_TYPE_Q4_0>(w, xt, post, y, m_rows, a, st);
        case ZQ_TYPE_Q4_1: return launch_tc<ZQ_TYPE_Q4_1>(w, xt, post, y, m_rows, a, st);
        case ZQ_TYPE_Q8_0: return launch_tc<ZQ_TYPE_Q8_0>(w, xt, post, y, m_rows, a, st);
        default: return ZQ_ERR_UNSUPPORTED;
    }
}

}  // namespace zq
