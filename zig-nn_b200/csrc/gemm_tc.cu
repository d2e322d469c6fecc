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
#include <cuda.h>  // CUtensorMap and the enums of cuTensorMapEncodeTiled (the entry point is looked up at run time)

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
// One look, without waiting (try_wait may suspend the thread for a while when the phase is not complete).
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
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
                          uint32_t M, uint32_t K, uint32_t m_pad, uint32_t n_seg, uint32_t quarter_rows) {
    __shared__ float red[8];
    __shared__ float s_pre;
    // quarter_rows = 0: row m of x sits at place m of a segment. Otherwise (few rows, streaming form) the places are
    // four quarters of quarter_rows each and row m sits at place m / 4 of quarter m % 4, so that the rows spread
    // over the four lane quarters of tensor memory and all four draining warps have work.
    const uint32_t place = blockIdx.x;
    const uint32_t m = quarter_rows ? (place % quarter_rows) * 4u + place / quarter_rows : place;
    const uint32_t key = (quarter_rows ? place % quarter_rows : place) & 7u;  // swizzle key: the row's place in its tile
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
        xt[((size_t)seg * m_pad + place) * 64 + ((c ^ key) << 3) + e] = __float2half_rn(v);
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

// ---- weight-streaming form for few activation rows (up to 128) ------------------------------------
//
// With few activation rows the product is bound by the weight stream, not by the tensor-core rate. What was
// measured on the way to this form (vocabulary head, q4_0, 16 activation rows):
//   * one tcgen05.mma (kind::f16, K = 16) takes 127 cycles whatever its M (64, 128) and N (16 ... 256): with
//     the weights as the M operand (128 rows per instruction, N = the few activation rows) a 64-K stage costs
//     four instructions = 0.27 us for 128 weight rows, which alone is 67 us for the head. So the weights are the
//     N operand here (up to 256 rows per instruction) and the activations the M operand (128 rows, of which
//     only the first m_rows hold data; the rest of the tile is whatever lies in shared memory, and its
//     accumulator rows are never read);
//   * 512 threads fetching their own packed words from global memory put the fetch latency into every stage
//     hand-over and keep the load/store pipe busy with one wavefront per lane (32 lanes, 32 lines): 134 us;
//   * one plain bulk copy per row and 256 bytes: 35 ns of the copy engine apiece = 7 GB/s per SM: 195 us.
// The form that came out:
//   * the kernel is persistent: CTA b walks the tiles of TN weight rows b, b + grid, ...; every ring, the copies
//     and the MMA thread run on across tile boundaries;
//   * the packed quants and the scales come in by tensor copies (cp.async.bulk.tensor.2d over [rows][row bytes]
//     maps of the weight's two arrays; per chunk of 128 packed bytes per row: one box of TN rows x 128 bytes
//     with the 128-byte swizzle and one box of scales), issued by a copy warp three chunks ahead, bytes counted
//     on the chunk's mbarrier; nothing of it passes through the load pipe;
//   * the 16 converting warps turn a stage (64 K of the TN rows) into the fp16 tile together, reading packed
//     words and scales from shared memory (conflict-free through the swizzle);
//   * the stage's activation tile (rows x 128 bytes) is one bulk copy into a ring of its own, issued by a second
//     copy warp well ahead;
//   * two accumulators in tensor memory take turns; four more warps drain the finished one (tcgen05.ld, scale,
//     epilogue, 64-byte stores) while the next tile's stages flow.
// Every wait is bounded; on a timeout the kernel records it, all roles leave their loops and tensor memory is
// released.
constexpr int TS_CONVERT_WARPS = 16;
constexpr int TS_MMA_WARP = TS_CONVERT_WARPS;
constexpr int TS_EPI_WARP0 = TS_MMA_WARP + 1;   // four warps: their ids mod 4 cover the four lane quarters
constexpr int TS_COPY_WARP = TS_EPI_WARP0 + 4;   // packed chunks
constexpr int TS_XCOPY_WARP = TS_COPY_WARP + 1;  // activation tiles (a warp of its own: one warp serving both rings
                                                 // waits for a free slot of one while the other runs dry)
constexpr int TS_MMA_WARP2 = TS_XCOPY_WARP + 1;  // the second accumulator's issuer (more than 128 activation rows)
constexpr int TS_RELAY_WARP = TS_MMA_WARP2 + 1;  // a pair's second CTA: passes `weight tile full` on to the leader
constexpr int TS_THREADS = (TS_RELAY_WARP + 1) * 32;  // 25 warps
constexpr int TS_MAX_STAGES = 6;    // fp16 weight tiles (TN x 128 bytes each)
constexpr int TS_MAX_BTILES = 16;   // activation tiles
constexpr int TS_MAX_CHUNKS = 4;
constexpr uint32_t TS_ACT_ROWS = 128;   // rows of the activation operand (UMMA M)

// One box of a 2-D map: rows [y, y + box rows) x bytes [x, x + box bytes) -> shared memory, bytes counted on `bar`.
__device__ __forceinline__ void tensor_copy_2d(uint32_t dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t saddr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t saddr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(saddr));
    return v;
}
// Scale bytes of a row in a chunk's scale box. Chunks of 128 packed bytes per row: q4_0 16 (two quads), q4_1 32,
// q8_0 16 (the quad and its neighbour: a box is at least 16 bytes wide). Chunks of 64 bytes (one quad of q4):
// q4_0 16 (the quad and its neighbour), q4_1 16.
template <int TYPE, int CROW>
struct StreamScales {
    static constexpr uint32_t kBox = (TYPE == ZQ_TYPE_Q4_1 && CROW == 128) ? 32u : 16u;
};
// 16-byte unit c of row r in a box of 64-byte rows written with the 64-byte swizzle
__device__ __forceinline__ uint32_t swz64(uint32_t r, uint32_t c) { return r * 64u + ((c ^ ((r >> 1) & 3u)) << 4); }
// The thread's share of quad `ql` of the chunk: (row, half) -> packed words and the quad's scales. `sq` is the
// quad's place in the row's scale box.
template <int TYPE, int CROW>
__device__ __forceinline__ void read_packed(PackedQuad<TYPE>& p, uint32_t chunk, uint32_t scales, uint32_t row,
                                            uint32_t half, uint32_t ql, uint32_t sq) {
    constexpr uint32_t UNITS = TYPE == ZQ_TYPE_Q8_0 ? 8 : 4;   // 16-byte units per quad
    constexpr uint32_t MINE = UNITS / 2;                        // units of one half
    const uint32_t u0 = ql * UNITS + half * MINE;
    if (CROW == 64) {
        p.w0 = lds128(chunk + swz64(row, u0));
        p.w1 = lds128(chunk + swz64(row, u0 + 1));
    } else {
        p.w0 = lds128(chunk + swz(row, u0));
        p.w1 = lds128(chunk + swz(row, u0 + 1));
    }
    if (TYPE == ZQ_TYPE_Q8_0) {
        p.w2 = lds128(chunk + swz(row, u0 + 2));
        p.w3 = lds128(chunk + swz(row, u0 + 3));
    }
    if (TYPE == ZQ_TYPE_Q4_1) {
        p.s = lds128(scales + row * StreamScales<TYPE, CROW>::kBox + sq * 16u);
    } else {
        const uint2 v = lds64(scales + row * 16u + sq * 8u);
        p.s.x = v.x;
        p.s.y = v.y;
    }
}
// ---- a pair of CTAs (cluster of two) on one tile: tcgen05 with cta_group::2 ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of this CTA's shared address `addr` in CTA `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// The relays' arrival. What it orders is a tensor-core read of the relaying CTA's own shared memory after that CTA's
// writes (made visible to the asynchronous proxy by the writers' fences, observed by the relay through its own
// barrier): the leader's threads never read that memory, so no release of it to the leader is needed, and a
// releasing arrival at cluster scope costs the relay about a thousand cycles.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// a barrier that CTAs of the cluster arrive on
__device__ __forceinline__ uint32_t mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
__device__ __forceinline__ uint32_t mbar_test_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  unsigned int* err_word) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicExch(err_word, kErrGemmTimeout);
    return false;
}
// The leader's commit for the barrier at the same place in both CTAs: one commit per CTA, its own barrier by its
// shared address (valid in the cluster's window too), the other CTA's through the window.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mapa_shared(bar, 1))
                 : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 16 consecutive columns of f32
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// TN = weight rows per tile (UMMA N): 256, or 128 for matrices with too few rows to give every SM a 256-row tile.
// CROW = packed bytes per row and chunk: 128 (2 quads of q4, 1 of q8_0) or, for q4, 64 (1 quad: chunks a quarter
// of a stage pair smaller, which leaves room for a deeper ring of activation tiles).
//
// PAIR: two CTAs (a cluster) share a tile of 256 weight rows x 512 activation rows. Each converts ITS 128 weight
// rows (TN = 128) and copies ITS 128 rows of each activation tile; the leader's two issuing threads run
// tcgen05.mma.cta_group::2 (M = 256: 128 activation rows from each CTA; N = 256: 128 weight rows from each), each
// CTA's tensor memory receives the accumulator rows of its own activation rows. Per stage a CTA then moves 121 KB
// through its shared memory instead of 178 (it writes half the weight tile and every instruction reads 4 + 4 KB
// instead of 4 + 8), which is what bounded the single-CTA form. Barriers: the leader's `full` barriers count the
// converting warps of both CTAs (the other CTA's arrive through the cluster's shared window); the leader's
// activation barriers count its own copy and a relay thread of the other CTA, which waits for that CTA's copy;
// the leader commits to both CTAs' barriers; the other CTA's draining warps arrive on the leader's `accumulator
// free` barrier. Every copy is a plain one into the issuing CTA's own shared memory.
template <int TYPE, int TN, int CROW, bool PAIR>
__global__ void __launch_bounds__(TS_THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap smap,
                   const __half* __restrict__ xt, const float* __restrict__ post, float* __restrict__ y, uint32_t N,
                   uint32_t M, uint32_t nbp, uint32_t act_rows, uint32_t interleave, uint32_t n_act, uint32_t m_tiles,
                   uint32_t m_pad, uint32_t n_ring, uint32_t n_bring, uint32_t n_chunk_ring, uint32_t first_half,
                   const __half* __restrict__ wimg, uint32_t wimg_rows, unsigned int* err_word, TcEpilogue ep) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr uint32_t QB = Q8 ? 32 : 16;          // packed bytes per block
    constexpr uint32_t QUADB = 4 * QB;             // packed bytes per quad
    static_assert(CROW == 128 || (CROW == 64 && !Q8), "chunk rows: 128 bytes, or 64 for the 4-bit types");
    constexpr uint32_t CQ = CROW / QUADB;          // quads per chunk: 2 (q4) or 1 (q8_0; q4 with 64-byte chunks)
    constexpr bool PAIRED = CQ == 1 && TYPE != ZQ_TYPE_Q4_1;  // the scale box holds the quad's scales and its neighbour's
    constexpr uint32_t SBOX = StreamScales<TYPE, CROW>::kBox;
    static_assert(!PAIR || TN == 128, "a pair: 128 weight rows from each CTA");
    constexpr uint32_t ACC_N = PAIR ? 256u : (uint32_t)TN;  // columns of an accumulator = weight rows of a tile
    constexpr uint32_t ACT_TILE = PAIR ? 256u : TS_ACT_ROWS;  // activation rows of an accumulator (all CTAs together)
    constexpr uint32_t W_STAGE = TN * 128u;        // fp16 weight tile of a stage
    constexpr uint32_t CHUNK_BYTES = TN * CROW + TN * SBOX;  // packed box, then the scale box (both multiples of 1 KB)
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int NBARS = 2 * TS_MAX_STAGES + 2 * TS_MAX_BTILES + 2 * TS_MAX_CHUNKS + 4;
    __shared__ __align__(8) unsigned long long bars[NBARS];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ float epi_stage[4][32][17];  // per draining warp: a 32 x 16 block of outputs on its way to row-wise stores

    // shared memory: fp16 weight tiles | activation tiles | packed chunks (the activation operand spans 128 rows
    // from its tile's start whatever the tile holds: what lies behind the ring must be shared memory too)
    const uint32_t smem32 = ((uint32_t)__cvta_generic_to_shared(smem) + 1023u) & ~1023u;
    // Activation tiles. Natural order: tile k at k * rows * 128 bytes. Quarter-interleaved (up to 32 rows): a tile is
    // four pieces of 1 KB at 0, 4, 8 and 12 KB from its start, and tile k starts k KB into the region, so four tiles
    // fit into 19 KB.
    const uint32_t btile_bytes = act_rows * 128u;  // bytes of a stage in the activation image
    const uint32_t bstride = interleave ? 1024u : btile_bytes;
    const uint32_t bring_bytes = interleave ? 20u * 1024u : ((n_bring * btile_bytes + 1023u) & ~1023u);
    const uint32_t bring32 = smem32 + n_ring * W_STAGE;
    const uint32_t chunk32 = bring32 + bring_bytes;
    const uint32_t bar32 = (uint32_t)__cvta_generic_to_shared(bars);
    auto full_bar = [&](uint32_t s) { return bar32 + s * 8; };
    auto empty_bar = [&](uint32_t s) { return bar32 + (TS_MAX_STAGES + s) * 8; };
    auto bfull_bar = [&](uint32_t s) { return bar32 + (2 * TS_MAX_STAGES + s) * 8; };
    auto bempty_bar = [&](uint32_t s) { return bar32 + (2 * TS_MAX_STAGES + TS_MAX_BTILES + s) * 8; };
    constexpr int CB0 = 2 * TS_MAX_STAGES + 2 * TS_MAX_BTILES;
    auto cfull_bar = [&](uint32_t c) { return bar32 + (CB0 + c) * 8; };
    auto cempty_bar = [&](uint32_t c) { return bar32 + (CB0 + TS_MAX_CHUNKS + c) * 8; };
    auto acc_full = [&](uint32_t a) { return bar32 + (CB0 + 2 * TS_MAX_CHUNKS + a) * 8; };
    auto acc_empty = [&](uint32_t a) { return bar32 + (CB0 + 2 * TS_MAX_CHUNKS + 2 + a) * 8; };

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // A CTA tile = TN weight rows x n_act activation tiles of 128 rows (n_act = 2 for more than 128 activation rows:
    // both accumulators then belong to one tile). Tile t = blockIdx.x + i * gridDim.x covers weight tile t % row_tiles
    // and activation rows [t / row_tiles * 128 * n_act, ...).
    // A pair: the same with tiles of 256 weight rows x 2 activation tiles of 256 rows, walked by the cluster.
    const uint32_t crank = PAIR ? cluster_ctarank() : 0u;  // 0: the leader
    const uint32_t walker = PAIR ? blockIdx.x >> 1 : blockIdx.x, walkers = PAIR ? gridDim.x >> 1 : gridDim.x;
    const uint32_t row_tiles = (N + ACC_N - 1) / ACC_N;
    // A pair's last round: when it would hold tiles for at most half of the pairs, those tiles (from `first_half`
    // on) are each walked as two half tiles of one activation tile, by twice as many pairs in half the time.
    const uint32_t tiles_whole = row_tiles * m_tiles;
    const uint32_t tiles_total = tiles_whole + (PAIR ? tiles_whole - first_half : 0u);
    // tile t -> weight tile, its first activation tile (of ACT_TILE rows) and how many activation tiles it has
    auto tile_of = [&](uint32_t t, uint32_t& wt, uint32_t& at0, uint32_t& acnt) {
        uint32_t whole = t, half = 0;
        acnt = n_act;
        if (PAIR && t >= first_half) {
            const uint32_t h = t - first_half;
            whole = first_half + (h >> 1);
            half = h & 1u;
            acnt = 1;
        }
        const uint32_t mt = whole / row_tiles;
        wt = whole - mt * row_tiles;
        at0 = mt * n_act + half;
    };
    const uint32_t nt = tiles_total > walker ? (tiles_total - walker - 1) / walkers + 1 : 0;  // this CTA's (pair's) tiles
    const uint32_t n_quads = nbp / 4, n_stages = nbp / 2;
    const uint32_t n_chunks = (n_quads + CQ - 1) / CQ;  // per tile
    constexpr uint32_t tmem_cols = 2 * ACC_N;            // two accumulators

    if (tid == 0) {
        for (uint32_t s = 0; s < n_ring; ++s) {
            // one arrival per converting warp; a pair: the stage's activation tiles are counted on the same barrier
            // (the copy warp's arrival with their bytes), and the leader's also counts the other CTA's relay
            // (weights that arrive as fp16 tiles, `wimg`: no converting warps, the copy warp's arrival counts them too)
            mbar_init(full_bar(s), (wimg ? 0 : TS_CONVERT_WARPS) + (PAIR ? 1 : 0) + ((PAIR && crank == 0) ? 1 : 0));
            mbar_init(empty_bar(s), n_act);            // one commit per issuer
        }
        for (uint32_t s = 0; s < n_bring; ++s) {
            // the copy warp's arrival with the byte count; the leader's also counts the other CTA's relay
            mbar_init(bfull_bar(s), (PAIR && crank == 0) ? 2 : 1);
            mbar_init(bempty_bar(s), 1);
        }
        for (uint32_t c = 0; c < n_chunk_ring; ++c) {
            mbar_init(cfull_bar(c), 1);                   // the copy warp's arrival with the byte count
            mbar_init(cempty_bar(c), TS_CONVERT_WARPS);   // every converting warp, once per chunk
        }
        for (uint32_t a = 0; a < 2; ++a) {
            mbar_init(acc_full(a), a == 0 ? n_act : 1u);  // two activation tiles: both issuers commit to the first
            mbar_init(acc_empty(a), PAIR ? 8 : 4);  // one arrival per draining warp (of both CTAs)
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TS_MMA_WARP) {
        const uint32_t slot = (uint32_t)__cvta_generic_to_shared(&tmem_base_slot);
        if (PAIR) {  // the same warp of both CTAs
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(tmem_cols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(tmem_cols)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // both CTAs' barriers are initialised before either arrives on the other's
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abort_p = &abort_flag;

    if (warp < TS_CONVERT_WARPS) {
        // ================= converting warps =================
        // TN = 128: thread = (row, half, block of the stage); TN = 256: thread = (row, block), both halves in turn
        constexpr int HALVES = TN == 256 ? 2 : 1;
        const uint32_t prow = TN == 256 ? (uint32_t)tid >> 1 : (uint32_t)tid >> 2;
        const uint32_t phalf0 = TN == 256 ? 0u : ((uint32_t)tid >> 1) & 1u, pjj = (uint32_t)tid & 1u;
        uint32_t slot = 0, round = 0;      // stage ring
        uint32_t cslot = 0, cround = 0;    // chunk ring
        bool alive = true;
        for (uint32_t ti = 0; ti < (wimg ? 0u : nt) && alive; ++ti) {
            for (uint32_t c = 0; c < n_chunks && alive; ++c) {
                alive = mbar_wait(cfull_bar(cslot), cround & 1u, abort_p, err_word);
                if (!alive) break;
                const uint32_t nqc = min(CQ, n_quads - c * CQ);
                const uint32_t chunk = chunk32 + cslot * CHUNK_BYTES, scales = chunk + TN * CROW;
                for (uint32_t ql = 0; ql < nqc && alive; ++ql) {
                    const uint32_t sq = PAIRED ? (c & 1u) : ql;  // paired: the box holds the scales of quads c & ~1 and c | 1
                    PackedQuad<TYPE> pk[HALVES];
#pragma unroll
                    for (int hh = 0; hh < HALVES; ++hh)
                        read_packed<TYPE, CROW>(pk[hh], chunk, scales, prow, phalf0 + hh, ql, sq);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (round > 0) alive = alive && mbar_wait(empty_bar(slot), (round - 1) & 1u, abort_p, err_word);
                        if (!alive) break;
                        const uint32_t w_tile = smem32 + slot * W_STAGE;
#pragma unroll
                        for (int hh = 0; hh < HALVES; ++hh) {
                            if (h == 0) store_dequant<TYPE, 0>(pk[hh], w_tile, prow, phalf0 + hh, pjj);
                            else store_dequant<TYPE, 2>(pk[hh], w_tile, prow, phalf0 + hh, pjj);
                        }
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(full_bar(slot));
                        if (++slot == n_ring) {
                            slot = 0;
                            ++round;
                        }
                    }
                }
                // this warp has read what it needs of the chunk (its loads have returned: their values were used)
                __syncwarp();
                if (lane == 0) mbar_arrive(cempty_bar(cslot));
                if (++cslot == n_chunk_ring) {
                    cslot = 0;
                    ++cround;
                }
            }
        }
    } else if (warp == TS_COPY_WARP) {
        // ================= copy warp: packed quants and scales =================
        uint32_t cslot = 0, cround = 0;
        bool alive = true;
        for (uint32_t ti = 0; ti < (wimg ? 0u : nt) && alive; ++ti) {
            uint32_t wt, at0, acnt;
            tile_of(walker + ti * walkers, wt, at0, acnt);
            const uint32_t row0 = wt * ACC_N + crank * TN;
            for (uint32_t c = 0; c < n_chunks && alive; ++c) {
                if (cround > 0) alive = mbar_wait(cempty_bar(cslot), (cround - 1) & 1u, abort_p, err_word);
                alive = __all_sync(0xFFFFFFFFu, alive);
                if (!alive) break;
                if (lane == 0) {
                    // boxes are written whole (zeros beyond the map's edges)
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(cfull_bar(cslot)),
                                 "r"((uint32_t)TN * ((uint32_t)CROW + SBOX))
                                 : "memory");
                    const uint32_t dst0 = chunk32 + cslot * CHUNK_BYTES;
                    tensor_copy_2d(dst0, &wmap, c * (uint32_t)CROW, row0, cfull_bar(cslot));
                    const uint32_t sx = PAIRED ? (c & ~1u) * 8u : c * SBOX;
                    tensor_copy_2d(dst0 + TN * CROW, &smap, sx, row0, cfull_bar(cslot));
                }
                __syncwarp();
                if (++cslot == n_chunk_ring) {
                    cslot = 0;
                    ++cround;
                }
            }
        }
        if (!alive) {
            // copies already issued still land in this CTA's shared memory: wait (bounded) for the newest fill of
            // every slot before the CTA may retire
            for (uint32_t s = 0; s < n_chunk_ring; ++s)
                for (uint32_t i = 0; i < (1u << 16); ++i)
                    if (mbar_try_wait(cfull_bar(s), 0) || mbar_try_wait(cfull_bar(s), 1)) break;
        }
    } else if (warp == TS_XCOPY_WARP) {
        // ================= copy warp: the activation tiles of the stages =================
        uint32_t bslot = 0, bround = 0;
        bool alive = true;
        if (PAIR) {
            // A pair keeps one ring: slot s holds the stage's weight tile and, in the activation region, its two
            // activation tiles (32 KB from s * 32 KB), all counted on the stage's `full` barrier and freed by the
            // issuers' commits to its `empty` barrier. The issuers then look at one barrier per stage.
            uint32_t slot = 0, round = 0;
            for (uint32_t ti = 0; ti < nt && alive; ++ti) {
                uint32_t wt, at0, acnt;
                tile_of(walker + ti * walkers, wt, at0, acnt);
                for (uint32_t sg = 0; sg < n_stages && alive; ++sg) {
                    if (round > 0) alive = mbar_wait(empty_bar(slot), (round - 1) & 1u, abort_p, err_word);
                    alive = __all_sync(0xFFFFFFFFu, alive);
                    if (!alive) break;
                    if (lane == 0) {
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full_bar(slot)),
                                     "r"(acnt * btile_bytes + (wimg ? W_STAGE : 0u))
                                     : "memory");
                        if (wimg) {
                            // the stage's weight tile, already fp16 and in the operand's layout: this CTA's 128 rows
                            const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(wimg) +
                                                        ((size_t)sg * wimg_rows + (size_t)wt * ACC_N + crank * TN) * 128u;
                            bulk_copy_g2s(smem32 + slot * W_STAGE, wsrc, W_STAGE, full_bar(slot));
                        }
                        for (uint32_t a = 0; a < acnt; ++a) {
                            const unsigned char* src =
                                reinterpret_cast<const unsigned char*>(xt) +
                                ((size_t)sg * m_pad + ((size_t)at0 + a) * ACT_TILE + crank * TS_ACT_ROWS) * 128u;
                            bulk_copy_g2s(bring32 + (slot * 2 + a) * btile_bytes, src, btile_bytes, full_bar(slot));
                        }
                    }
                    __syncwarp();
                    if (++slot == n_ring) {
                        slot = 0;
                        ++round;
                    }
                }
            }
            if (!alive) {
                for (uint32_t s = 0; s < n_ring; ++s)
                    for (uint32_t i = 0; i < (1u << 16); ++i)
                        if (mbar_try_wait(full_bar(s), 0) || mbar_try_wait(full_bar(s), 1)) break;
            }
        }
        for (uint32_t ti = 0; ti < nt && alive && !PAIR; ++ti) {
            uint32_t wt, at0, acnt;
            tile_of(walker + ti * walkers, wt, at0, acnt);
            // one ring entry per stage and activation tile
            for (uint32_t sa = 0; sa < n_stages * n_act && alive; ++sa) {
                const uint32_t sg = n_act == 1 ? sa : sa >> 1, a = n_act == 1 ? 0u : sa & 1u;
                if (bround > 0) alive = mbar_wait(bempty_bar(bslot), (bround - 1) & 1u, abort_p, err_word);
                alive = __all_sync(0xFFFFFFFFu, alive);
                if (!alive) break;
                if (lane == 0) {
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bfull_bar(bslot)),
                                 "r"(btile_bytes)
                                 : "memory");
                    const unsigned char* src = reinterpret_cast<const unsigned char*>(xt) +
                                               ((size_t)sg * m_pad + ((size_t)at0 + a) * ACT_TILE + crank * TS_ACT_ROWS) * 128u;
                    if (interleave) {
                        for (uint32_t q = 0; q < 4; ++q)
                            bulk_copy_g2s(bring32 + bslot * bstride + q * 4096u, src + q * 1024u, 1024u, bfull_bar(bslot));
                    } else {
                        bulk_copy_g2s(bring32 + bslot * bstride, src, btile_bytes, bfull_bar(bslot));
                    }
                }
                __syncwarp();
                if (++bslot == n_bring) {
                    bslot = 0;
                    ++bround;
                }
            }
        }
        if (!alive && !PAIR) {
            for (uint32_t s = 0; s < n_bring; ++s)
                for (uint32_t i = 0; i < (1u << 16); ++i)
                    if (mbar_try_wait(bfull_bar(s), 0) || mbar_try_wait(bfull_bar(s), 1)) break;
        }
    } else if (warp == TS_RELAY_WARP) {
        // A pair's second CTA: when its 16 converting warps have filled a stage's weight tile and its copies of the
        // stage's activation tiles have landed, one arrival on the leader's barrier of that stage. (An arrival with cluster-wide release by every converting warp cost each of them
        // about a thousand cycles per stage, measured.)
        if (PAIR && crank != 0 && lane == 0) {
            uint32_t slot = 0, round = 0;
            bool alive = true;
            for (uint32_t e = 0; e < nt * n_stages && alive; ++e) {
                alive = mbar_wait(full_bar(slot), round & 1u, abort_p, err_word);
                if (!alive) break;
                mbar_arrive_cluster_relaxed(mapa_shared(full_bar(slot), 0));
                if (++slot == n_ring) {
                    slot = 0;
                    ++round;
                }
            }
            if (!alive) *abort_p = 1;
        }
        __syncwarp();
    } else if (warp == TS_MMA_WARP || warp == TS_MMA_WARP2) {
        // ================= MMA issuers: D[activation row][weight row] += X . W^T =================
        // Up to 128 activation rows: one issuer, the two accumulators take turns between tiles. More: both
        // accumulators belong to the tile and each has an issuer of its own (a thread of another warp). A look at a
        // barrier costs the issuing thread some 250 cycles while the tensor pipe holds little work in its queue
        // (measured: one thread issuing a stage's eight instructions and looking at three barriers spent 1430 + 970
        // cycles per stage); two threads look at theirs at the same time.
        const uint32_t me = warp == TS_MMA_WARP ? 0u : 1u;
        if (PAIR && crank != 0) {
            // the other CTA of a pair issues nothing
        } else if (lane == 0 && me < n_act) {
            const uint32_t idesc = idesc_f16(PAIR ? 256u : TS_ACT_ROWS, ACC_N);
            uint32_t slot = 0, round = 0, bslot = me, bround = 0;  // this issuer's ring entries: me, me + n_act, ...
            bool alive = true, ready = false;
            for (uint32_t i = 0; i < nt && alive; ++i) {
                uint32_t wt, at0, acnt;
                tile_of(walker + i * walkers, wt, at0, acnt);
                const bool mine = me < acnt;  // a half tile: the second issuer keeps step with the ring and issues nothing
                const uint32_t acc = n_act == 1 ? (i & 1u) : me;
                if (n_act == 1) {
                    if (i >= 2) alive = mbar_wait(acc_empty(acc), ((i >> 1) - 1) & 1u, abort_p, err_word);
                } else if (i >= 1) {
                    alive = PAIR ? mbar_wait_cluster(acc_empty(0), (i - 1) & 1u, abort_p, err_word)
                                 : mbar_wait(acc_empty(0), (i - 1) & 1u, abort_p, err_word);
                }
                if (!alive) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * ACC_N;
                for (uint32_t s = 0; s < n_stages && alive; ++s) {
                    if (!ready) {
                        if (PAIR) {
                            alive = mbar_wait_cluster(full_bar(slot), round & 1u, abort_p, err_word);
                        } else {
                            alive = mbar_wait(full_bar(slot), round & 1u, abort_p, err_word);
                            alive = alive && mbar_wait(bfull_bar(bslot), bround & 1u, abort_p, err_word);
                        }
                        if (!alive) break;
                    }
                    tc_fence_after();
                    const uint64_t w_desc = smem_desc_sw128(smem32 + slot * W_STAGE);
                    const uint64_t x_desc = smem_desc_sw128(PAIR ? bring32 + (slot * 2 + me) * btile_bytes : bring32 + bslot * bstride);
                    // the next stage's places in the rings (the rings run on across tiles)
                    uint32_t nslot = slot + 1, nround = round, nbslot = bslot + n_act, nbround = bround;
                    if (nslot == n_ring) {
                        nslot = 0;
                        ++nround;
                    }
                    if (nbslot >= n_bring) {
                        nbslot -= n_bring;
                        ++nbround;
                    }
                    // A look at a barrier takes this thread a few hundred cycles. Looking at the next stage's two
                    // barriers between this stage's instructions, while the tensor pipe still has those before
                    // them to run, keeps the looks off the pipe's critical path; a barrier that is not yet
                    // complete is waited for at the top of the next stage.
                    bool r1, r2;
                    if (PAIR) {
                        if (mine) {
                            tc_mma_f16_pair(d_tmem, x_desc, w_desc, idesc, s != 0 ? 1u : 0u);
                            tc_mma_f16_pair(d_tmem, x_desc + 2, w_desc + 2, idesc, 1u);
                            tc_mma_f16_pair(d_tmem, x_desc + 4, w_desc + 4, idesc, 1u);
                        }
                        r1 = mbar_test_wait_cluster(full_bar(nslot), nround & 1u);
                        r2 = true;
                        if (mine) tc_mma_f16_pair(d_tmem, x_desc + 6, w_desc + 6, idesc, 1u);
                        tc_commit_pair(empty_bar(slot));
                    } else {
                        tc_mma_f16(d_tmem, x_desc, w_desc, idesc, s != 0 ? 1u : 0u);
                        tc_mma_f16(d_tmem, x_desc + 2, w_desc + 2, idesc, 1u);
                        r1 = mbar_test_wait(full_bar(nslot), nround & 1u);
                        tc_mma_f16(d_tmem, x_desc + 4, w_desc + 4, idesc, 1u);
                        r2 = mbar_test_wait(bfull_bar(nbslot), nbround & 1u);
                        tc_mma_f16(d_tmem, x_desc + 6, w_desc + 6, idesc, 1u);
                        tc_commit(bempty_bar(bslot));
                        tc_commit(empty_bar(slot));
                    }
                    ready = r1 && r2;
                    slot = nslot, round = nround, bslot = nbslot, bround = nbround;
                }
                if (alive) {
                    if (PAIR) tc_commit_pair(acc_full(0));
                    else tc_commit(acc_full(n_act == 1 ? acc : 0u));
                }
            }
            if (!alive) *abort_p = 1;
        }
        __syncwarp();
    } else {
        // ================= epilogue warps: lane = activation row, columns = the tile's weight rows =================
        // A lane holds 16 consecutive outputs of ITS activation row: stored from there, the 32 lanes of a store hit
        // 32 rows of y, N floats apart, 16 bytes each (measured: 1.7-3 us per 16 columns, 32 us per tile, the whole
        // kernel waiting for it). So the 32 x 16 block is turned round in shared memory and each half-warp stores one
        // row's 64 contiguous bytes.
        const uint32_t lane_base = ((uint32_t)warp & 3u) * 32u;
        const uint32_t ew = (uint32_t)warp - TS_EPI_WARP0;
        float(*stage)[17] = epi_stage[ew];
        const uint32_t quarter = (uint32_t)warp & 3u;
        const uint32_t hr = (uint32_t)lane >> 4, hc = (uint32_t)lane & 15u;  // half-warp and column of the store pass
        const bool plain = !ep.bias && !ep.gelu && !ep.mul && !ep.residual;
        bool alive = true;
        for (uint32_t i = 0; i < nt && alive; ++i) {
            const uint32_t acc = n_act == 1 ? (i & 1u) : 0u;
            alive = mbar_wait(acc_full(acc), (n_act == 1 ? (i >> 1) : i) & 1u, abort_p, err_word);
            alive = __all_sync(0xFFFFFFFFu, alive);
            if (!alive) break;
            tc_fence_after();
            uint32_t wt, at0, acnt;
            tile_of(walker + i * walkers, wt, at0, acnt);
            const uint32_t n0 = wt * ACC_N;
            for (uint32_t a = 0; a < acnt; ++a) {
                // activation rows of this accumulator: lane j of this quarter holds row m0 + 4 j + quarter when
                // interleaved (up to 32 rows in all), m0 + 32 quarter + j otherwise
                const uint32_t m0 = (at0 + a) * ACT_TILE + crank * TS_ACT_ROWS;
                const uint32_t m = interleave ? 4u * (uint32_t)lane + quarter : m0 + lane_base + lane;
                const uint32_t first = interleave ? quarter : m0 + lane_base;  // first row of this quarter
                if (first >= M) continue;                                         // uniform over the warp
                const uint32_t rows_here = interleave ? min(8u, (M - quarter + 3u) / 4u) : min(32u, M - first);
                const float scale = (m < M && (!interleave || lane < 8)) ? post[m] : 0.0f;
                const uint32_t m_step = interleave ? 8u : 2u;
                const uint32_t m_first = interleave ? 4u * hr + quarter : first + hr;
                for (uint32_t c = 0; c < ACC_N; c += 16) {
                    if (n0 + c >= N) break;  // uniform over the warp
                    uint32_t v16[16];
                    tc_ld16(tmem_base + (lane_base << 16) + (acc + a) * ACC_N + c, v16);
                    tc_wait_ld();
#pragma unroll
                    for (int k = 0; k < 16; ++k) stage[lane][k] = __uint_as_float(v16[k]) * scale;
                    __syncwarp();
                    const uint32_t n = n0 + c + hc;
                    if (n < N) {
                        // half-warp hr takes the block's rows hr, hr + 2, ...: 64 contiguous bytes of one row of y per store
                        if (plain) {
                            float* dst = y + (size_t)m_first * N + n;
                            const size_t step = (size_t)m_step * N;
                            uint32_t r = hr;
#pragma unroll 1
                            for (; r + 6 < rows_here; r += 8) {
                                const float v0 = stage[r][hc], v1 = stage[r + 2][hc], v2 = stage[r + 4][hc], v3 = stage[r + 6][hc];
                                dst[0] = v0;
                                dst[step] = v1;
                                dst[2 * step] = v2;
                                dst[3 * step] = v3;
                                dst += 4 * step;
                            }
#pragma unroll 1
                            for (; r < rows_here; r += 2) {
                                dst[0] = stage[r][hc];
                                dst += step;
                            }
                        } else {
#pragma unroll 1
                            for (uint32_t r = hr, mr = m_first; r < rows_here; r += 2, mr += m_step) {
                                const size_t at = (size_t)mr * N + n;
                                float v = stage[r][hc];
                                if (ep.bias) v = __fadd_rn(v, ep.bias[n]);
                                if (ep.gelu) v = gelu_tanh(v);
                                if (ep.mul) v = __fmul_rn(v, ep.mul[at]);
                                if (ep.residual) v = __fadd_rn(ep.residual[at], v);
                                y[at] = v;
                            }
                        }
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(mapa_shared(acc_empty(0), 0));  // the leader's issuers wait for both CTAs
                else mbar_arrive(acc_empty(acc));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == TS_MMA_WARP && !PAIR) {
        if (abort_flag && lane == 0) {  // abandoned: give MMAs in flight a bounded chance to finish
            for (uint32_t a = 0; a < n_act; ++a) tc_commit(acc_full(0));
            for (uint32_t i = 0; i < kSpinLimit; ++i)
                if (mbar_try_wait(acc_full(0), 0) || mbar_try_wait(acc_full(0), 1)) break;
        }
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
    if (PAIR) {
        if (warp == TS_MMA_WARP && crank == 0 && abort_flag && lane == 0) {
            // abandoned: the leader gives the pair's instructions in flight a bounded chance to finish (the commits
            // reach both CTAs; a phase may already be complete, so either parity ends the wait)
            tc_commit_pair(acc_full(1));
            for (uint32_t i = 0; i < kSpinLimit; ++i)
                if (mbar_try_wait(acc_full(1), 0)) break;
        }
        __syncwarp();
        // Neither CTA retires, frees tensor memory or lets go of its shared memory while the other may still arrive
        // on its barriers or read its tiles: both have left their loops (every wait in them is bounded) first.
        cluster_sync_all();
        if (warp == TS_MMA_WARP) {
            tc_fence_after();
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
        }
    }
}

constexpr uint32_t kStreamMaxRows = 128;   // activation rows the streaming form takes
constexpr uint32_t kStreamMinTiles = 96;   // it needs about a tile per SM to pull the weight stream

// Up to 32 activation rows are spread over the four lane quarters of tensor memory (8 places each); more rows lie
// in their natural order, padded to 16.
inline uint32_t stream_quarter_rows(uint32_t m_rows) { return m_rows <= 32u ? 8u : 0u; }
inline uint32_t stream_act_rows(uint32_t m_rows) { return m_rows <= 32u ? 32u : ((m_rows + 15u) / 16u) * 16u; }

// The two arrays of a weight as 2-D maps for tensor copies: [out_dim rows][row bytes] of bytes, zeros beyond the
// edges. Quants: boxes of `box_rows` rows x 128 (64) bytes with the 128-byte (64-byte) swizzle; scales: boxes of the same rows x
// the scale bytes of a chunk, as stored. cuTensorMapEncodeTiled is a host-side computation; its entry point is
// taken from the driver at first use (the library does not link against libcuda).
int tensor_map_2d(const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes, uint32_t box_rows,
                  uint32_t swizzle_bytes, CUtensorMap* out) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        ZQ_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return ZQ_ERR_UNSUPPORTED;
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    if (((uintptr_t)base & 15u) || (row_bytes & 15u) || (box_bytes & 15u)) return ZQ_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                              : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                    : CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? ZQ_OK : ZQ_ERR_UNSUPPORTED;
}

// More than 128 activation rows: the same kernel with two activation tiles per CTA tile (256 weight rows x 256
// activation rows, both accumulators in use, an issuing thread for each). What bounds it is shared-memory traffic:
// per 64-K stage the converters write 32 KB and read 8, the copies write 42 and the eight tensor-core instructions
// read 96 (each reads its 4 KB of activations and 8 KB of weights), 178 KB = 1390 cycles at 128 bytes a cycle
// against 1016 cycles of tensor-core time; measured 1800 cycles per stage. Measured against the large-batch
// kernel (TFLOP/s, q4_0 unless noted): vocabulary head 1152 -> 262144 at 256 / 2048 rows 757 / 843;
// 4096 -> 14336 at 512 / 2048 / 4096 rows 606 / 776 / 899 against 562 / 707 / 824 (q8_0: 611 / 753 / 864 against
// 516 / 651 / 679); 1152 -> 6912 at 1024 / 4096 rows 332 / 563 against 276 / 451; 14336 -> 4096 at 2048 rows 738
// against 744. With fewer CTA tiles than about two thirds of the SMs it loses (4096 -> 14336 at 256 rows: 320
// against 399), so that is the rule.
inline bool stream_wide_takes(const zq_weight* w, uint32_t m_rows) {
    if (m_rows <= kStreamMaxRows) return false;
    const uint64_t tiles = (uint64_t)((w->out_dim + 255u) / 256u) * ((m_rows + 255u) / 256u);
    return tiles >= kStreamMinTiles;
}

template <int TYPE, int TN, int CROW>
int launch_stream_tn(const zq_weight* w, const __half* xt, const float* post, float* y, uint32_t M, TcEpilogue ep,
                     cudaStream_t st, uint32_t m_pad_given = 0) {
    auto kern = gemm_stream_kernel<TYPE, TN, CROW, false>;
    const bool wide = M > kStreamMaxRows;              // two activation tiles of 128 rows per CTA tile
    const uint32_t n_act = wide ? 2u : 1u;
    const uint32_t act_rows = wide ? TS_ACT_ROWS : stream_act_rows(M);  // rows of a ring entry
    const uint32_t m_tiles = wide ? (M + 255u) / 256u : 1u;
    // rows per K segment of the activation image: as this form pads them, or as the caller has laid the image out
    const uint32_t m_pad = (wide && m_pad_given >= m_tiles * 256u) ? m_pad_given : wide ? m_tiles * 256u : act_rows;
    const uint32_t btile_bytes = act_rows * 128u;
    constexpr uint32_t SBOX = StreamScales<TYPE, CROW>::kBox;
    constexpr uint32_t W_STAGE = TN * 128u, CHUNK_BYTES = TN * CROW + TN * SBOX;
    int dev = 0, max_smem = 0;
    ZQ_CUDA(cudaGetDevice(&dev));
    ZQ_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    // Shared memory: fp16 weight tiles, activation tiles, packed chunks. A weight tile is free again only when its
    // MMAs have run and their commit has arrived (half a microsecond after issue, measured), so up to 128
    // activation rows the ring of weight tiles is deep: four of 256 rows or six of 128 rows where that leaves
    // two chunks. With two activation tiles per stage the converters refill a weight tile (0.3 us) sooner than a
    // copy refills an activation tile (about a microsecond): two weight tiles, two chunks, and all the rest
    // activation tiles (measured with two stages of them: the copies' latency was half of every stage).
    const uint32_t budget = (uint32_t)max_smem - 1024u - 10240u;  // alignment slack, static shared memory
    const uint32_t interleave = (!wide && stream_quarter_rows(M)) ? 1u : 0u;
    uint32_t n_ring, n_bring, n_chunk_ring, bring_bytes;
    if (wide) {
        // An even number of activation tiles: entry e of the ring's sequence belongs to issuer e & 1, so with an
        // even ring a slot always serves the same issuer, in that issuer's own order. (With an odd ring a slot
        // changes hands every round, and the issuer that is ahead would find the parity it waits for already
        // there, left by the round before.)
        n_ring = 3;  // three weight tiles where that leaves four activation tiles (the 4-bit types), else two
        n_chunk_ring = 2;
        if (budget < n_ring * W_STAGE + n_chunk_ring * CHUNK_BYTES + 4u * btile_bytes) n_ring = 2;
        if (budget < n_ring * W_STAGE + n_chunk_ring * CHUNK_BYTES + 4u * btile_bytes) return ZQ_ERR_UNSUPPORTED;
        n_bring = (budget - n_ring * W_STAGE - n_chunk_ring * CHUNK_BYTES) / btile_bytes;
        if (n_bring > (uint32_t)TS_MAX_BTILES) n_bring = TS_MAX_BTILES;
        n_bring &= ~1u;
        bring_bytes = n_bring * btile_bytes;  // 16 KB each
    } else {
        n_bring = (16u * 1024u) / btile_bytes;
        if (n_bring > (uint32_t)TS_MAX_BTILES) n_bring = TS_MAX_BTILES;
        if (n_bring < 2) n_bring = 2;
        if (n_bring < 3 && btile_bytes <= 8192u) n_bring = 3;
        if (interleave) n_bring = 4;
        bring_bytes = interleave ? 20u * 1024u : ((n_bring * btile_bytes + 1023u) & ~1023u);
        n_ring = TN == 256 ? 4 : 6;
        while (n_ring > 2 && budget < bring_bytes + n_ring * W_STAGE + 2 * CHUNK_BYTES) --n_ring;
        if (budget < bring_bytes + n_ring * W_STAGE + 2 * CHUNK_BYTES) return ZQ_ERR_UNSUPPORTED;
        n_chunk_ring = (budget - bring_bytes - n_ring * W_STAGE) / CHUNK_BYTES;
        if (n_chunk_ring > (uint32_t)TS_MAX_CHUNKS) n_chunk_ring = TS_MAX_CHUNKS;
    }
    const size_t smem = (size_t)n_ring * W_STAGE + bring_bytes + (size_t)n_chunk_ring * CHUNK_BYTES + 1024;
    ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const uint32_t row_tiles = (w->out_dim + TN - 1) / TN;
    const uint64_t tiles_total = (uint64_t)row_tiles * m_tiles;
    const uint32_t sms = (uint32_t)sm_count();
    const uint32_t grid = tiles_total < sms ? (uint32_t)tiles_total : sms;
    unsigned int* err_word = nullptr;
    int rc = device_error_word(&err_word);
    if (rc != ZQ_OK) return rc;
    constexpr uint32_t SB = TYPE == ZQ_TYPE_Q4_1 ? 4 : 2;
    CUtensorMap wmap, smap;
    rc = tensor_map_2d(w->qs, (uint64_t)w->nbp * w->qb, w->out_dim, CROW, TN, CROW, &wmap);
    if (rc == ZQ_OK) rc = tensor_map_2d(w->sc, (uint64_t)w->scp * SB, w->out_dim, SBOX, TN, 0, &smap);
    if (rc != ZQ_OK) return rc;
    kern<<<grid, TS_THREADS, smem, st>>>(wmap, smap, xt, post, y, w->out_dim, M, w->nbp, act_rows, interleave, n_act, m_tiles,
                                         m_pad, n_ring, n_bring, n_chunk_ring, (uint32_t)tiles_total, nullptr, 0u, err_word, ep);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

// A pair of CTAs per tile of 256 weight rows x 512 activation rows (see the kernel). 74 pairs walk the tiles.
constexpr uint32_t kPairActRows = 512;
int g_cluster_launch = 1;  // zq_set_cluster_launch
// Measured against the single-CTA form with two activation tiles and the large-batch kernel (TFLOP/s, q4_0 unless
// noted): 4096 -> 14336 at 512 / 1024 / 2048 / 4096 rows 742 / 868 / 943 / 1081 against 606 / 713 / 776 / 899 and
// 562 / 638 / 707 / 824 (q8_0 at 4096 rows: 1021 against 864 and 679); 14336 -> 4096 at 2048 / 4096 rows 876 / 928
// against 738 / 774 and 744 / 788; vocabulary head 1152 -> 262144 at 512 / 2048 rows 917 / 953 against 818 / 843;
// 1152 -> 6912 at 1024 / 4096 rows 343 / 594 against 332 / 563. It loses where half of its 512-row activation tile
// is empty (head at 256 rows: 577 against 757), where the pairs get fewer than about 48 tiles (14336 -> 4096 at 1024
// rows: 32 tiles, 533 against 561 of the large-batch kernel) and by a little on short K, where the drain of the
// accumulators outweighs the stages (768 -> 50257 at 4096 rows: 611 against 656).
inline bool stream_pair_takes(const zq_weight* w, uint32_t m_rows) {
    if (m_rows <= 256u || w->in_dim < 1024u) return false;
    const uint64_t tiles = (uint64_t)((w->out_dim + 255u) / 256u) * ((m_rows + kPairActRows - 1) / kPairActRows);
    return tiles >= 48;
}

template <int TYPE>
int launch_stream_pair(const zq_weight* w, const __half* xt, const float* post, float* y, uint32_t M, TcEpilogue ep,
                       cudaStream_t st) {
    constexpr int TN = 128, CROW = TYPE == ZQ_TYPE_Q8_0 ? 128 : 64;
    auto kern = gemm_stream_kernel<TYPE, TN, CROW, true>;
    const uint32_t n_act = 2, act_rows = TS_ACT_ROWS;
    const uint32_t m_tiles = (M + kPairActRows - 1) / kPairActRows, m_pad = m_tiles * kPairActRows;
    const uint32_t btile_bytes = act_rows * 128u;
    constexpr uint32_t SBOX = StreamScales<TYPE, CROW>::kBox;
    constexpr uint32_t W_STAGE = TN * 128u, CHUNK_BYTES = TN * CROW + TN * SBOX;
    int dev = 0, max_smem = 0;
    ZQ_CUDA(cudaGetDevice(&dev));
    ZQ_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    const uint32_t budget = (uint32_t)max_smem - 1024u - 10240u;  // alignment slack, static shared memory
    // one ring: a stage's weight tile (16 KB) and its two activation tiles (32 KB); two chunks (20-36 KB)
    const uint32_t n_chunk_ring = 2;
    uint32_t n_ring = (budget - n_chunk_ring * CHUNK_BYTES) / (W_STAGE + 2u * btile_bytes);  // 4 (q4) or 3 (q8_0)
    if (n_ring > (uint32_t)TS_MAX_STAGES) n_ring = TS_MAX_STAGES;
    if (n_ring < 2) return ZQ_ERR_UNSUPPORTED;
    const uint32_t n_bring = 2u * n_ring;
    const size_t smem = (size_t)n_ring * W_STAGE + (size_t)n_bring * btile_bytes + (size_t)n_chunk_ring * CHUNK_BYTES + 1024;
    ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const uint64_t tiles_whole = (uint64_t)((w->out_dim + 255u) / 256u) * m_tiles;
    if (tiles_whole > 0x7FFFFFFFu) return ZQ_ERR_LIMIT;
    const uint32_t pairs_max = (uint32_t)sm_count() / 2u;
    // the tiles of a last round that would occupy at most half of the pairs are walked as half tiles (see the kernel)
    const uint32_t rest = tiles_whole > pairs_max ? (uint32_t)(tiles_whole % pairs_max) : 0u;
    const uint32_t first_half = (rest > 0 && rest <= pairs_max / 2u) ? (uint32_t)tiles_whole - rest : (uint32_t)tiles_whole;
    const uint64_t tiles_total = tiles_whole + (tiles_whole - first_half);
    const uint32_t pairs = tiles_total < pairs_max ? (uint32_t)tiles_total : pairs_max;
    unsigned int* err_word = nullptr;
    int rc = device_error_word(&err_word);
    if (rc != ZQ_OK) return rc;
    constexpr uint32_t SB = TYPE == ZQ_TYPE_Q4_1 ? 4 : 2;
    CUtensorMap wmap, smap;
    rc = tensor_map_2d(w->qs, (uint64_t)w->nbp * w->qb, w->out_dim, CROW, TN, CROW, &wmap);
    if (rc == ZQ_OK) rc = tensor_map_2d(w->sc, (uint64_t)w->scp * SB, w->out_dim, SBOX, TN, 0, &smap);
    if (rc != ZQ_OK) return rc;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2u * pairs);
    cfg.blockDim = dim3(TS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ZQ_CUDA(cudaLaunchKernelEx(&cfg, kern, wmap, smap, xt, post, y, w->out_dim, M, w->nbp, act_rows, 0u, n_act, m_tiles, m_pad,
                               n_ring, n_bring, n_chunk_ring, first_half, static_cast<const __half*>(nullptr), 0u, err_word, ep));
    return ZQ_OK;
}

template <int TYPE>
int launch_stream(const zq_weight* w, const __half* xt, const float* post, float* y, uint32_t M, TcEpilogue ep,
                  cudaStream_t st) {
    if (stream_pair_takes(w, M)) {
        const int rc = g_cluster_launch ? launch_stream_pair<TYPE>(w, xt, post, y, M, ep, st) : ZQ_ERR_CUDA;
        if (rc != ZQ_ERR_CUDA) return rc;
        // The launch of the pairs was refused (nothing ran; a partitioned GPU may not schedule clusters) or is
        // switched off: the single-CTA form takes the call, on the activation image as it is laid out for the
        // pairs (rows padded to 512s).
        if (g_cluster_launch) cudaGetLastError();
        return launch_stream_tn<TYPE, 256, TYPE == ZQ_TYPE_Q8_0 ? 128 : 64>(w, xt, post, y, M, ep, st,
                                                                             ((M + kPairActRows - 1) / kPairActRows) * kPairActRows);
    }
    // More than 128 activation rows: 64-byte chunks for the 4-bit types (room for seven activation tiles instead
    // of four). Otherwise 256-row tiles do twice the work per tensor-core instruction; 128-row tiles when those
    // would leave SMs idle.
    if (M > kStreamMaxRows) return launch_stream_tn<TYPE, 256, TYPE == ZQ_TYPE_Q8_0 ? 128 : 64>(w, xt, post, y, M, ep, st);
    if ((w->out_dim + 255u) / 256u >= (uint32_t)sm_count()) return launch_stream_tn<TYPE, 256, 128>(w, xt, post, y, M, ep, st);
    return launch_stream_tn<TYPE, 128, 128>(w, xt, post, y, M, ep, st);
}

inline bool stream_takes(const zq_weight* w, uint32_t m_rows) {
    if (m_rows > kStreamMaxRows) return stream_pair_takes(w, m_rows) || stream_wide_takes(w, m_rows);
    return (w->out_dim + TC_BN - 1) / TC_BN >= kStreamMinTiles;
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

// ---- the transposed product on the pair form: grad_x[M][K] = grad_out[M][N] . W[N][K] --------------------------
// The contraction runs over the weight ROWS, so the operand the tensor cores need is W^T: rows = the K output
// columns, 64 contraction values (weight rows) per stage. It is built once per call as fp16 tiles in the operand's
// layout (the values the forward kernel's converting warps produce, transposed): segment s = weight rows
// [64 s, 64 s + 64), row k of the segment = 128 bytes = W[64 s .. 64 s + 63][k], 16-byte pieces swizzled by k & 7.
// A CTA's weight tile of a stage is then 16 contiguous KB and arrives by one bulk copy on the stage's barrier; the
// pair kernel runs without converting warps and chunks.
template <int TYPE>
__global__ void __launch_bounds__(256)
weights_to_image_kernel(const uint8_t* __restrict__ qs, const void* __restrict__ sc, __half* __restrict__ wimg, uint32_t N,
                        uint32_t nb, uint32_t nbp, uint32_t scp, uint32_t rows_pad) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr uint32_t QB = Q8 ? 32 : 16;
    __shared__ __align__(16) __half tile[128][72];  // [k within the quad][weight row within the segment], rows of 144 bytes
    const uint32_t quad = blockIdx.x, seg = blockIdx.y;
    const uint32_t t = threadIdx.x, nl = t >> 2, j = t & 3u;  // weight row of the segment, block of the quad
    const uint32_t n = seg * 64u + nl, blk = quad * 4u + j;
    if (n < N && blk < nb) {
        const uint8_t* qrow = qs + (size_t)n * nbp * QB;
        __half d, mn = __float2half_rn(0.0f);
        if (TYPE == ZQ_TYPE_Q4_1) {
            const __half2 dm = reinterpret_cast<const __half2*>(sc)[(size_t)n * scp + blk];
            d = __low2half(dm);
            mn = __high2half(dm);
        } else {
            d = reinterpret_cast<const __half*>(sc)[(size_t)n * scp + blk];
        }
        if (Q8) {
#pragma unroll
            for (uint32_t wd = 0; wd < 8; ++wd) {
                const uint32_t word = *reinterpret_cast<const uint32_t*>(qrow + qs_word_offset(32, blk, wd));
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    const int q = (int)(int8_t)((word >> (8 * i)) & 0xFFu);
                    tile[j * 32 + wd * 4 + i][nl] = __hmul(__int2half_rn(q), d);
                }
            }
        } else {
#pragma unroll
            for (uint32_t wd = 0; wd < 4; ++wd) {
                const uint32_t word = *reinterpret_cast<const uint32_t*>(qrow + qs_word_offset(16, blk, wd));
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) {
                    const int lo = (int)((word >> (8 * i)) & 0xFu), hi = (int)((word >> (8 * i + 4)) & 0xFu);
                    if (TYPE == ZQ_TYPE_Q4_0) {
                        tile[j * 32 + wd * 4 + i][nl] = __hmul(__int2half_rn(lo - 8), d);
                        tile[j * 32 + 16 + wd * 4 + i][nl] = __hmul(__int2half_rn(hi - 8), d);
                    } else {
                        tile[j * 32 + wd * 4 + i][nl] = __hfma(__int2half_rn(lo), d, mn);
                        tile[j * 32 + 16 + wd * 4 + i][nl] = __hfma(__int2half_rn(hi), d, mn);
                    }
                }
            }
        }
    } else {
#pragma unroll
        for (uint32_t e = 0; e < 32; ++e) tile[j * 32 + e][nl] = __float2half_rn(0.0f);
    }
    __syncthreads();
    for (uint32_t i = t; i < 128u * 8u; i += 256u) {
        const uint32_t k = i >> 3, c = i & 7u, krow = quad * 128u + k;
        if (krow >= rows_pad) continue;
        const uint4 v = *reinterpret_cast<const uint4*>(&tile[k][c * 8]);
        *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(wimg) + ((size_t)seg * rows_pad + krow) * 128u +
                                  ((c ^ (krow & 7u)) << 4)) = v;
    }
}

inline uint32_t trans_rows_pad(const zq_weight* w) { return ((w->in_dim + 255u) / 256u) * 256u; }  // K output columns, in tiles
inline uint32_t trans_m_pad(uint32_t m_rows) { return ((m_rows + kPairActRows - 1) / kPairActRows) * kPairActRows; }

// Taken where the pair form pays (as in stream_pair_takes, with the roles of the dimensions exchanged) and the
// weight rows are whole quads of the contraction.
bool trans_pair_takes(const zq_weight* w, uint32_t m_rows) {
    if (!g_cluster_launch || m_rows <= 256u || w->out_dim < 1024u || (w->out_dim & 127u) != 0) return false;
    const uint64_t tiles = (uint64_t)(trans_rows_pad(w) / 256u) * (trans_m_pad(m_rows) / kPairActRows);
    return tiles >= 48;
}

size_t trans_pair_workspace_bytes(const zq_weight* w, uint32_t m_rows) {
    const size_t n_seg = w->out_dim / 64;
    const size_t xb = n_seg * trans_m_pad(m_rows) * 128;                         // grad_out as activation tiles
    const size_t pb = ((size_t)m_rows * sizeof(float) + 255) & ~(size_t)255;     // its row scales
    const size_t wb = n_seg * trans_rows_pad(w) * 128;                           // W^T as weight tiles
    return xb + pb + wb;
}

int launch_trans_pair(const zq_weight* w, const float* grad_out, float* grad_x, uint32_t M, int accumulate, void* workspace,
                      cudaStream_t st) {
    const uint32_t N = w->out_dim, K = w->in_dim, n_seg = N / 64, m_pad = trans_m_pad(M), rows_pad = trans_rows_pad(w);
    const size_t xb = (size_t)n_seg * m_pad * 128;
    const size_t pb = ((size_t)M * sizeof(float) + 255) & ~(size_t)255;
    __half* xt = static_cast<__half*>(workspace);
    float* post = reinterpret_cast<float*>(static_cast<char*>(workspace) + xb);
    __half* wimg = reinterpret_cast<__half*>(static_cast<char*>(workspace) + xb + pb);
    convert_rows_tiled_kernel<<<m_pad, 256, 0, st>>>(grad_out, xt, post, M, N, m_pad, n_seg, 0u);
    ZQ_LAUNCH_CHECK();
    const dim3 wgrid(rows_pad / 128u, n_seg);
    switch (w->type) {
        case ZQ_TYPE_Q4_0:
            weights_to_image_kernel<ZQ_TYPE_Q4_0><<<wgrid, 256, 0, st>>>(w->qs, w->sc, wimg, N, w->nb, w->nbp, w->scp, rows_pad);
            break;
        case ZQ_TYPE_Q4_1:
            weights_to_image_kernel<ZQ_TYPE_Q4_1><<<wgrid, 256, 0, st>>>(w->qs, w->sc, wimg, N, w->nb, w->nbp, w->scp, rows_pad);
            break;
        case ZQ_TYPE_Q8_0:
            weights_to_image_kernel<ZQ_TYPE_Q8_0><<<wgrid, 256, 0, st>>>(w->qs, w->sc, wimg, N, w->nb, w->nbp, w->scp, rows_pad);
            break;
        default: return ZQ_ERR_UNSUPPORTED;
    }
    ZQ_LAUNCH_CHECK();

    // the pair kernel without converting warps and chunks: any instantiation serves (nothing of the weight's type is
    // left in it); one ring of weight tile + two activation tiles per stage
    constexpr int TN = 128;
    auto kern = gemm_stream_kernel<ZQ_TYPE_Q4_0, TN, 64, true>;
    const uint32_t m_tiles = m_pad / kPairActRows, btile_bytes = TS_ACT_ROWS * 128u;
    constexpr uint32_t W_STAGE = TN * 128u;
    int dev = 0, max_smem = 0;
    ZQ_CUDA(cudaGetDevice(&dev));
    ZQ_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    const uint32_t budget = (uint32_t)max_smem - 1024u - 10240u;
    uint32_t n_ring = budget / (W_STAGE + 2u * btile_bytes);
    if (n_ring > (uint32_t)TS_MAX_STAGES) n_ring = TS_MAX_STAGES;
    if (n_ring < 2) return ZQ_ERR_UNSUPPORTED;
    const uint32_t n_bring = 2u * n_ring;
    const size_t smem = (size_t)n_ring * W_STAGE + (size_t)n_bring * btile_bytes + 1024;
    ZQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const uint64_t tiles_whole = (uint64_t)(rows_pad / 256u) * m_tiles;
    if (tiles_whole > 0x7FFFFFFFu) return ZQ_ERR_LIMIT;
    const uint32_t pairs_max = (uint32_t)sm_count() / 2u;
    const uint32_t rest = tiles_whole > pairs_max ? (uint32_t)(tiles_whole % pairs_max) : 0u;
    const uint32_t first_half = (rest > 0 && rest <= pairs_max / 2u) ? (uint32_t)tiles_whole - rest : (uint32_t)tiles_whole;
    const uint64_t tiles_total = tiles_whole + (tiles_whole - first_half);
    const uint32_t pairs = tiles_total < pairs_max ? (uint32_t)tiles_total : pairs_max;
    unsigned int* err_word = nullptr;
    int rc = device_error_word(&err_word);
    if (rc != ZQ_OK) return rc;
    TcEpilogue ep{nullptr, nullptr, nullptr, 0};
    if (accumulate) ep.residual = grad_x;  // the reference's kernels add to grad_x
    CUtensorMap none;
    memset(&none, 0, sizeof(none));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2u * pairs);
    cfg.blockDim = dim3(TS_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ZQ_CUDA(cudaLaunchKernelEx(&cfg, kern, none, none, static_cast<const __half*>(xt), static_cast<const float*>(post), grad_x, K, M,
                               N / 32u, (uint32_t)TS_ACT_ROWS, 0u, 2u, m_tiles, m_pad, n_ring, n_bring, 0u, first_half,
                               static_cast<const __half*>(wimg), rows_pad, err_word, ep));
    return ZQ_OK;
}

}  // namespace

bool gemm_stream_takes(const zq_weight* w, uint32_t m_rows) { return stream_takes(w, m_rows); }

bool gemm_trans_pair_takes(const zq_weight* w, uint32_t m_rows) { return trans_pair_takes(w, m_rows); }
size_t gemm_trans_pair_workspace_bytes(const zq_weight* w, uint32_t m_rows) { return trans_pair_workspace_bytes(w, m_rows); }
int launch_gemm_trans_pair(const zq_weight* w, const float* grad_out, float* grad_x, uint32_t m_rows, int accumulate,
                           void* workspace, cudaStream_t st) {
    return launch_trans_pair(w, grad_out, grad_x, m_rows, accumulate, workspace, st);
}

size_t gemm_tc_workspace_bytes(const zq_weight* w, uint32_t m_rows) {
    uint32_t n_mma, m_pad;
    tc_tiling(m_rows, &n_mma, &m_pad);  // never less than the streaming form's padding to 16 rows ...
    if (m_rows > 128 && m_pad < ((m_rows + 511u) / 512u) * 512u) m_pad = ((m_rows + 511u) / 512u) * 512u;  // ... or to 512
    const size_t xb = ((size_t)(w->nbp / 2) * m_pad * 64 * sizeof(__half) + 255) & ~(size_t)255;
    const size_t pb = ((size_t)m_rows * sizeof(float) + 255) & ~(size_t)255;
    return xb + pb;
}

int launch_gemm_tc(const zq_weight* w, const float* x, float* y, uint32_t m_rows, const zq_epilogue* ep,
                   void* workspace, cudaStream_t st) {
    if (m_rows > 65535u * TC_BM) return ZQ_ERR_LIMIT;
    uint32_t n_mma, m_pad;
    tc_tiling(m_rows, &n_mma, &m_pad);
    const bool stream = stream_takes(w, m_rows);
    if (stream) {
        m_pad = m_rows <= kStreamMaxRows ? stream_act_rows(m_rows)
                : stream_pair_takes(w, m_rows) ? ((m_rows + kPairActRows - 1) / kPairActRows) * kPairActRows
                                               : ((m_rows + 255u) / 256u) * 256u;
    }
    const uint32_t n_seg = w->nbp / 2;
    const size_t xb = ((size_t)n_seg * m_pad * 64 * sizeof(__half) + 255) & ~(size_t)255;
    __half* xt = static_cast<__half*>(workspace);
    float* post = reinterpret_cast<float*>(static_cast<char*>(workspace) + xb);
    convert_rows_tiled_kernel<<<m_pad, 256, 0, st>>>(x, xt, post, m_rows, w->in_dim, m_pad, n_seg,
                                                     stream ? stream_quarter_rows(m_rows) : 0u);
    ZQ_LAUNCH_CHECK();
    TcEpilogue a{nullptr, nullptr, nullptr, 0};
    if (ep) {
        a.bias = ep->d_bias;
        a.gelu = ep->gelu;
        a.mul = ep->d_mul;
        a.residual = ep->d_residual;
    }
    if (stream) {
        switch (w->type) {
            case ZQ_TYPE_Q4_0: return launch_stream<ZQ_TYPE_Q4_0>(w, xt, post, y, m_rows, a, st);
            case ZQ_TYPE_Q4_1: return launch_stream<ZQ_TYPE_Q4_1>(w, xt, post, y, m_rows, a, st);
            case ZQ_TYPE_Q8_0: return launch_stream<ZQ_TYPE_Q8_0>(w, xt, post, y, m_rows, a, st);
            default: return ZQ_ERR_UNSUPPORTED;
        }
    }
    switch (w->type) {
        case ZQ_TYPE_Q4_0: return launch_tc<ZQ_TYPE_Q4_0>(w, xt, post, y, m_rows, a, st);
        case ZQ_TYPE_Q4_1: return launch_tc<ZQ_TYPE_Q4_1>(w, xt, post, y, m_rows, a, st);
        case ZQ_TYPE_Q8_0: return launch_tc<ZQ_TYPE_Q8_0>(w, xt, post, y, m_rows, a, st);
        default: return ZQ_ERR_UNSUPPORTED;
    }
}

}  // namespace zq

extern "C" int zq_set_cluster_launch(int enabled) {
    zq::g_cluster_launch = enabled ? 1 : 0;
    return ZQ_OK;
}
