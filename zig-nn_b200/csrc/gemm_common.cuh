// Pieces shared by the mma.sync GEMMs over quantised weights (gemm.cu, gemm_trans.cu): the swizzled
// [rows][64 halves] shared-memory tile, ldmatrix / mma wrappers, and the dequantisation of one quad of
// blocks of one weight row into fp16 — value = (n - 8) * d, n * d + m or q * d, rounded once to fp16.
#pragma once
#include "zq_internal.h"

namespace zq {
namespace gemm_common {

constexpr uint32_t HALF_TILE = 128 * 128;  // bytes of a [128 rows][64 halves] tile

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

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
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

}  // namespace gemm_common
}  // namespace zq
