// The GPT-2 decode step as ONE persistent cooperative kernel (one launch per token, or per greedy run).
//
// The launch sequence of the engine (ln1 | qkv | cache write + scores | softmax.V | proj + residual | ln2 |
// fc + gelu | mproj + residual, twelve times, then ln_f, the f32 vocabulary head and the arg-max:
// src/models/gpt2.zig:423-509) costs about a hundred launches of 4 us per token. Here 148 CTAs (one per SM,
// 16 consumer warps + a producer warp) walk the same phases and hand the vectors between them through
// global memory as 64-bit words that carry their exchange number, as the Gemma-3 kernel does
// (decode_gemma.cu): no grid barrier, one L2 round trip per hand-over.
//
//   * Weights stream through a ring of shared-memory slots: a unit = a tile of up to 8 weight rows (a K-chunk of
//     it for the 3072-wide projection), or three f32 rows of the vocabulary head; the producer warp issues the
//     units as bulk copies, a lane per ring slot, and runs ahead across phase boundaries.
//   * This path's activations are f32 (gpt2.zig:632-686 -> dequant.zig:170-309) and its parity bar is a tolerance
//     (rel-L2 1e-3 on logits, identical greedy tokens), not bit equality: dots are plain f32 multiply-adds over
//     nibbles unpacked in registers, reductions are trees. Every reduction has a fixed order, so a run is
//     reproducible bit for bit.
//   * The residual stream lives in every CTA's shared memory (all CTAs add the same exchanged vectors in the same
//     order); LayerNorm is recomputed by every CTA instead of being exchanged once more.
//   * Every wait (exchange words, mbarriers) is bounded; a CTA that gives up raises an abort word that all CTAs
//     test at phase boundaries, and the kernel returns with the library's device-error word set.
#include <math.h>
#include <string.h>

#include <new>
#include <vector>

#include "decode_common.cuh"
#include "decode_gpt2.h"
#include "zq_internal.h"

namespace zq {
namespace {

using namespace dk;

struct GMat {
    const uint8_t* qs;
    const uint8_t* sc;
    const float* bias;
    uint32_t type, n_rows, nb, nbp;
    uint32_t row_q_bytes, row_s_bytes;
    uint32_t n_tiles, tiles_div, tiles_rem;  // tiles of 8 rows; CTA c owns tiles_div + (c < tiles_rem) of them
    uint32_t chunks, chunk_quads, chunk_q_pitch, chunks_magic;  // pieces of a tile along K (at most 16 quads each)
    uint32_t pad_;
};

struct alignas(16) GLayer {
    GMat qkv, proj, fc, mproj;
    const float *ln1_w, *ln1_b, *ln2_w, *ln2_b;
    float *kc, *vc;
};

// Exchange buffers, two of each (layer parity). A word is (epoch << 32) | float bits.
struct GExchange {
    unsigned long long *qkv, *scores, *att, *proj, *fc, *mproj, *best;
    uint32_t qkv_n, scores_n, att_n, proj_n, fc_n, mproj_n, best_n;  // words per parity
};

struct GParams {
    const GLayer* layers;
    const float *wte, *wpe, *ln_f_w, *ln_f_b;
    float* logits;
    uint32_t *state, *record, *abort_word;
    unsigned int* err;
    GExchange ex;
    uint32_t n_layer, E, H, D, F, ctx, vocab;
    float eps;
    uint32_t n_slots, slot_magic, slot_bytes;
    uint32_t head_rows, head_units, head_div, head_rem;  // f32 rows per unit of the vocabulary head; units; per CTA
    uint32_t magic_H, magic_D8;                          // floor(2^32 / x): heads; D / 8
    uint32_t part_rows;                                  // rows of the per-warp partial sums
    uint32_t h_floats;                                   // floats of the GEMV input vector (rows padded to whole quads)
    // shared-memory carve-up (bytes from the start of dynamic shared memory)
    uint32_t off_layers, off_xres, off_h, off_q, off_lnw, off_part, off_scratch, off_ring;
};

struct GShared {
    GParams p;
    unsigned long long full[64];
    unsigned long long empty[64];
    uint32_t released[64];  // per ring slot: uses consumed so far
    int abort;
    uint32_t launch_id;
    float red[2][kConsumerWarps];  // block reductions, two sets in turn
    float bval[kConsumerWarps];
    uint32_t bidx[kConsumerWarps];
};
constexpr uint32_t kGSharedHead = (sizeof(GShared) + 127u) & ~127u;

__device__ __forceinline__ unsigned char* gsmem() {
    extern __shared__ __align__(128) unsigned char zq_gpt2_smem[];
    return zq_gpt2_smem;
}
__device__ __forceinline__ GShared& gsh() { return *reinterpret_cast<GShared*>(gsmem()); }

struct GCta {
    unsigned char* smem;
    uint32_t smem32, full0, empty0;
    volatile int* s_abort;
    volatile uint32_t* released;
    int tid, lane, warp;
    uint32_t launch_id;
};
__device__ __forceinline__ GCta gcta() {
    GShared& S = gsh();
    GCta c;
    c.smem = gsmem();
    c.smem32 = (uint32_t)__cvta_generic_to_shared(c.smem);
    c.full0 = (uint32_t)__cvta_generic_to_shared(S.full);
    c.empty0 = (uint32_t)__cvta_generic_to_shared(S.empty);
    c.s_abort = &S.abort;
    c.released = S.released;
    c.tid = threadIdx.x;
    c.lane = threadIdx.x & 31;
    c.warp = threadIdx.x >> 5;
    c.launch_id = S.launch_id;
    return c;
}

__device__ __forceinline__ void g_raise_abort(const GCta& c, const GParams& p, unsigned int code) {
    *c.s_abort = 1;
    if (ld_relaxed_gpu_u32(p.abort_word) != c.launch_id) atomicExch(p.err, code);
    atomicExch(p.abort_word, c.launch_id);
}

// Up to N words of an exchange buffer per thread (first, first + stride, ...; valid below n), all loads in flight at
// once; words whose producer has not written yet are polled again, a bounded number of times.
template <int N>
__device__ __forceinline__ void g_xload_batch(const GCta& c, const GParams& p, const unsigned long long* buf, uint32_t first,
                                              uint32_t stride, uint32_t n, uint32_t epoch, float (&out)[N]) {
    unsigned long long w[N];
#pragma unroll
    for (int u = 0; u < N; ++u) w[u] = first + u * stride < n ? xload(buf + first + u * stride) : 0ull;
    bool missing = false;
#pragma unroll
    for (int u = 0; u < N; ++u)
        if (first + u * stride < n && (uint32_t)(w[u] >> 32) != epoch) missing = true;
    if (missing) {
        for (uint32_t spin = 0; missing && spin < kPollLimit; ++spin) {
            missing = false;
#pragma unroll
            for (int u = 0; u < N; ++u) {
                if (first + u * stride < n && (uint32_t)(w[u] >> 32) != epoch) {
                    w[u] = xload(buf + first + u * stride);
                    if ((uint32_t)(w[u] >> 32) != epoch) missing = true;
                }
            }
            if (missing && (spin & 63u) == 63u && (*c.s_abort || ld_relaxed_gpu_u32(p.abort_word) == c.launch_id)) break;
        }
        if (missing) g_raise_abort(c, p, kErrExchange);
    }
#pragma unroll
    for (int u = 0; u < N; ++u) out[u] = __uint_as_float((uint32_t)w[u]);
}

// An exchanged vector of n floats into shared memory; `add` adds it onto what is there (the residual stream).
__device__ __forceinline__ void load_vector(const GCta& c, const GParams& p, const unsigned long long* buf, uint32_t n,
                                            uint32_t epoch, float* dst, bool add) {
#pragma unroll 1
    for (uint32_t base = 0; base < n; base += kConsumers * 8) {
        float v[8];
        g_xload_batch<8>(c, p, buf, base + c.tid, kConsumers, n, epoch, v);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t i = base + u * kConsumers + c.tid;
            if (i < n) dst[i] = add ? __fadd_rn(dst[i], v[u]) : v[u];
        }
    }
}

__device__ __forceinline__ bool g_slot_wait(const GCta& c, const GParams& p, uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < (1u << 19); ++i) {
        if (mbar_try_wait_hint(bar, parity, 2000u)) return true;
        if ((i & 15u) == 15u && *c.s_abort) return false;
    }
    g_raise_abort(c, p, kErrUnitWait);
    return false;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}
// Sum over the 512 consumer threads, the same value (and the same bits) in every thread. `set` alternates between
// consecutive calls so that one barrier per sum is enough.
__device__ __forceinline__ float block_sum(const GCta& c, float v, int set) {
    GShared& S = gsh();
    v = warp_sum(v);
    if (c.lane == 0) S.red[set][c.warp] = v;
    cbar();
    float s = S.red[set][0];
#pragma unroll
    for (int w = 1; w < kConsumerWarps; ++w) s += S.red[set][w];
    return s;
}
__device__ __forceinline__ float block_max(const GCta& c, float v, int set) {
    GShared& S = gsh();
    v = warp_max(v);
    if (c.lane == 0) S.red[set][c.warp] = v;
    cbar();
    float s = S.red[set][0];
#pragma unroll
    for (int w = 1; w < kConsumerWarps; ++w) s = fmaxf(s, S.red[set][w]);
    return s;
}

// Two-pass layer norm of xres into h (gpt2.zig:541-596): mean, then sum (x - mean)^2. The weights were requested
// into `lnw` (gamma, then beta) by stage_ln.
__device__ __noinline__ void layer_norm_to(const float* xres, float* h, const float* lnw, uint32_t E, float eps) {
    const GCta c = gcta();
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    float s = 0.0f;
    for (uint32_t i = c.tid; i < E; i += kConsumers) s += xres[i];
    const float mean = block_sum(c, s, 0) / (float)E;  // (the barrier inside also completes xres and lnw for every thread)
    float v = 0.0f;
    for (uint32_t i = c.tid; i < E; i += kConsumers) {
        const float d = xres[i] - mean;
        v = fmaf(d, d, v);
    }
    const float var = block_sum(c, v, 1) / (float)E;
    const float inv = 1.0f / sqrtf(var + eps);
    for (uint32_t i = c.tid; i < E; i += kConsumers)
        h[i] = __fadd_rn(__fmul_rn(__fmul_rn(xres[i] - mean, inv), lnw[i]), lnw[E + i]);
    cbar();
}
// gamma and beta on their way into shared memory (asynchronous copies, waited for in layer_norm_to)
__device__ __forceinline__ void stage_ln(const GCta& c, const float* g, const float* b, float* lnw, uint32_t E) {
    const uint32_t dst = c.smem32 + (uint32_t)(reinterpret_cast<unsigned char*>(lnw) - c.smem);
    for (uint32_t i = c.tid * 4; i < E; i += kConsumers * 4) {
        cp_async16(dst + i * 4, g + i);
        cp_async16(dst + (E + i) * 4, b + i);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// Geometry of one unit (piece `ch` of tile `tile`) as both sides of the ring compute it.
struct GUnit {
    uint32_t rows, row0, q_first, nqc, q_pitch, s_pitch, s_off, s_delta;
};
__device__ __forceinline__ GUnit g_unit(const GMat& m, uint32_t tile, uint32_t ch) {
    GUnit u;
    const uint32_t nq = m.nbp >> 2;
    const uint32_t SB = m.type == ZQ_TYPE_Q4_1 ? 4u : 2u;
    u.row0 = tile * 8;
    u.rows = min(8u, m.n_rows - u.row0);
    u.q_first = ch * m.chunk_quads;
    u.nqc = min(m.chunk_quads, nq - u.q_first);
    if (m.chunks == 1) {
        u.q_pitch = m.row_q_bytes;
        u.s_pitch = m.row_s_bytes;
        u.s_off = u.rows * m.row_q_bytes;
        u.s_delta = 0;
    } else {
        u.q_pitch = m.chunk_q_pitch;
        const uint32_t so = u.q_first * 4 * SB;
        u.s_delta = so & 15u;
        u.s_pitch = ((m.chunk_quads * 4 * SB + 15u) & ~15u) + 16u;
        u.s_off = 8 * u.q_pitch;
    }
    return u;
}

// Partial dot products of one unit against the f32 activation vector x (whole K in shared memory), quads [q_lo, q_hi)
// of the piece. Lane (g, t) holds word t (and 4 + t for q8_0) of the four blocks of a quad of row g: elements 4t..4t+3
// and 16+4t..16+4t+3 of each block. Returns the lane's share of row g's dot (to be added over the four t lanes).
template <int TYPE>
__device__ __forceinline__ float unit_dot(const unsigned char* slab_q, uint32_t q_pitch, const unsigned char* slab_s,
                                          uint32_t s_pitch, uint32_t rows, uint32_t q_lo, uint32_t q_hi, uint32_t q_first,
                                          const float* x, int lane) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QUAD = Q8 ? 128 : 64;
    const int t = lane & 3;
    const uint32_t g = (uint32_t)lane >> 2;
    const uint32_t gr = g < rows ? g : 0u;
    const unsigned char* wrow = slab_q + (size_t)gr * q_pitch + 16 * t;
    const unsigned char* srow = slab_s + (size_t)gr * s_pitch;
    float acc = 0.0f;
#pragma unroll 1
    for (uint32_t q = q_lo; q < q_hi; ++q) {
        const uint4 wa = *reinterpret_cast<const uint4*>(wrow + q * QUAD);
        uint4 wb = wa;
        if (Q8) wb = *reinterpret_cast<const uint4*>(wrow + q * QUAD + 64);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t blk = (q_first + q) * 4 + j, bl = q * 4 + j;
            const float4 xa = *reinterpret_cast<const float4*>(x + blk * 32 + 4 * t);
            const float4 xb = *reinterpret_cast<const float4*>(x + blk * 32 + 16 + 4 * t);
            const uint32_t ua = pick(wa, j), ub = pick(wb, j);
            float part;
            if (Q8) {
                part = (float)(int8_t)(ua & 0xFF) * xa.x;
                part = fmaf((float)(int8_t)((ua >> 8) & 0xFF), xa.y, part);
                part = fmaf((float)(int8_t)((ua >> 16) & 0xFF), xa.z, part);
                part = fmaf((float)(int8_t)(ua >> 24), xa.w, part);
                part = fmaf((float)(int8_t)(ub & 0xFF), xb.x, part);
                part = fmaf((float)(int8_t)((ub >> 8) & 0xFF), xb.y, part);
                part = fmaf((float)(int8_t)((ub >> 16) & 0xFF), xb.z, part);
                part = fmaf((float)(int8_t)(ub >> 24), xb.w, part);
            } else {
                const int off = TYPE == ZQ_TYPE_Q4_0 ? 8 : 0;
                part = (float)((int)(ua & 15u) - off) * xa.x;
                part = fmaf((float)((int)((ua >> 8) & 15u) - off), xa.y, part);
                part = fmaf((float)((int)((ua >> 16) & 15u) - off), xa.z, part);
                part = fmaf((float)((int)((ua >> 24) & 15u) - off), xa.w, part);
                part = fmaf((float)((int)((ua >> 4) & 15u) - off), xb.x, part);
                part = fmaf((float)((int)((ua >> 12) & 15u) - off), xb.y, part);
                part = fmaf((float)((int)((ua >> 20) & 15u) - off), xb.z, part);
                part = fmaf((float)((int)((ua >> 28) & 15u) - off), xb.w, part);
            }
            if (Q41) {
                const __half2 dm = *reinterpret_cast<const __half2*>(srow + bl * 4);
                const float sx = ((xa.x + xa.y) + (xa.z + xa.w)) + ((xb.x + xb.y) + (xb.z + xb.w));
                acc = fmaf(__low2float(dm), part, acc);
                acc = fmaf(__high2float(dm), sx, acc);
            } else {
                acc = fmaf(__half2float(*reinterpret_cast<const __half*>(srow + bl * 2)), part, acc);
            }
        }
    }
    return acc;
}
template <typename... A>
__device__ __forceinline__ float unit_dot_any(uint32_t type, A... a) {
    if (type == ZQ_TYPE_Q8_0) return unit_dot<ZQ_TYPE_Q8_0>(a...);
    if (type == ZQ_TYPE_Q4_0) return unit_dot<ZQ_TYPE_Q4_0>(a...);
    return unit_dot<ZQ_TYPE_Q4_1>(a...);
}

__device__ __forceinline__ bool g_unit_acquire(const GCta& c, const GParams& p, uint32_t slot, uint32_t use) {
    // The slot's previous use must have been consumed before its barrier is read: a parity wait alone cannot tell
    // fill `use` from fill `use - 2`.
    bool ready = true;
    if (use > 0) {
        uint32_t spins = 0;
        while (c.released[slot] < use && ++spins < kSlotSpinLimit) __nanosleep(64);
        ready = c.released[slot] >= use;
        if (!ready) g_raise_abort(c, p, kErrUnitWait);
    }
    ready = ready && g_slot_wait(c, p, c.full0 + slot * 8, use & 1u);
    return __all_sync(0xFFFFFFFFu, ready);
}
__device__ __forceinline__ void g_unit_release(const GCta& c, uint32_t slot, uint32_t use, uint32_t count) {
    __syncwarp();
    if (c.lane == 0) {
        c.released[slot] = use + 1;
        __threadfence_block();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(c.empty0 + slot * 8), "r"(count) : "memory");
    }
}

__device__ __noinline__ float g_gelu(float v) {
    const float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v);
    const float inner = __fmul_rn(0.7978845608f, __fadd_rn(v, cube));
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, (float)tanh((double)inner)));
}

// One matrix-vector phase over a quantised matrix: y = W x + bias [gelu], this CTA's tiles (tile = cta, cta + grid,
// ...). x (whole K, f32) is complete in shared memory before the call. The quads of all the CTA's units, as one
// sequence, are cut into 16 equal runs, one per warp; a warp adds what it finds of a row into its own line of the
// partial sums, and after a barrier one thread per row adds the 16 lines in order, applies the epilogue and writes the
// exchange word. A unit's 16 slot-release arrivals are shared out over the warps that read it as in the Gemma kernel.
// Returns the advanced unit counter.
__device__ __noinline__ uint32_t g_gemv_phase(const GMat& m, uint32_t unit_base, const float* x, int gelu,
                                              unsigned long long* xout, uint32_t epoch) {
    const GCta c = gcta();
    const GParams& p = gsh().p;
    float* part = reinterpret_cast<float*>(c.smem + p.off_part);
    const uint32_t G = gridDim.x, cta = blockIdx.x;
    const uint32_t C = m.chunks;
    const uint32_t mine = m.tiles_div + (cta < m.tiles_rem ? 1u : 0u);
    const uint32_t base = unit_base;
    const uint32_t nq = m.nbp >> 2, cq = m.chunk_quads;
    const uint32_t rows_all = min(mine * 8, p.part_rows);
    float* my = part + (size_t)c.warp * p.part_rows;
    for (uint32_t r = c.lane; r < rows_all; r += 32) my[r] = 0.0f;
    __syncwarp();
    // the bias of the row this thread finishes below: requested now, it arrives under the dots
    const uint32_t r_mine = (uint32_t)(c.tid >= kChainTid ? c.tid - kChainTid : c.tid + kConsumers - kChainTid);
    const uint32_t row_mine = (cta + (r_mine >> 3) * G) * 8 + (r_mine & 7u);
    const float bias_mine = (r_mine < rows_all && row_mine < m.n_rows) ? __ldg(m.bias + row_mine) : 0.0f;
    const uint32_t total = mine * nq;
    const uint32_t run_lo = ((uint32_t)c.warp * total) >> 4, run_hi = (((uint32_t)c.warp + 1u) * total) >> 4;
    uint32_t i = 0, ch = 0, us = 0;
#pragma unroll 1
    for (uint32_t n = 0; n < mine * C; ++n) {
        const uint32_t q_first = ch * cq;
        const uint32_t nqc = min(cq, nq - q_first);
        const uint32_t ue = us + nqc;
        if (run_lo < ue && run_hi > us) {
            const uint32_t lo = max(run_lo, us) - us, hi = min(run_hi, ue) - us;
            uint32_t slot, use;
            fast_divmod(base + n, p.n_slots, p.slot_magic, use, slot);
            const GUnit u = g_unit(m, cta + i * G, ch);
            if (!g_unit_acquire(c, p, slot, use)) break;
            const unsigned char* slab_q = c.smem + p.off_ring + (size_t)slot * p.slot_bytes;
            float v = unit_dot_any(m.type, slab_q, u.q_pitch, slab_q + u.s_off + u.s_delta, u.s_pitch, u.rows, lo, hi, q_first,
                                   x, c.lane);
            g_unit_release(c, slot, use, (hi == nqc ? (uint32_t)kConsumerWarps : hi) - lo);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
            const uint32_t r = i * 8 + ((uint32_t)c.lane >> 2);
            if ((c.lane & 3) == 0 && r < rows_all) my[r] += v;
            __syncwarp();
        }
        us = ue;
        if (++ch == C) {
            ch = 0;
            ++i;
        }
    }
    cbar();  // every warp's line of partial sums is complete
#pragma unroll 1
    for (uint32_t r = r_mine; r < rows_all; r += kConsumers) {
        const uint32_t row = (cta + (r >> 3) * G) * 8 + (r & 7u);
        if (row < m.n_rows) {
            const size_t pr = p.part_rows;
            float a0 = part[r], a1 = part[pr + r], a2 = part[2 * pr + r], a3 = part[3 * pr + r];
#pragma unroll
            for (int w = 4; w < kConsumerWarps; w += 4) {  // four running sums: the order is fixed, the adds overlap
                a0 += part[(size_t)w * pr + r];
                a1 += part[(size_t)(w + 1) * pr + r];
                a2 += part[(size_t)(w + 2) * pr + r];
                a3 += part[(size_t)(w + 3) * pr + r];
            }
            float v = (a0 + a1) + (a2 + a3);
            v += r == r_mine ? bias_mine : __ldg(m.bias + row);
            if (gelu) v = g_gelu(v);
            xstore(xout + row, v, epoch);
        }
    }
    return base + mine * C;
}

// The vocabulary head: logits[v] = wte[v] . h (f32 rows, gpt2.zig:652-671), units of head_rows rows, one warp per
// unit. Returns the advanced unit counter; `best` follows the arg-max (first maximum wins) when given.
struct GBest {
    float v;
    uint32_t i;
};
__device__ __forceinline__ void g_best_update(GBest& b, float v, uint32_t i) {
    if (v > b.v || (v == b.v && i < b.i)) {
        b.v = v;
        b.i = i;
    }
}
__device__ __noinline__ uint32_t g_head_phase(uint32_t unit_base, const float* h, GBest* best) {
    const GCta c = gcta();
    const GParams& p = gsh().p;
    const uint32_t G = gridDim.x, cta = blockIdx.x, E = p.E, R = p.head_rows;
    const uint32_t mine = p.head_div + (cta < p.head_rem ? 1u : 0u);
#pragma unroll 1
    for (uint32_t i = c.warp; i < mine; i += kConsumerWarps) {
        uint32_t slot, use;
        fast_divmod(unit_base + i, p.n_slots, p.slot_magic, use, slot);
        if (!g_unit_acquire(c, p, slot, use)) break;
        const float* rows = reinterpret_cast<const float*>(c.smem + p.off_ring + (size_t)slot * p.slot_bytes);
        const uint32_t row0 = (cta + i * G) * R, nr = min(R, p.vocab - row0);
        float acc[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) acc[r] = 0.0f;
#pragma unroll 1
        for (uint32_t k = (uint32_t)c.lane * 4; k < E; k += 128) {
            const float4 hv = *reinterpret_cast<const float4*>(h + k);
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if ((uint32_t)r < nr) {
                    const float4 wv = *reinterpret_cast<const float4*>(rows + (size_t)r * E + k);
                    acc[r] = fmaf(hv.x, wv.x, acc[r]);
                    acc[r] = fmaf(hv.y, wv.y, acc[r]);
                    acc[r] = fmaf(hv.z, wv.z, acc[r]);
                    acc[r] = fmaf(hv.w, wv.w, acc[r]);
                }
            }
        }
        g_unit_release(c, slot, use, (uint32_t)kConsumerWarps);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if ((uint32_t)r < nr) {
                const float v = warp_sum(acc[r]);
                if (c.lane == 0) {
                    p.logits[row0 + r] = v;
                    if (best) g_best_update(*best, v, row0 + r);
                }
            }
        }
    }
    return unit_base + mine;
}

// The producer's side: issue this CTA's units of `m` (or of the head when m == nullptr) into the ring, a lane per ring
// slot. The warp meets again at the end of a phase (see decode_gemma.cu for why). Returns false on a timeout.
__device__ __noinline__ bool g_produce_phase(const GMat* mp, uint32_t* unit_base) {
    const GCta c = gcta();
    const GParams& p = gsh().p;
    const uint32_t G = gridDim.x, cta = blockIdx.x;
    const uint32_t lanes = p.n_slots < 32u ? p.n_slots : 32u;
    const uint32_t base = *unit_base;
    bool ok = true;
    if (!mp) {
        const uint32_t mine = p.head_div + (cta < p.head_rem ? 1u : 0u);
        *unit_base = base + mine;
        const uint32_t row_bytes = p.E * 4u;
#pragma unroll 1
        for (uint32_t n = (uint32_t)c.lane; ok && (uint32_t)c.lane < lanes && n < mine; n += lanes) {
            uint32_t slot, use;
            fast_divmod(base + n, p.n_slots, p.slot_magic, use, slot);
            if (use > 0 && !g_slot_wait(c, p, c.empty0 + slot * 8, (use - 1) & 1u)) {
                ok = false;
                break;
            }
            const uint32_t row0 = (cta + n * G) * p.head_rows, nr = min(p.head_rows, p.vocab - row0);
            const uint32_t bar = c.full0 + slot * 8;
            mbar_arrive_expect_tx(bar, nr * row_bytes);
            bulk_copy_g2s(c.smem32 + p.off_ring + slot * p.slot_bytes, p.wte + (size_t)row0 * p.E, nr * row_bytes, bar);
        }
        return __all_sync(0xFFFFFFFFu, ok);
    }
    const GMat& m = *mp;
    const uint32_t C = m.chunks;
    const uint32_t mine = m.tiles_div + (cta < m.tiles_rem ? 1u : 0u);
    *unit_base = base + mine * C;
    const uint32_t rqb = m.row_q_bytes, rsb = m.row_s_bytes;
    const uint32_t QUAD = m.type == ZQ_TYPE_Q8_0 ? 128u : 64u, SB = m.type == ZQ_TYPE_Q4_1 ? 4u : 2u;
#pragma unroll 1
    for (uint32_t n = (uint32_t)c.lane; ok && (uint32_t)c.lane < lanes && n < mine * C; n += lanes) {
        uint32_t i, ch;
        fast_divmod(n, C, m.chunks_magic, i, ch);
        uint32_t slot, use;
        fast_divmod(base + n, p.n_slots, p.slot_magic, use, slot);
        if (use > 0 && !g_slot_wait(c, p, c.empty0 + slot * 8, (use - 1) & 1u)) {
            ok = false;
            break;
        }
        const uint32_t dst = c.smem32 + p.off_ring + slot * p.slot_bytes;
        const uint32_t bar = c.full0 + slot * 8;
        const GUnit u = g_unit(m, cta + i * G, ch);
        if (C == 1) {
            const uint32_t qb = u.rows * rqb, sb = u.rows * rsb;
            mbar_arrive_expect_tx(bar, qb + sb);
            bulk_copy_g2s(dst, m.qs + (size_t)u.row0 * rqb, qb, bar);
            bulk_copy_g2s(dst + qb, m.sc + (size_t)u.row0 * rsb, sb, bar);
        } else {
            const uint32_t qbytes = u.nqc * QUAD;
            const uint32_t so = u.q_first * 4 * SB, sa = so & ~15u;
            const uint32_t sbytes = ((u.s_delta + u.nqc * 4 * SB + 15u) & ~15u);
            mbar_arrive_expect_tx(bar, u.rows * (qbytes + sbytes));
#pragma unroll 1
            for (uint32_t r = 0; r < u.rows; ++r) {
                const size_t row = u.row0 + r;
                bulk_copy_g2s(dst + r * u.q_pitch, m.qs + row * rqb + (size_t)u.q_first * QUAD, qbytes, bar);
                bulk_copy_g2s(dst + u.s_off + r * u.s_pitch, m.sc + row * rsb + sa, sbytes, bar);
            }
        }
    }
    return __all_sync(0xFFFFFFFFu, ok);
}

// Attention, first half (gpt2.zig:796-849): every CTA takes the exchanged q|k|v row; the last CTA stores the key /
// value rows of position `pos`; the scores of positions 0..pos are spread over the CTAs in tiles of 32 (position,
// head) pairs: 16 lanes per dot (lane l takes elements l, l + 16, ...; lanes added in order), times 1/sqrt(D).
__device__ __noinline__ bool g_scores_phase(const GLayer& L, uint32_t pos, float* q, const unsigned long long* qkv_in,
                                            uint32_t ep_in, unsigned long long* scores_out, uint32_t ep_out) {
    const GCta c = gcta();
    const GParams& p = gsh().p;
    const uint32_t E = p.E, H = p.H, D = p.D;
    load_vector(c, p, qkv_in, 3 * E, ep_in, q, false);  // q | k | v of this position
    if (cbar_or(*c.s_abort != 0)) return false;
    const float* knew = q + E;
    const float* vnew = q + 2 * E;
    if (blockIdx.x == gridDim.x - 1) {
        for (uint32_t i = c.tid; i < E; i += kConsumers) {
            L.kc[(size_t)pos * E + i] = knew[i];
            L.vc[(size_t)pos * E + i] = vnew[i];
        }
    }
    const uint32_t jobs = (pos + 1) * H, tiles = (jobs + 31) >> 5;
    const uint32_t l = c.tid & 15u, js = c.tid >> 4;
    const float scale = 1.0f / sqrtf((float)D);
#pragma unroll 1
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const uint32_t job = tile * 32 + js;
        const bool live = job < jobs;
        const uint32_t jc = live ? job : jobs - 1;
        uint32_t pi, h;
        fast_divmod(jc, H, p.magic_H, pi, h);
        const float* qh = q + h * D;
        const bool cur = pi == pos;
        const float* kr = cur ? knew + h * D : L.kc + (size_t)pi * E + h * D;
        float acc = 0.0f;
        if (D <= 128u) {  // the lane's key elements all requested before the first is used
            float kv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t d = l + 16u * u;
                kv[u] = d < D ? (cur ? kr[d] : __ldcg(kr + d)) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t d = l + 16u * u;
                if (d < D) acc = __fadd_rn(acc, __fmul_rn(qh[d], kv[u]));
            }
        } else {
#pragma unroll 1
            for (uint32_t d = l; d < D; d += 16) acc = __fadd_rn(acc, __fmul_rn(qh[d], cur ? kr[d] : __ldcg(kr + d)));
        }
        float s = __shfl_sync(0xFFFFFFFFu, acc, 0, 16);
#pragma unroll
        for (int j = 1; j < 16; ++j) s = __fadd_rn(s, __shfl_sync(0xFFFFFFFFu, acc, j, 16));
        if (l == 0 && live) xstore(scores_out + (size_t)h * p.ctx + pi, __fmul_rn(s, scale), ep_out);
    }
    return true;
}

// Attention, second half: a job owns 8 output dimensions of one head. Softmax of the head's scores, then
// out[d] = sum_p w[p] v[p][d]: thread (group, d) adds the positions of its group (64 groups), one thread per d adds the
// 64 group sums in order.
__device__ __noinline__ bool g_softmax_v_phase(const GLayer& L, uint32_t pos, const float* q, float* scratch,
                                               const unsigned long long* scores_in, uint32_t ep_in,
                                               unsigned long long* att_out, uint32_t ep_out) {
    const GCta c = gcta();
    const GParams& p = gsh().p;
    const uint32_t E = p.E, D = p.D, n = pos + 1;
    const uint32_t chunks = D / 8, jobs = p.H * chunks;
    const float* vnew = q + 2 * E;
    float* w = scratch;                                   // [ctx]
    float* gsum = w + ((p.ctx + 3u) & ~3u);               // [64][8]
    bool ok = true;
#pragma unroll 1
    for (uint32_t job = blockIdx.x; ok && job < jobs; job += gridDim.x) {
        uint32_t h, dc;
        fast_divmod(job, chunks, p.magic_D8, h, dc);
        const unsigned long long* sh_ = scores_in + (size_t)h * p.ctx;
        // the first eight value rows of this thread do not depend on the scores: requested now
        const uint32_t grp = (uint32_t)c.tid >> 3, d = (uint32_t)c.tid & 7u;
        const uint32_t col = h * D + dc * 8 + d;
        float vfirst[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const uint32_t pp = grp + 64u * u;
            vfirst[u] = pp < n ? (pp == pos ? vnew[col] : __ldcg(L.vc + (size_t)pp * E + col)) : 0.0f;
        }
        float mx = -INFINITY;
#pragma unroll 1
        for (uint32_t base = 0; base < n; base += kConsumers * 4) {
            float v[4];
            g_xload_batch<4>(c, p, sh_, base + c.tid, kConsumers, n, ep_in, v);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = base + u * kConsumers + c.tid;
                if (i < n) {
                    w[i] = v[u];
                    mx = fmaxf(mx, v[u]);
                }
            }
        }
        mx = block_max(c, mx, 0);
        if (*c.s_abort) ok = false;  // (read after a barrier every thread passed; re-checked uniformly below)
        float s = 0.0f;
#pragma unroll 1
        for (uint32_t i = c.tid; i < n; i += kConsumers) {
            const float e = (float)exp((double)(w[i] - mx));
            w[i] = e;
            s += e;
        }
        const float inv = 1.0f / block_sum(c, s, 1);
        // (the barrier inside block_sum also completes w for every thread)
        float acc = 0.0f;
#pragma unroll 1
        for (uint32_t p0 = grp; p0 < n; p0 += 64 * 8) {  // eight value rows in flight per thread
            float vv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t pp = p0 + 64u * u;
                if (p0 == grp) vv[u] = vfirst[u];
                else vv[u] = pp < n ? (pp == pos ? vnew[col] : __ldcg(L.vc + (size_t)pp * E + col)) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t pp = p0 + 64u * u;
                if (pp < n) acc = fmaf(w[pp] * inv, vv[u], acc);
            }
        }
        // the 64 group sums of a dimension: four groups meet inside a warp (lanes d, d + 8, d + 16, d + 24), the 16
        // warps' sums through shared memory
        acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 8);
        acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 16);
        if (c.lane < 8) gsum[c.lane * kConsumerWarps + c.warp] = acc;
        ok = !cbar_or(!ok);
        if (c.tid < 8 && ok) {
            const float4* g4 = reinterpret_cast<const float4*>(gsum + c.tid * kConsumerWarps);
            const float4 a = g4[0], b = g4[1], cc = g4[2], dd = g4[3];
            const float o = (((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w))) +
                            (((cc.x + cc.y) + (cc.z + cc.w)) + ((dd.x + dd.y) + (dd.z + dd.w)));
            xstore(att_out + h * D + dc * 8 + c.tid, o, ep_out);
        }
        cbar();  // w and gsum are rewritten by the next job
    }
    return ok;
}

__global__ void __launch_bounds__(kThreads, 1)
gpt2_decode_kernel(const __grid_constant__ GParams p_in, uint32_t n_steps, int variant, uint32_t launch_id,
                   uint32_t epoch_base) {
    unsigned char* smem = gsmem();
    GShared& S = gsh();
    {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(&p_in);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&S.p);
        for (uint32_t i = threadIdx.x; i < sizeof(GParams) / 4; i += kThreads) dst[i] = src[i];
    }
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p_in.n_slots; ++s) {
            mbar_init((uint32_t)__cvta_generic_to_shared(&S.full[s]), 1);
            mbar_init((uint32_t)__cvta_generic_to_shared(&S.empty[s]), kConsumerWarps);
            S.released[s] = 0;
        }
        S.abort = 0;
        S.launch_id = launch_id;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const GParams& p = S.p;
    GLayer* layers = reinterpret_cast<GLayer*>(smem + p_in.off_layers);
    {
        const uint4* src = reinterpret_cast<const uint4*>(p_in.layers);
        uint4* dst = reinterpret_cast<uint4*>(layers);
        for (uint32_t i = threadIdx.x; i < p_in.n_layer * (uint32_t)(sizeof(GLayer) / 16); i += kThreads) dst[i] = __ldg(src + i);
    }
    __syncthreads();
    const GCta c = gcta();
    const bool want_logits = variant != DECODE_CACHE_ONLY;
    uint32_t unit_base = 0;

    if (c.warp == kConsumerWarps) {
        // ---------------------------------------------------------------- producer warp
        bool ok = true;
        for (uint32_t step = 0; ok && step < n_steps; ++step) {
            for (uint32_t l = 0; ok && l < p.n_layer; ++l) {
                const GLayer& L = layers[l];
                ok = g_produce_phase(&L.qkv, &unit_base) && g_produce_phase(&L.proj, &unit_base) &&
                     g_produce_phase(&L.fc, &unit_base) && g_produce_phase(&L.mproj, &unit_base);
            }
            if (ok && want_logits) ok = g_produce_phase(nullptr, &unit_base);
        }
        if (!ok && c.lane == 0) {
            // Stopped early: copies already issued still land in this CTA's shared memory; give every slot's barrier
            // a bounded chance to complete before the CTA retires.
            for (uint32_t s = 0; s < p.n_slots; ++s)
                for (uint32_t i = 0; i < (1u << 16); ++i)
                    if (mbar_try_wait(c.full0 + s * 8, 0) || mbar_try_wait(c.full0 + s * 8, 1)) break;
        }
        __syncwarp();
        return;
    }

    // -------------------------------------------------------------------- consumer warps
    float* xres = reinterpret_cast<float*>(smem + p.off_xres);
    float* h = reinterpret_cast<float*>(smem + p.off_h);       // the GEMV input vector: E or F floats
    float* q = reinterpret_cast<float*>(smem + p.off_q);       // q | k | v of the current position
    float* lnw = reinterpret_cast<float*>(smem + p.off_lnw);   // gamma | beta of the coming layer norm
    float* scratch = reinterpret_cast<float*>(smem + p.off_scratch);
    const uint32_t E = p.E;
    const GExchange& ex = p.ex;
    // blocks that only pad a row to whole quads have zero weights; what they are multiplied by must be finite
    for (uint32_t i = c.tid; i < p.h_floats; i += kConsumers) h[i] = 0.0f;
    cbar();
    uint32_t tok = __ldcg(p.state + 0), pos = __ldcg(p.state + 1), rec = __ldcg(p.state + 2);
    uint32_t epoch = epoch_base;  // the next exchange's number; every CTA counts alike
    uint32_t lc = 0;              // layers run so far in this launch: picks the buffer parity
#define ZQ_CHECK_ABORT()                      \
    do {                                      \
        if (cbar_or(S.abort != 0)) return;    \
    } while (0)

    for (uint32_t step = 0; step < n_steps; ++step) {
        __threadfence();  // cache rows that the last CTA stored during earlier steps are read below
        for (uint32_t i = c.tid; i < E; i += kConsumers)  // token + position embedding (gpt2.zig:423-440)
            xres[i] = __fadd_rn(__ldg(p.wte + (size_t)tok * E + i), __ldg(p.wpe + (size_t)pos * E + i));
        for (uint32_t l = 0; l < p.n_layer; ++l, ++lc) {
            const GLayer& L = layers[l];
            const uint32_t par = lc & 1u, prev = par ^ 1u;
            const uint32_t e_prev = epoch - 1;  // the previous layer's last exchange (unused for l == 0)
            const uint32_t e_qkv = epoch, e_scores = epoch + 1, e_att = epoch + 2, e_proj = epoch + 3, e_fc = epoch + 4,
                           e_mproj = epoch + 5;
            epoch += 6;
            // --- attention block
            stage_ln(c, L.ln1_w, L.ln1_b, lnw, E);
            if (l) {
                load_vector(c, p, ex.mproj + (size_t)prev * ex.mproj_n, E, e_prev, xres, true);
                // every CTA has finished the previous layer: its buffers of this parity may be rewritten
                for (uint32_t base = 0; base < gridDim.x; base += kConsumers) {
                    float v[1];
                    g_xload_batch<1>(c, p, ex.mproj + (size_t)prev * ex.mproj_n, E + base + (uint32_t)c.tid, 1u, E + gridDim.x,
                                     e_prev, v);
                }
            }
            layer_norm_to(xres, h, lnw, E, p.eps);
            ZQ_CHECK_ABORT();
            unit_base = g_gemv_phase(L.qkv, unit_base, h, 0, ex.qkv + (size_t)par * ex.qkv_n, e_qkv);
            if (!g_scores_phase(L, pos, q, ex.qkv + (size_t)par * ex.qkv_n, e_qkv, ex.scores + (size_t)par * ex.scores_n, e_scores))
                return;
            if (!g_softmax_v_phase(L, pos, q, scratch, ex.scores + (size_t)par * ex.scores_n, e_scores,
                                   ex.att + (size_t)par * ex.att_n, e_att))
                return;
            load_vector(c, p, ex.att + (size_t)par * ex.att_n, E, e_att, h, false);
            ZQ_CHECK_ABORT();
            unit_base = g_gemv_phase(L.proj, unit_base, h, 0, ex.proj + (size_t)par * ex.proj_n, e_proj);
            // --- MLP block
            stage_ln(c, L.ln2_w, L.ln2_b, lnw, E);
            load_vector(c, p, ex.proj + (size_t)par * ex.proj_n, E, e_proj, xres, true);
            layer_norm_to(xres, h, lnw, E, p.eps);
            ZQ_CHECK_ABORT();
            unit_base = g_gemv_phase(L.fc, unit_base, h, 1, ex.fc + (size_t)par * ex.fc_n, e_fc);
            load_vector(c, p, ex.fc + (size_t)par * ex.fc_n, p.F, e_fc, h, false);
            ZQ_CHECK_ABORT();
            unit_base = g_gemv_phase(L.mproj, unit_base, h, 0, ex.mproj + (size_t)par * ex.mproj_n, e_mproj);
            cbar();  // every warp of this CTA is through the layer: sign the presence word
            if (c.tid == 0) xstore(ex.mproj + (size_t)par * ex.mproj_n + E + blockIdx.x, 0.0f, e_mproj);
        }
        if (want_logits) {
            const uint32_t last = (lc - 1) & 1u;
            stage_ln(c, p.ln_f_w, p.ln_f_b, lnw, E);
            load_vector(c, p, ex.mproj + (size_t)last * ex.mproj_n, E, epoch - 1, xres, true);
            layer_norm_to(xres, h, lnw, E, p.eps);
            ZQ_CHECK_ABORT();
            GBest best{-INFINITY, 0xFFFFFFFFu};
            unit_base = g_head_phase(unit_base, h, variant == DECODE_GREEDY ? &best : nullptr);
            if (variant == DECODE_GREEDY) {
                // first maximum wins (gpt2.zig:980-990): lanes, warps, CTAs, always preferring the lower index
                const uint32_t e_best = epoch++;
                unsigned long long* bx = ex.best + (size_t)(step & 1u) * ex.best_n;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    GBest o;
                    o.v = __shfl_xor_sync(0xFFFFFFFFu, best.v, off);
                    o.i = __shfl_xor_sync(0xFFFFFFFFu, best.i, off);
                    g_best_update(best, o.v, o.i);
                }
                if (c.lane == 0) {
                    S.bval[c.warp] = best.v;
                    S.bidx[c.warp] = best.i;
                }
                cbar();
                if (c.tid == 0) {
                    GBest b{S.bval[0], S.bidx[0]};
                    for (int wv = 1; wv < kConsumerWarps; ++wv) g_best_update(b, S.bval[wv], S.bidx[wv]);
                    xstore(bx + 2 * blockIdx.x, b.v, e_best);
                    xstore_u32(bx + 2 * blockIdx.x + 1, b.i, e_best);
                }
                GBest b{-INFINITY, 0xFFFFFFFFu};
                for (uint32_t base = 0; base < gridDim.x; base += 32) {
                    const uint32_t k = base + c.lane;
                    float v[2];
                    g_xload_batch<2>(c, p, bx, 2 * k, 1u, 2 * gridDim.x, e_best, v);
                    if (k < gridDim.x) g_best_update(b, v[0], __float_as_uint(v[1]));
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    GBest o;
                    o.v = __shfl_xor_sync(0xFFFFFFFFu, b.v, off);
                    o.i = __shfl_xor_sync(0xFFFFFFFFu, b.i, off);
                    g_best_update(b, o.v, o.i);
                }
                ZQ_CHECK_ABORT();
                tok = b.i;
                if (blockIdx.x == 0 && c.tid == 0) p.record[rec] = tok;
                rec += 1;
            }
        } else {
            // cache-only step: the last layer's output is not read; the next step's layer 0 checks nothing of it
            cbar();
        }
        pos += 1;
    }
#undef ZQ_CHECK_ABORT
    if (blockIdx.x == 0 && c.tid == 0) {
        p.state[0] = tok;
        p.state[1] = pos;
        p.state[2] = rec;
    }
}

// ---- host side --------------------------------------------------------------------------------

bool g_describe(GMat* d, const zq_weight* w, const float* bias, uint32_t slot_bytes, uint32_t grid) {
    if (!w || !bias) return false;
    d->qs = w->qs;
    d->sc = static_cast<const uint8_t*>(w->sc);
    d->bias = bias;
    d->type = (uint32_t)w->type;
    d->n_rows = w->out_dim;
    d->nb = w->nb;
    d->nbp = w->nbp;
    d->row_q_bytes = w->nbp * w->qb;
    d->row_s_bytes = w->scp * (w->type == ZQ_TYPE_Q4_1 ? 4u : 2u);
    d->pad_ = 0;
    d->n_tiles = (w->out_dim + 7) / 8;
    d->tiles_div = d->n_tiles / grid;
    d->tiles_rem = d->n_tiles % grid;
    const uint32_t QUAD = w->qb * 4, SB = w->type == ZQ_TYPE_Q4_1 ? 4u : 2u, nq = w->nbp / 4;
    auto q_pitch = [&](uint32_t cq) { return cq * QUAD + ((QUAD == 64 && !(cq & 1u)) ? 64u : 0u); };
    auto piece_bytes = [&](uint32_t cq) { return 8 * (q_pitch(cq) + ((cq * 4 * SB + 15u) & ~15u) + 16u); };
    if (nq <= 16 && 8 * (d->row_q_bytes + d->row_s_bytes) <= slot_bytes) {
        d->chunks = 1;
        d->chunk_quads = nq;
        d->chunk_q_pitch = d->row_q_bytes;
    } else {
        uint32_t cq = nq < 16 ? nq : 16;
        while (cq > 1 && piece_bytes(cq) > slot_bytes) --cq;
        if (piece_bytes(cq) > slot_bytes) return false;
        d->chunk_quads = cq;
        d->chunks = (nq + cq - 1) / cq;
        d->chunk_q_pitch = q_pitch(cq);
    }
    d->chunks_magic = d->chunks <= 1 ? 0xFFFFFFFFu : (uint32_t)(0x100000000ull / d->chunks);
    return true;
}

}  // namespace

struct GptDecoder {
    GParams p;
    GLayer* d_layers = nullptr;
    void* d_misc = nullptr;  // abort word and the exchange buffers
    size_t smem = 0;
    uint32_t grid = 0;
    uint32_t launches = 0;
    uint32_t epoch = 1;
    uint32_t exchanges_per_step = 0;
    size_t misc_bytes = 0;
    ~GptDecoder() {
        cudaFree(d_layers);
        cudaFree(d_misc);
    }
};

void gpt_decoder_free(GptDecoder* d) { delete d; }

int gpt_decoder_create(const GptDecoderDesc& desc, GptDecoder** out) {
    *out = nullptr;
    const uint32_t E = desc.embed, H = desc.n_head, F = desc.ffn;
    if (!E || !H || E % H || E % 32 || F % 32) return ZQ_ERR_UNSUPPORTED;
    const uint32_t D = E / H;
    if (D % 16 || desc.layers.empty()) return ZQ_ERR_UNSUPPORTED;
    int dev = 0, max_smem = 0, coop = 0;
    ZQ_CUDA(cudaGetDevice(&dev));
    ZQ_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    ZQ_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) return ZQ_ERR_UNSUPPORTED;

    GptDecoder* d = new (std::nothrow) GptDecoder;
    if (!d) return ZQ_ERR_NO_MEM;
    GParams& p = d->p;
    memset(&p, 0, sizeof(p));
    const uint32_t grid = (uint32_t)sm_count();
    const uint32_t slot_bytes = 9856u;  // eight q4_0 / q8_0 rows of 1152 weights with their scales; three f32 rows of 768
    if (E * 4u > slot_bytes) {
        delete d;
        return ZQ_ERR_UNSUPPORTED;
    }
    std::vector<GLayer> layers(desc.layers.size());
    memset(static_cast<void*>(layers.data()), 0, layers.size() * sizeof(GLayer));
    bool ok = true;
    uint32_t max_tiles = 0;
    auto note = [&](const GMat& m) {
        const uint32_t t = m.tiles_div + (m.tiles_rem ? 1u : 0u);
        if (t > max_tiles) max_tiles = t;
    };
    for (size_t l = 0; ok && l < layers.size(); ++l) {
        const GptDecoderLayer& s = desc.layers[l];
        GLayer& L = layers[l];
        ok = g_describe(&L.qkv, s.qkv, s.qkv_b, slot_bytes, grid) && g_describe(&L.proj, s.proj, s.proj_b, slot_bytes, grid) &&
             g_describe(&L.fc, s.fc, s.fc_b, slot_bytes, grid) && g_describe(&L.mproj, s.mproj, s.mproj_b, slot_bytes, grid);
        if (!ok) break;
        ok = s.qkv->in_dim == E && s.qkv->out_dim == 3 * E && s.proj->in_dim == E && s.proj->out_dim == E &&
             s.fc->in_dim == E && s.fc->out_dim == F && s.mproj->in_dim == F && s.mproj->out_dim == E;
        note(L.qkv);
        note(L.proj);
        note(L.fc);
        note(L.mproj);
        L.ln1_w = s.ln1_w;
        L.ln1_b = s.ln1_b;
        L.ln2_w = s.ln2_w;
        L.ln2_b = s.ln2_b;
        L.kc = s.kc;
        L.vc = s.vc;
    }
    if (!ok) {
        delete d;
        return ZQ_ERR_UNSUPPORTED;
    }
    p.wte = desc.wte;
    p.wpe = desc.wpe;
    p.ln_f_w = desc.ln_f_w;
    p.ln_f_b = desc.ln_f_b;
    p.logits = desc.logits;
    p.state = desc.state;
    p.record = desc.record;
    p.n_layer = (uint32_t)layers.size();
    p.E = E;
    p.H = H;
    p.D = D;
    p.F = F;
    p.ctx = desc.ctx;
    p.vocab = desc.vocab;
    p.eps = desc.eps;
    p.head_rows = slot_bytes / (E * 4u);
    if (p.head_rows > 8) p.head_rows = 8;
    p.head_units = (desc.vocab + p.head_rows - 1) / p.head_rows;
    p.head_div = p.head_units / grid;
    p.head_rem = p.head_units % grid;
    auto magic = [](uint32_t x) { return x <= 1 ? 0xFFFFFFFFu : (uint32_t)(0x100000000ull / x); };
    p.magic_H = magic(H);
    p.magic_D8 = magic(D / 8);
    p.part_rows = max_tiles * 8;

    auto up = [](size_t v, size_t a) { return (v + a - 1) / a * a; };
    const uint32_t K = ((E > F ? E : F) + 127u) & ~127u;  // whole quads
    p.h_floats = K;
    size_t off = kGSharedHead;
    p.off_layers = (uint32_t)off;
    off = up(off + layers.size() * sizeof(GLayer), 128);
    p.off_xres = (uint32_t)off;
    off = up(off + (size_t)E * 4, 128);
    p.off_h = (uint32_t)off;
    off = up(off + (size_t)K * 4, 128);
    p.off_q = (uint32_t)off;
    off = up(off + (size_t)3 * E * 4, 128);
    p.off_lnw = (uint32_t)off;
    off = up(off + (size_t)2 * E * 4, 128);
    p.off_part = (uint32_t)off;
    off = up(off + (size_t)kConsumerWarps * p.part_rows * 4, 128);
    p.off_scratch = (uint32_t)off;
    off = up(off + ((size_t)((desc.ctx + 3u) & ~3u) + 64 * 8) * 4, 128);
    p.off_ring = (uint32_t)off;
    const size_t budget = (size_t)max_smem - 256;
    if (off + 8 * (size_t)slot_bytes > budget) {
        delete d;
        return ZQ_ERR_UNSUPPORTED;
    }
    uint32_t n_slots = (uint32_t)((budget - off) / slot_bytes);
    if (n_slots > 16) n_slots = 16;
    p.n_slots = n_slots;
    p.slot_magic = (uint32_t)(0x100000000ull / n_slots);
    p.slot_bytes = slot_bytes;
    d->smem = off + (size_t)n_slots * slot_bytes;
    d->grid = grid;
    cudaError_t e = cudaFuncSetAttribute(gpt2_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d->smem);
    int per_sm = 0;
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gpt2_decode_kernel, kThreads, d->smem);
    if (e != cudaSuccess || per_sm < 1) {
        delete d;
        if (e != cudaSuccess) return cuda_fail(e);
        return ZQ_ERR_UNSUPPORTED;
    }
    GExchange& ex = p.ex;
    ex.qkv_n = 3 * E;
    ex.scores_n = H * desc.ctx;
    ex.att_n = E;
    ex.proj_n = E;
    ex.fc_n = F;
    ex.mproj_n = E + grid;
    ex.best_n = 2 * grid;
    const size_t words = 2 * ((size_t)ex.qkv_n + ex.scores_n + ex.att_n + ex.proj_n + ex.fc_n + ex.mproj_n + ex.best_n);
    d->misc_bytes = 256 + words * 8;
    if (cudaMalloc(&d->d_layers, layers.size() * sizeof(GLayer)) != cudaSuccess ||
        cudaMalloc(&d->d_misc, d->misc_bytes) != cudaSuccess) {
        delete d;
        return ZQ_ERR_NO_MEM;
    }
    e = cudaMemcpy(d->d_layers, layers.data(), layers.size() * sizeof(GLayer), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(d->d_misc, 0, d->misc_bytes);
    if (e != cudaSuccess) {
        delete d;
        return cuda_fail(e);
    }
    p.layers = d->d_layers;
    p.abort_word = static_cast<uint32_t*>(d->d_misc);
    unsigned long long* w = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(d->d_misc) + 256);
    ex.qkv = w;
    w += 2 * (size_t)ex.qkv_n;
    ex.scores = w;
    w += 2 * (size_t)ex.scores_n;
    ex.att = w;
    w += 2 * (size_t)ex.att_n;
    ex.proj = w;
    w += 2 * (size_t)ex.proj_n;
    ex.fc = w;
    w += 2 * (size_t)ex.fc_n;
    ex.mproj = w;
    w += 2 * (size_t)ex.mproj_n;
    ex.best = w;
    d->exchanges_per_step = 6 * p.n_layer + 1;
    int rc = device_error_word(&p.err);
    if (rc != ZQ_OK) {
        delete d;
        return rc;
    }
    *out = d;
    return ZQ_OK;
}

int gpt_decoder_run(GptDecoder* d, uint32_t n_steps, int variant, cudaStream_t st) {
    if (n_steps == 0) return ZQ_OK;
    // Only a greedy run ends every step with an exchange among all CTAs (the arg-max candidates), which is what lets
    // the next step reuse the buffers of the layers before.
    if (n_steps > 1 && variant != DECODE_GREEDY) return ZQ_ERR_BAD_ARG;
    uint32_t launch_id = d->launches + 1u;
    if (launch_id == 0u) launch_id = 1u;
    // Exchange numbers never repeat while a buffer may still hold an old one: when the 32-bit counter would wrap,
    // the buffers are cleared (stream-ordered) and numbering restarts.
    const uint64_t need = (uint64_t)n_steps * d->exchanges_per_step + 2;
    if ((uint64_t)d->epoch + need >= 0xFFFFFFF0ull) {
        ZQ_CUDA(cudaMemsetAsync(static_cast<unsigned char*>(d->d_misc) + 256, 0, d->misc_bytes - 256, st));
        d->epoch = 1;
    }
    uint32_t epoch_base = d->epoch;
    void* args[] = {&d->p, &n_steps, &variant, &launch_id, &epoch_base};
    ZQ_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(gpt2_decode_kernel), dim3(d->grid), dim3(kThreads), args,
                                        d->smem, st));
    d->launches = launch_id;
    d->epoch += (uint32_t)need;
    return ZQ_OK;
}

}  // namespace zq
