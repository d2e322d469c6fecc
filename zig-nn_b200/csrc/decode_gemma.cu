// One persistent cooperative kernel per Gemma-3 decode step (or per run of greedy steps): the whole
// token — embedding, 26 x (norm, qkv, attention, o, norm, gate/up, GeGLU, down), final norm, logits,
// argmax — runs as phases of ONE grid of one CTA per SM, separated by grid barriers, instead of about
// 270 dependent kernel launches (gemma3.zig:662-846; the one-encoder form of gemma3_metal.zig:189-260).
//
// Arithmetic. Every phase performs the roundings of the launch-sequence engine (ops.cu, gemv_q8.cu) in
// the same order — exact int8 block dots, block terms (d*s)*float(idot) added in block order, 16-lane
// sums of squares, exponentials added one by one, values accumulated position by position — so logits
// are bit-identical to that path and to the CPU code.
//
// Structure of a CTA: 16 consumer warps + 1 producer warp.
//   * The producer walks the static schedule of weight "units" (a few whole rows of a matrix with their
//     scales) that this CTA will need, in order, and streams them into a ring of shared-memory slots
//     with cp.async.bulk + mbarrier. Weights do not depend on activations, so the producer runs ahead
//     of the consumers across phase and token boundaries: HBM keeps streaming while the consumers sit
//     in a grid barrier, a norm or the attention's serial chains.
//   * Small vectors (the residual stream, norms, the quantised activation image) are recomputed by every
//     CTA in its own shared memory rather than exchanged: that removes the grid barrier a separate
//     norm phase would need.
//   * Cross-CTA data (qkv, scores, attention output, projections) goes through global memory (L2).
//
// Every wait is bounded: a grid barrier or slot wait that runs out records a code in the device error
// word, raises the abort flag, and every CTA drains its copies in flight and returns.
#include <math.h>
#include <stdlib.h>

#include <new>
#include <vector>

#include "decode_gemma.h"
#include "zq_internal.h"

namespace zq {
namespace {

constexpr int kConsumerWarps = 16;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;
constexpr unsigned int kErrGridBarrier = 0x47424152u;  // 'GBAR'
constexpr unsigned int kErrUnitWait = 0x554E4954u;     // 'UNIT'
constexpr uint32_t kGridSpinLimit = 1u << 22;
constexpr uint32_t kSlotSpinLimit = 1u << 22;
constexpr uint32_t kVTile = 512;  // positions per V tile of the attention phase

enum { EP_STORE = 0, EP_GEGLU = 1, EP_LOGITS = 2 };

// A quantised matrix as the kernel walks it: units of `rows_per_unit` whole rows.
struct DMat {
    const uint8_t* qs;
    const uint8_t* sc;
    uint32_t type, n_rows, nb, nbp;
    uint32_t row_q_bytes, row_s_bytes;
    uint32_t rows_per_unit, n_units;
    uint32_t split;  // 1: a unit holds rows_per_unit/2 rows of the first half and the matching rows of the second
};

struct DLayer {
    DMat qkv, o, gate_up, down;
    const float *attn_norm_w, *post_attn_norm_w, *q_norm_w, *k_norm_w, *ffn_norm_w, *post_ffw_norm_w;
    float *kc, *vc;
    uint32_t window;  // 0: every position (global layer)
};

struct DParams {
    const DLayer* layers;
    DMat head;  // token_embd: embedding rows and the tied logits head
    const float* output_norm_w;
    const float* freqs;
    float *qkv, *scores, *att, *proj, *g, *ffn, *logits;
    uint32_t* state;   // [0] token, [1] position, [2] next slot of the greedy record
    uint32_t* record;
    uint32_t* sync;    // [0], [1]: barrier counters used by alternate launches; [2]: abort flag
    float* part_val;   // per-CTA argmax candidates
    uint32_t* part_idx;
    unsigned int* err;
    long long* prof;   // optional: per-CTA cycle stamps of one step (prof_cap per CTA); nullptr = off
    uint32_t prof_cap;
    uint32_t n_layer, E, D, n_head, n_kv, F, ctx, max_len;
    float eps, embed_scale;
    // shared-memory carve-up (bytes from the start of dynamic shared memory)
    uint32_t n_slots, slot_bytes, off_ring, off_xres, off_xs, off_rope, off_scratch, terms_per_warp, nbp_max;
};

// ---- small device helpers --------------------------------------------------------------------

__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

__device__ __forceinline__ float exp_f32(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float gelu_tanh(float v) {
    const float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v);
    const float inner = __fmul_rn(0.7978845608f, __fadd_rn(v, cube));
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, (float)tanh((double)inner)));
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    return v;
}
__device__ __forceinline__ uint32_t pick(const uint4& v, int j) {
    return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w;
}
__device__ __forceinline__ int quad_transpose_reduce(const int (&p)[4], int t) {
    const bool upper = t & 2;
    const int keep0 = upper ? p[2] : p[0], keep1 = upper ? p[3] : p[1];
    const int send0 = upper ? p[0] : p[2], send1 = upper ? p[1] : p[3];
    const int a0 = keep0 + __shfl_xor_sync(0xFFFFFFFFu, send0, 2);
    const int a1 = keep1 + __shfl_xor_sync(0xFFFFFFFFu, send1, 2);
    const bool odd = t & 1;
    const int keep = odd ? a1 : a0, send = odd ? a0 : a1;
    return keep + __shfl_xor_sync(0xFFFFFFFFu, send, 1);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Shared state of one CTA.
struct Cta {
    unsigned char* smem;
    uint32_t smem32;
    uint32_t full0, empty0;  // shared addresses of the mbarrier arrays
    volatile int* s_abort;
    int* s_ok;
    float* part;   // 16 lane sums
    float* bc;     // broadcast cell
    float* red;    // 16 per-warp partials + spare
    int tid, lane, warp;
    uint32_t epoch;   // grid barriers passed (thread 0 only uses it)
    uint32_t launch_id;  // the abort word holds the id of the launch that gave up
    volatile uint32_t* released;  // per ring slot: uses consumed so far
};

// Bounded wait for a ring slot. On a timeout the CTA-wide abort flag is raised; the caller skips its work
// and the CTA leaves together at the next grid barrier.
__device__ __forceinline__ bool slot_wait(const Cta& c, uint32_t bar, uint32_t parity, unsigned int* err) {
    for (uint32_t i = 0; i < kSlotSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *c.s_abort) return false;
    }
    *c.s_abort = 1;
    atomicExch(err, kErrUnitWait);
    return false;
}

// Grid barrier over the consumer threads of every CTA. Returns false (to every consumer thread of the CTA)
// when this CTA has raised its abort flag, another CTA has, or the wait ran out.
__device__ __forceinline__ bool grid_barrier(Cta& c, const DParams& p, uint32_t* counter) {
    cbar();
    if (c.tid == 0) {
        bool ok = !*c.s_abort;
        if (ok) {
            c.epoch += 1;
            const uint32_t target = c.epoch * gridDim.x;
            red_release_gpu_add(counter, 1u);
            ok = false;
            for (uint32_t i = 0; i < kGridSpinLimit; ++i) {
                if ((int32_t)(ld_acquire_gpu(counter) - target) >= 0) {
                    ok = true;
                    break;
                }
                if ((i & 63u) == 63u && ld_acquire_gpu(p.sync + 2) == c.launch_id) break;
            }
            if (!ok && ld_acquire_gpu(p.sync + 2) != c.launch_id) atomicExch(p.err, kErrGridBarrier);
        }
        if (!ok) {
            atomicExch(p.sync + 2, c.launch_id);
            *c.s_abort = 1;
        }
        *c.s_ok = ok ? 1 : 0;
    }
    cbar();
    return *c.s_ok != 0;
}

// Sum of squares in the CPU loop's order (gemma3.zig:920-930): 16 lane accumulators, lanes added 0..15,
// then the tail. `xs` complete before the call (a cbar lies between its writes and this call).
__device__ __forceinline__ float sumsq_lanes16(const Cta& c, const float* xs, uint32_t dim) {
    const uint32_t dim16 = dim & ~15u;
    if (c.tid < 16) {
        float acc = 0.0f;
        uint32_t i = c.tid;
        for (; i + 16 * 7 < dim16; i += 16 * 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = xs[i + 16 * u];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = __fmul_rn(v[u], v[u]);
#pragma unroll
            for (int u = 0; u < 8; ++u) acc = __fadd_rn(acc, v[u]);
        }
        for (; i < dim16; i += 16) acc = __fadd_rn(acc, __fmul_rn(xs[i], xs[i]));
        c.part[c.tid] = acc;
    }
    cbar();
    if (c.tid == 0) {
        float ss = c.part[0];
#pragma unroll
        for (int l = 1; l < 16; ++l) ss = __fadd_rn(ss, c.part[l]);
        for (uint32_t i = dim16; i < dim; ++i) ss = __fadd_rn(ss, __fmul_rn(xs[i], xs[i]));
        *c.bc = ss;
    }
    cbar();
    return *c.bc;
}
// Squares added one by one (rms_norm_in_place, gemma3.zig:949-959).
__device__ __forceinline__ float sumsq_sequential(const float* xs, uint32_t dim) {
    float ss = 0.0f;
    uint32_t i = 0;
    for (; i + 8 <= dim; i += 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = xs[i + u];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __fmul_rn(v[u], v[u]);
#pragma unroll
        for (int u = 0; u < 8; ++u) ss = __fadd_rn(ss, v[u]);
    }
    for (; i < dim; ++i) ss = __fadd_rn(ss, __fmul_rn(xs[i], xs[i]));
    return ss;
}

// The quantised activation row as the dot kernels read it: word w of block b at xl/xh[(b/4)*4 + w%4]
// component b%4 (xl: w < 4, xh: w >= 4) — the interleave of the weights.
struct XImage {
    uint4* xl;
    uint4* xh;
    float* xsc;
    int32_t* xsum;
};
__device__ __forceinline__ XImage ximage(unsigned char* scratch, uint32_t nbp_max) {
    XImage x;
    x.xl = reinterpret_cast<uint4*>(scratch);
    x.xh = x.xl + nbp_max;
    x.xsc = reinterpret_cast<float*>(x.xh + nbp_max);
    x.xsum = reinterpret_cast<int32_t*>(x.xsc + nbp_max);
    return x;
}

// quantize_row_q8 (simd_dot.zig:25-64) of the 32 values held one per lane, written into the image.
__device__ __forceinline__ void quant_block_to_image(float v, uint32_t b, int lane, const XImage& x) {
    float amax = fabsf(v);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, s);
    float r = roundf(__fmul_rn(v, inv));
    r = fminf(127.0f, fmaxf(-127.0f, r));
    const int qi = (int)r;
    int acc = qi;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    const uint32_t w = (uint32_t)lane >> 2;
    unsigned char* dst = reinterpret_cast<unsigned char*>(w < 4 ? x.xl : x.xh);
    dst[((((b >> 2) * 4 + (w & 3u)) * 4 + (b & 3u)) << 2) + ((uint32_t)lane & 3u)] = (unsigned char)(signed char)qi;
    if (lane == 0) {
        x.xsc[b] = s;
        x.xsum[b] = acc;
    }
}
// Blocks [nb, nbp) of the image (row padding): zero quants, scale 1.
__device__ __forceinline__ void image_padding(const Cta& c, const XImage& x, uint32_t nb, uint32_t nbp) {
    for (uint32_t i = nb * 8 + c.tid; i < nbp * 8; i += kConsumers) {
        const uint32_t b = i >> 3, w = i & 7u;
        uint32_t* dst = reinterpret_cast<uint32_t*>(w < 4 ? x.xl : x.xh);
        dst[((b >> 2) * 4 + (w & 3u)) * 4 + (b & 3u)] = 0u;
    }
    for (uint32_t b = nb + c.tid; b < nbp; b += kConsumers) {
        x.xsc[b] = 1.0f;
        x.xsum[b] = 0;
    }
}
// Quantise a dense f32 vector from global memory into the image.
__device__ __forceinline__ void quantise_global(const Cta& c, const float* src, uint32_t dim, const XImage& x) {
    for (uint32_t i = c.tid; i < dim; i += kConsumers) quant_block_to_image(__ldcg(src + i), i >> 5, c.lane, x);
    image_padding(c, x, dim >> 5, (dim / 32 + 3u) & ~3u);
}

// xres (+)= rms_norm(src, w1) when src != nullptr; then h = rms_norm(xres, w2) quantised into the image
// (gemma3.zig:662-666, 725-737, 768-773 followed by the row quantiser of the next linear).
__device__ __forceinline__ void norm_quant(const Cta& c, const float* src, const float* w1, const float* w2,
                                           float* xres, float* xs, uint32_t dim, float eps, const XImage& x) {
    if (src) {
        for (uint32_t i = c.tid; i < dim; i += kConsumers) xs[i] = __ldcg(src + i);
        cbar();
        const float ss = sumsq_lanes16(c, xs, dim);
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
        for (uint32_t i = c.tid; i < dim; i += kConsumers)
            xres[i] = __fadd_rn(xres[i], __fmul_rn(__fmul_rn(xs[i], inv), __ldg(w1 + i)));
    }
    cbar();
    const float ss = sumsq_lanes16(c, xres, dim);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
    for (uint32_t i = c.tid; i < dim; i += kConsumers)
        quant_block_to_image(__fmul_rn(__fmul_rn(xres[i], inv), __ldg(w2 + i)), i >> 5, c.lane, x);
    image_padding(c, x, dim >> 5, (dim / 32 + 3u) & ~3u);
}

// Block terms of one unit (`rows` whole rows in shared memory): lane (pair, t) handles (row, quad) pairs,
// 8 per warp pass; after the 4-lane transpose-reduce lane t holds the exact dot of block 4*quad + t.
template <int TYPE>
__device__ __forceinline__ void unit_terms(const unsigned char* slab_q, const unsigned char* slab_s, uint32_t rows,
                                           uint32_t nq, uint32_t row_q_bytes, uint32_t row_s_bytes, const XImage& x,
                                           float* terms, uint32_t pitch, int lane) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QUAD = Q8 ? 128 : 64;
    const int t = lane & 3;
    const uint32_t total = rows * nq;
    uint32_t r = ((uint32_t)lane >> 2) / nq, q = ((uint32_t)lane >> 2) - r * nq;
    const uint32_t passes = (total + 7) / 8;
#pragma unroll 2
    for (uint32_t it = 0; it < passes; ++it) {
        const bool valid = r < rows;
        const uint32_t rr = valid ? r : 0u, qq = valid ? q : 0u;
        const unsigned char* pw = slab_q + (size_t)rr * row_q_bytes + qq * QUAD + 16 * t;
        const uint4 wa = *reinterpret_cast<const uint4*>(pw);
        uint4 wa2 = wa;
        if (Q8) wa2 = *reinterpret_cast<const uint4*>(pw + 64);
        const uint32_t blk = qq * 4 + t;
        float d, m = 0.0f;
        if (Q41) {
            const __half2 h = *reinterpret_cast<const __half2*>(slab_s + (size_t)rr * row_s_bytes + blk * 4);
            d = __low2float(h);
            m = __high2float(h);
        } else {
            d = __half2float(*reinterpret_cast<const __half*>(slab_s + (size_t)rr * row_s_bytes + blk * 2));
        }
        const uint4 xlo = x.xl[qq * 4 + t], xhi = x.xh[qq * 4 + t];
        int p4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int x0 = (int)pick(xlo, j), x1 = (int)pick(xhi, j);
            if (Q8) {
                p4[j] = __dp4a((int)pick(wa2, j), x1, __dp4a((int)pick(wa, j), x0, 0));
            } else {
                const uint32_t u = pick(wa, j);
                p4[j] = __dp4a((int)((u >> 4) & 0x0F0F0F0Fu), x1, __dp4a((int)(u & 0x0F0F0F0Fu), x0, 0));
            }
        }
        int idot = quad_transpose_reduce(p4, t);
        const float s = x.xsc[blk];
        const int qsum = x.xsum[blk];
        if (TYPE == ZQ_TYPE_Q4_0) idot -= 8 * qsum;
        float term = __fmul_rn(__fmul_rn(d, s), (float)idot);
        if (Q41) term = __fadd_rn(term, __fmul_rn(__fmul_rn(m, s), (float)qsum));
        if (valid) terms[rr * pitch + blk] = term;
        q += 8;
        while (q >= nq) {
            q -= nq;
            ++r;
        }
    }
}

struct Best {
    float v;
    uint32_t i;
};
__device__ __forceinline__ void best_update(Best& b, float v, uint32_t i) {
    if (v > b.v || (v == b.v && i < b.i)) {
        b.v = v;
        b.i = i;
    }
}

// One matrix-vector phase: this CTA's units of `m`, taken by the consumer warps in turn from the ring.
// The activation image is complete (cbar) before the call. Returns with *unit_base advanced.
__device__ __forceinline__ void gemv_phase(const Cta& c, const DParams& p, const DMat& m, uint32_t* unit_base,
                                           const XImage& x, float* terms_all, int ep, float* out, Best* best) {
    const uint32_t G = gridDim.x, cta = blockIdx.x;
    const uint32_t n_units = m.n_units;
    const uint32_t mine = n_units > cta ? (n_units - cta - 1) / G + 1 : 0;
    const uint32_t base = *unit_base;
    *unit_base = base + mine;
    if (c.warp >= kConsumerWarps) return;
    const uint32_t type = m.type, nb = m.nb, nq = m.nbp >> 2, pitch = m.nbp + 1;
    const uint32_t rqb = m.row_q_bytes, rsb = m.row_s_bytes, R = m.rows_per_unit, N = m.n_rows;
    float* terms = terms_all + (size_t)c.warp * p.terms_per_warp;
    for (uint32_t i = c.warp; i < mine; i += kConsumerWarps) {
        const uint32_t gi = base + i, slot = gi % p.n_slots, use = gi / p.n_slots;
        const uint32_t u = cta + i * G;
        uint32_t rows, row0;
        if (m.split) {
            const uint32_t half = R >> 1, n_half = N >> 1;
            row0 = u * half;
            rows = 2 * min(half, n_half - row0);
        } else {
            row0 = u * R;
            rows = min(R, N - row0);
        }
        // The slot's previous use must have been consumed before its barrier is read: a parity wait alone
        // cannot tell fill `use` from fill `use - 2`.
        bool ready = true;
        if (use > 0) {
            uint32_t spins = 0;
            while (c.released[slot] < use && ++spins < kSlotSpinLimit) {
            }
            ready = c.released[slot] >= use;
            if (!ready) {
                *c.s_abort = 1;
                atomicExch(p.err, kErrUnitWait);
            }
        }
        ready = ready && slot_wait(c, c.full0 + slot * 8, use & 1u, p.err);
        if (!__all_sync(0xFFFFFFFFu, ready)) break;  // the whole warp leaves together
        const unsigned char* slab_q = c.smem + p.off_ring + (size_t)slot * p.slot_bytes;
        const unsigned char* slab_s = slab_q + (size_t)rows * rqb;
        if (type == ZQ_TYPE_Q8_0)
            unit_terms<ZQ_TYPE_Q8_0>(slab_q, slab_s, rows, nq, rqb, rsb, x, terms, pitch, c.lane);
        else if (type == ZQ_TYPE_Q4_0)
            unit_terms<ZQ_TYPE_Q4_0>(slab_q, slab_s, rows, nq, rqb, rsb, x, terms, pitch, c.lane);
        else
            unit_terms<ZQ_TYPE_Q4_1>(slab_q, slab_s, rows, nq, rqb, rsb, x, terms, pitch, c.lane);
        __syncwarp();
        if (c.lane == 0) {  // the slot's bytes have been read
            c.released[slot] = use + 1;
            __threadfence_block();
            mbar_arrive(c.empty0 + slot * 8);
        }
        // one lane per row adds the row's terms in block order, as the CPU loop does
        float run = 0.0f;
        if ((uint32_t)c.lane < rows) {
            const float* tr = terms + c.lane * pitch;
            uint32_t b = 0;
            for (; b + 4 <= nb; b += 4) {
                const float t0 = tr[b], t1 = tr[b + 1], t2 = tr[b + 2], t3 = tr[b + 3];
                run = __fadd_rn(run, t0);
                run = __fadd_rn(run, t1);
                run = __fadd_rn(run, t2);
                run = __fadd_rn(run, t3);
            }
            for (; b < nb; ++b) run = __fadd_rn(run, tr[b]);
        }
        if (ep == EP_GEGLU) {
            const uint32_t half = rows >> 1;
            const float up = __shfl_down_sync(0xFFFFFFFFu, run, half);
            if ((uint32_t)c.lane < half) out[row0 + c.lane] = __fmul_rn(gelu_tanh(run), up);
        } else if ((uint32_t)c.lane < rows) {
            out[row0 + c.lane] = run;
            if (ep == EP_LOGITS && best) best_update(*best, run, row0 + c.lane);
        }
        __syncwarp();  // the terms are rewritten by the warp's next unit
    }
}

// The producer's side of gemv_phase: issue this CTA's units of `m` into the ring, in the same order.
__device__ __forceinline__ bool produce_phase(const Cta& c, const DParams& p, const DMat& m, uint32_t* unit_base,
                                              uint32_t* issued) {
    const uint32_t G = gridDim.x, cta = blockIdx.x;
    const uint32_t mine = m.n_units > cta ? (m.n_units - cta - 1) / G + 1 : 0;
    const uint32_t base = *unit_base;
    *unit_base = base + mine;
    const uint32_t rqb = m.row_q_bytes, rsb = m.row_s_bytes, R = m.rows_per_unit, N = m.n_rows;
    for (uint32_t i = 0; i < mine; ++i) {
        const uint32_t gi = base + i, slot = gi % p.n_slots, use = gi / p.n_slots;
        const uint32_t u = cta + i * G;
        if (use > 0 && !slot_wait(c, c.empty0 + slot * 8, (use - 1) & 1u, p.err)) return false;
        const uint32_t dst = c.smem32 + p.off_ring + slot * p.slot_bytes;
        const uint32_t bar = c.full0 + slot * 8;
        if (m.split) {
            const uint32_t half = R >> 1, n_half = N >> 1;
            const uint32_t row0 = u * half, h = min(half, n_half - row0);
            const uint32_t qb = h * rqb, sb = h * rsb;
            mbar_arrive_expect_tx(bar, 2 * (qb + sb));
            bulk_copy_g2s(dst, m.qs + (size_t)row0 * rqb, qb, bar);
            bulk_copy_g2s(dst + qb, m.qs + (size_t)(n_half + row0) * rqb, qb, bar);
            bulk_copy_g2s(dst + 2 * qb, m.sc + (size_t)row0 * rsb, sb, bar);
            bulk_copy_g2s(dst + 2 * qb + sb, m.sc + (size_t)(n_half + row0) * rsb, sb, bar);
        } else {
            const uint32_t row0 = u * R, rows = min(R, N - row0);
            const uint32_t qb = rows * rqb, sb = rows * rsb;
            mbar_arrive_expect_tx(bar, qb + sb);
            bulk_copy_g2s(dst, m.qs + (size_t)row0 * rqb, qb, bar);
            bulk_copy_g2s(dst + qb, m.sc + (size_t)row0 * rsb, sb, bar);
        }
        *issued = gi + 1;
    }
    return true;
}

// Embedding row of `tok`, dequantised and scaled (gemma3.zig:800-803, 855-871): q*d, then *scale.
__device__ __forceinline__ void embed_row(const Cta& c, const DMat& m, uint32_t tok, float scale, float* xres,
                                          uint32_t dim) {
    const unsigned char* qrow = m.qs + (size_t)tok * m.row_q_bytes;
    const unsigned char* srow = m.sc + (size_t)tok * m.row_s_bytes;
    for (uint32_t k = c.tid; k < dim; k += kConsumers) {
        const uint32_t blk = k >> 5, j = k & 31u;
        float v;
        if (m.type == ZQ_TYPE_Q8_0) {
            const float d = __half2float(reinterpret_cast<const __half*>(srow)[blk]);
            const int8_t q = (int8_t)qrow[qs_word_offset(32, blk, j >> 2) + (j & 3u)];
            v = __fmul_rn((float)q, d);
        } else {
            const uint32_t jb = j & 15u;
            const unsigned char byte = qrow[qs_word_offset(16, blk, jb >> 2) + (jb & 3u)];
            const int nib = (j < 16) ? (byte & 0x0F) : (byte >> 4);
            if (m.type == ZQ_TYPE_Q4_0) {
                v = __fmul_rn((float)(nib - 8), __half2float(reinterpret_cast<const __half*>(srow)[blk]));
            } else {
                const __half2 dm = reinterpret_cast<const __half2*>(srow)[blk];
                v = __fadd_rn(__fmul_rn((float)nib, __low2float(dm)), __high2float(dm));
            }
        }
        xres[k] = __fmul_rn(v, scale);
    }
}

// Attention, first half (gemma3.zig:689-716, 1062-1090): every CTA normalises and rotates the query heads
// and this step's key heads in its own shared memory; CTA 0 stores the key / value rows of position `pos`;
// the scores of the window are spread over the CTAs in tiles of 32 (position, head) pairs.
__device__ __forceinline__ void scores_phase(const Cta& c, const DParams& p, const DLayer& L, uint32_t pos,
                                             uint32_t kv_start, uint32_t kv_len, const float* rope, float* qn) {
    const uint32_t D = p.D, nh = p.n_head, nkv = p.n_kv, group = nh / nkv, kv_dim = nkv * D;
    const uint32_t nvec = nh + nkv;
    for (uint32_t i = c.tid; i < nvec * D; i += kConsumers) qn[i] = __ldcg(p.qkv + i);
    cbar();
    for (uint32_t v = c.warp; v < nvec; v += kConsumerWarps)  // one chain per vector, one warp each
        if (c.lane == 0)
            c.red[v & 31u] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq_sequential(qn + v * D, D), (float)D), p.eps)));
    cbar();
    for (uint32_t i = c.tid; i < nvec * (D / 2); i += kConsumers) {
        const uint32_t v = i / (D / 2), j = i - v * (D / 2);
        const float* wn = v < nh ? L.q_norm_w : L.k_norm_w;
        float* vec = qn + v * D;
        const float inv = c.red[v & 31u];
        const float x0 = __fmul_rn(__fmul_rn(vec[2 * j], inv), __ldg(wn + 2 * j));
        const float x1 = __fmul_rn(__fmul_rn(vec[2 * j + 1], inv), __ldg(wn + 2 * j + 1));
        const float cs = rope[2 * j], sn = rope[2 * j + 1];
        vec[2 * j] = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
        vec[2 * j + 1] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
    }
    cbar();
    if (blockIdx.x == 0) {
        for (uint32_t i = c.tid; i < kv_dim; i += kConsumers) {
            L.kc[(size_t)pos * kv_dim + i] = qn[nh * D + i];
            L.vc[(size_t)pos * kv_dim + i] = __ldcg(p.qkv + (nh + nkv) * D + i);
        }
    }
    const uint32_t jobs = kv_len * nh, tiles = (jobs + 31) / 32;
    const uint32_t l = c.tid & 15u, js = c.tid >> 4;
    const uint32_t dim16 = D & ~15u;
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)D));
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const uint32_t job = tile * 32 + js;
        const bool live = job < jobs;
        const uint32_t jc = live ? job : jobs - 1;
        const uint32_t pi = jc / nh, h = jc - pi * nh, kvh = h / group;
        const float* qh = qn + h * D;
        const bool from_smem = pi == kv_len - 1;
        const float* kr = from_smem ? qn + (nh + kvh) * D : L.kc + (size_t)(kv_start + pi) * kv_dim + (size_t)kvh * D;
        float acc = 0.0f;
        for (uint32_t d0 = l; d0 < dim16; d0 += 16 * 8) {
            float kv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t d = d0 + 16 * u;
                kv[u] = d < dim16 ? (from_smem ? kr[d] : __ldcg(kr + d)) : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t d = d0 + 16 * u;
                if (d < dim16) acc = __fadd_rn(acc, __fmul_rn(qh[d], kv[u]));
            }
        }
        // lanes added in order 0..15 by lane 0 of the 16-lane group
        float s = __shfl_sync(0xFFFFFFFFu, acc, 0, 16);
#pragma unroll
        for (int j = 1; j < 16; ++j) s = __fadd_rn(s, __shfl_sync(0xFFFFFFFFu, acc, j, 16));
        if (l == 0 && live) {
            for (uint32_t d = dim16; d < D; ++d) s = __fadd_rn(s, __fmul_rn(qh[d], from_smem ? kr[d] : __ldcg(kr + d)));
            p.scores[(size_t)h * p.max_len + pi] = __fmul_rn(s, scale);
        }
    }
}

// Attention, second half (gemma3.zig:1092-1120): a job owns 8 output dimensions of one kv head for all the
// query heads that share it. Softmax per head (maximum, exp, the exponentials added one by one, times
// 1/sum), then out[d] += w[p] * v[p][d] position by position; V streams through shared memory in tiles.
__device__ __forceinline__ void softmax_v_phase(const Cta& c, const DParams& p, const DLayer& L, uint32_t kv_start,
                                                uint32_t kv_len, unsigned char* scratch) {
    const uint32_t D = p.D, nh = p.n_head, nkv = p.n_kv, group = nh / nkv, kv_dim = nkv * D;
    const uint32_t chunks = D / 8, jobs = nkv * chunks;
    float* w = reinterpret_cast<float*>(scratch);                      // [group][max_len]
    float* vt = w + (size_t)group * p.max_len;                         // [2][kVTile][8]
    const uint32_t vt32 = c.smem32 + (uint32_t)(reinterpret_cast<unsigned char*>(vt) - c.smem);
    const uint32_t wph = kConsumerWarps / group;                       // warps per head
    for (uint32_t job = blockIdx.x; job < jobs; job += gridDim.x) {
        const uint32_t kvh = job / chunks, dc = job - kvh * chunks;
        const float* vbase = L.vc + (size_t)kv_start * kv_dim + (size_t)kvh * D + dc * 8;
        auto fetch_tile = [&](uint32_t tile) {
            const uint32_t p0 = tile * kVTile, n = min(kVTile, kv_len - p0);
            const uint32_t dst = vt32 + (tile & 1u) * kVTile * 32;
            for (uint32_t i = c.tid; i < n * 2; i += kConsumers)
                cp_async16(dst + i * 16, vbase + (size_t)(p0 + (i >> 1)) * kv_dim + (i & 1u) * 4);
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        fetch_tile(0);  // in flight during the softmax
        {
            const uint32_t hg = c.warp / wph, tl = c.tid - hg * wph * 32, nt = wph * 32;
            const float* sh = p.scores + (size_t)(kvh * group + hg) * p.max_len;
            float* wh = w + (size_t)hg * p.max_len;
            float mx = -INFINITY;
            for (uint32_t q = tl; q < kv_len; q += nt) {
                const float v = __ldcg(sh + q);
                wh[q] = v;
                mx = fmaxf(mx, v);
            }
            mx = warp_max(mx);
            if (c.lane == 0) c.red[c.warp] = mx;
            cbar();
            mx = c.red[hg * wph];
            for (uint32_t k = 1; k < wph; ++k) mx = fmaxf(mx, c.red[hg * wph + k]);
            for (uint32_t q = tl; q < kv_len; q += nt) wh[q] = exp_f32(__fsub_rn(wh[q], mx));
            cbar();
            if ((uint32_t)c.tid < group) {  // one serial sum per head
                const float* wq = w + (size_t)c.tid * p.max_len;
                float s = 0.0f;
                uint32_t q = 0;
                for (; q + 8 <= kv_len; q += 8) {
                    const float4 a = *reinterpret_cast<const float4*>(wq + q);
                    const float4 b = *reinterpret_cast<const float4*>(wq + q + 4);
                    s = __fadd_rn(s, a.x); s = __fadd_rn(s, a.y); s = __fadd_rn(s, a.z); s = __fadd_rn(s, a.w);
                    s = __fadd_rn(s, b.x); s = __fadd_rn(s, b.y); s = __fadd_rn(s, b.z); s = __fadd_rn(s, b.w);
                }
                for (; q < kv_len; ++q) s = __fadd_rn(s, wq[q]);
                c.part[c.tid] = __fdiv_rn(1.0f, s);
            }
            cbar();
            const float inv = c.part[hg];
            for (uint32_t q = tl; q < kv_len; q += nt) wh[q] = __fmul_rn(wh[q], inv);
        }
        const uint32_t n_tiles = (kv_len + kVTile - 1) / kVTile;
        const bool chain = (uint32_t)c.tid < group * 8;  // thread (hg, d): one accumulation chain
        const uint32_t hg = (uint32_t)c.tid >> 3, d = (uint32_t)c.tid & 7u;
        float acc = 0.0f;
        for (uint32_t tile = 0; tile < n_tiles; ++tile) {
            if (tile + 1 < n_tiles) {
                fetch_tile(tile + 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            cbar();  // the tile (and, first pass, the weights) are complete for every thread
            if (chain) {
                const uint32_t p0 = tile * kVTile, n = min(kVTile, kv_len - p0);
                const float* vtile = vt + (size_t)(tile & 1u) * kVTile * 8;
                const float* wq = w + (size_t)hg * p.max_len + p0;
                uint32_t i = 0;
                for (; i + 8 <= n; i += 8) {
                    float vv[8], ww[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        vv[j] = vtile[(i + j) * 8 + d];
                        ww[j] = wq[i + j];
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc = __fadd_rn(acc, __fmul_rn(ww[j], vv[j]));
                }
                for (; i < n; ++i) acc = __fadd_rn(acc, __fmul_rn(wq[i], vtile[i * 8 + d]));
            }
            cbar();  // the buffer the next fetch overwrites has been consumed
        }
        if (chain) p.att[(size_t)(kvh * group + hg) * D + dc * 8 + d] = acc;
    }
}

__global__ void __launch_bounds__(kThreads, 1)
gemma3_decode_kernel(const __grid_constant__ DParams p, uint32_t n_steps, int variant, uint32_t launch_id) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ __align__(8) unsigned long long s_bars[2 * 64];
    __shared__ int s_abort, s_ok;
    __shared__ uint32_t s_released[64];
    __shared__ float s_part[16], s_bc, s_red[32];
    __shared__ float s_bval[kConsumerWarps];
    __shared__ uint32_t s_bidx[kConsumerWarps];

    Cta c;
    c.smem = smem;
    c.smem32 = (uint32_t)__cvta_generic_to_shared(smem);
    c.full0 = (uint32_t)__cvta_generic_to_shared(s_bars);
    c.empty0 = c.full0 + 64 * 8;
    c.s_abort = &s_abort;
    c.s_ok = &s_ok;
    c.part = s_part;
    c.bc = &s_bc;
    c.red = s_red;
    c.tid = threadIdx.x;
    c.lane = threadIdx.x & 31;
    c.warp = threadIdx.x >> 5;
    c.epoch = 0;
    c.released = s_released;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.n_slots; ++s) {
            mbar_init(c.full0 + s * 8, 1);
            mbar_init(c.empty0 + s * 8, 1);
            s_released[s] = 0;
        }

        s_abort = 0;
        s_ok = 1;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the counter of the next launch: nobody touches it during this one
        if (blockIdx.x == 0) p.sync[(launch_id ^ 1u) & 1u] = 0u;
    }
    __syncthreads();
    uint32_t* counter = p.sync + (launch_id & 1u);
    c.launch_id = launch_id;
    const bool want_logits = variant != DECODE_CACHE_ONLY;
    uint32_t unit_base = 0;

    if (c.warp == kConsumerWarps) {
        // ---------------------------------------------------------------- producer warp
        if (c.lane == 0) {
            bool ok = true;
            uint32_t issued = 0;
            for (uint32_t step = 0; ok && step < n_steps; ++step) {
                for (uint32_t l = 0; ok && l < p.n_layer; ++l) {
                    const DLayer& L = p.layers[l];
                    ok = produce_phase(c, p, L.qkv, &unit_base, &issued) && produce_phase(c, p, L.o, &unit_base, &issued) &&
                         produce_phase(c, p, L.gate_up, &unit_base, &issued) &&
                         produce_phase(c, p, L.down, &unit_base, &issued);
                }
                if (ok && want_logits) ok = produce_phase(c, p, p.head, &unit_base, &issued);
            }
            if (!ok) {
                // Stopped early: copies already issued still land in this CTA's shared memory. Wait (bounded)
                // for the newest fill of every slot before the CTA may retire.
                for (uint32_t s = 0; s < p.n_slots && s < issued; ++s) {
                    const uint32_t last = issued - 1 - ((issued - 1 - s) % p.n_slots);  // newest unit index in slot s
                    const uint32_t use = last / p.n_slots;
                    for (uint32_t i = 0; i < (1u << 16); ++i)
                        if (mbar_try_wait(c.full0 + s * 8, use & 1u)) break;
                }
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumer warps
    float* xres = reinterpret_cast<float*>(smem + p.off_xres);
    float* xs = reinterpret_cast<float*>(smem + p.off_xs);
    float* rope = reinterpret_cast<float*>(smem + p.off_rope);
    unsigned char* scratch = smem + p.off_scratch;
    const XImage x = ximage(scratch, p.nbp_max);
    float* terms_all = reinterpret_cast<float*>(x.xsum + p.nbp_max);
    const uint32_t E = p.E, D = p.D;
    uint32_t tok = __ldcg(p.state + 0), pos = __ldcg(p.state + 1), rec = __ldcg(p.state + 2);
    uint32_t n_stamp = 0;
    // cycle stamp of this CTA at a phase boundary (thread 0; profiling runs only)
#define ZQ_STAMP()                                                                              \
    do {                                                                                        \
        if (p.prof && c.tid == 0 && n_stamp < p.prof_cap) p.prof[(size_t)blockIdx.x * p.prof_cap + n_stamp++] = clock64(); \
    } while (0)

    for (uint32_t step = 0; step < n_steps; ++step) {
        ZQ_STAMP();
        embed_row(c, p.head, tok, p.embed_scale, xres, E);
        for (uint32_t j = c.tid; j < D / 2; j += kConsumers) {  // RoPE angles of this position, every layer
            const float theta = __fmul_rn((float)pos, __ldg(p.freqs + j));
            rope[2 * j] = (float)cos((double)theta);
            rope[2 * j + 1] = (float)sin((double)theta);
        }
        for (uint32_t l = 0; l < p.n_layer; ++l) {
            const DLayer& L = p.layers[l];
            // --- attention block
            norm_quant(c, l ? p.ffn : nullptr, l ? p.layers[l - 1].post_ffw_norm_w : nullptr, L.attn_norm_w, xres, xs, E,
                       p.eps, x);
            cbar();
            ZQ_STAMP();
            gemv_phase(c, p, L.qkv, &unit_base, x, terms_all, EP_STORE, p.qkv, nullptr);
            ZQ_STAMP();
            if (!grid_barrier(c, p, counter)) return;
            ZQ_STAMP();
            const uint32_t end = pos + 1;
            const uint32_t kv_len = (L.window && end > L.window) ? L.window : end;
            const uint32_t kv_start = end - kv_len;
            scores_phase(c, p, L, pos, kv_start, kv_len, rope, reinterpret_cast<float*>(scratch));
            ZQ_STAMP();
            if (!grid_barrier(c, p, counter)) return;
            ZQ_STAMP();
            softmax_v_phase(c, p, L, kv_start, kv_len, scratch);
            ZQ_STAMP();
            if (!grid_barrier(c, p, counter)) return;
            ZQ_STAMP();
            quantise_global(c, p.att, p.n_head * D, x);
            cbar();
            ZQ_STAMP();
            gemv_phase(c, p, L.o, &unit_base, x, terms_all, EP_STORE, p.proj, nullptr);
            ZQ_STAMP();
            if (!grid_barrier(c, p, counter)) return;
            ZQ_STAMP();
            // --- FFN block
            norm_quant(c, p.proj, L.post_attn_norm_w, L.ffn_norm_w, xres, xs, E, p.eps, x);
            cbar();
            ZQ_STAMP();
            gemv_phase(c, p, L.gate_up, &unit_base, x, terms_all, EP_GEGLU, p.g, nullptr);
            ZQ_STAMP();
            if (!grid_barrier(c, p, counter)) return;
            ZQ_STAMP();
            quantise_global(c, p.g, p.F, x);
            cbar();
            ZQ_STAMP();
            gemv_phase(c, p, L.down, &unit_base, x, terms_all, EP_STORE, p.ffn, nullptr);
            ZQ_STAMP();
            if (!grid_barrier(c, p, counter)) return;
            ZQ_STAMP();
        }
        if (want_logits) {
            norm_quant(c, p.ffn, p.layers[p.n_layer - 1].post_ffw_norm_w, p.output_norm_w, xres, xs, E, p.eps, x);
            cbar();
            ZQ_STAMP();
            Best best{-INFINITY, 0xFFFFFFFFu};
            gemv_phase(c, p, p.head, &unit_base, x, terms_all, EP_LOGITS, p.logits, variant == DECODE_GREEDY ? &best : nullptr);
            ZQ_STAMP();
            if (variant == DECODE_GREEDY) {
                // first maximum wins (gpt2.zig:980-990): lanes, warps, CTAs, always preferring the lower index
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    Best o;
                    o.v = __shfl_xor_sync(0xFFFFFFFFu, best.v, off);
                    o.i = __shfl_xor_sync(0xFFFFFFFFu, best.i, off);
                    best_update(best, o.v, o.i);
                }
                if (c.lane == 0) {
                    s_bval[c.warp] = best.v;
                    s_bidx[c.warp] = best.i;
                }
                cbar();
                if (c.tid == 0) {
                    Best b{s_bval[0], s_bidx[0]};
                    for (int wv = 1; wv < kConsumerWarps; ++wv) best_update(b, s_bval[wv], s_bidx[wv]);
                    p.part_val[blockIdx.x] = b.v;
                    p.part_idx[blockIdx.x] = b.i;
                }
                if (!grid_barrier(c, p, counter)) return;
                Best b{-INFINITY, 0xFFFFFFFFu};
                for (uint32_t k = c.lane; k < gridDim.x; k += 32) best_update(b, __ldcg(p.part_val + k), __ldcg(p.part_idx + k));
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    Best o;
                    o.v = __shfl_xor_sync(0xFFFFFFFFu, b.v, off);
                    o.i = __shfl_xor_sync(0xFFFFFFFFu, b.i, off);
                    best_update(b, o.v, o.i);
                }
                tok = b.i;
                if (blockIdx.x == 0 && c.tid == 0) p.record[rec] = tok;
                rec += 1;
            }
        }
        pos += 1;
    }
#undef ZQ_STAMP
    if (blockIdx.x == 0 && c.tid == 0) {
        p.state[0] = tok;
        p.state[1] = pos;
        p.state[2] = rec;
    }
}

// ---- host side --------------------------------------------------------------------------------

bool describe(DMat* d, const zq_weight* w, uint32_t slot_bytes, bool split) {
    d->qs = w->qs;
    d->sc = static_cast<const uint8_t*>(w->sc);
    d->type = (uint32_t)w->type;
    d->n_rows = w->out_dim;
    d->nb = w->nb;
    d->nbp = w->nbp;
    d->row_q_bytes = w->nbp * w->qb;
    d->row_s_bytes = w->scp * (w->type == ZQ_TYPE_Q4_1 ? 4u : 2u);
    uint32_t r = slot_bytes / (d->row_q_bytes + d->row_s_bytes);
    if (r > 8) r = 8;
    d->split = split ? 1u : 0u;
    if (split) {
        r &= ~1u;
        if (r < 2 || (w->out_dim & 1u)) return false;
        const uint32_t half = r / 2, n_half = w->out_dim / 2;
        d->n_units = (n_half + half - 1) / half;
    } else {
        if (r < 1) return false;
        d->n_units = (w->out_dim + r - 1) / r;
    }
    d->rows_per_unit = r;
    return true;
}

}  // namespace

struct GemmaDecoder {
    DParams p;
    DLayer* d_layers = nullptr;
    void* d_misc = nullptr;  // sync words, argmax partials
    size_t smem = 0;
    uint32_t grid = 0;
    uint32_t launches = 0;
    long long* d_prof = nullptr;
    ~GemmaDecoder() {
        cudaFree(d_layers);
        cudaFree(d_misc);
        cudaFree(d_prof);
    }
};

void gemma_decoder_free(GemmaDecoder* d) { delete d; }
uint32_t gemma_decoder_grid(const GemmaDecoder* d) { return d->grid; }

int gemma_decoder_create(const GemmaDecoderDesc& desc, GemmaDecoder** out) {
    *out = nullptr;
    const uint32_t E = desc.embed, D = desc.head_dim, nh = desc.n_head, nkv = desc.n_kv, F = desc.ffn;
    if (nkv == 0 || nh % nkv) return ZQ_ERR_UNSUPPORTED;
    const uint32_t group = nh / nkv;
    if (group > (uint32_t)kConsumerWarps || (kConsumerWarps % group) || nh + nkv > 32 || D % 16 || E % 32 || F % 32)
        return ZQ_ERR_UNSUPPORTED;
    int dev = 0, max_smem = 0, coop = 0;
    ZQ_CUDA(cudaGetDevice(&dev));
    ZQ_CUDA(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    ZQ_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) return ZQ_ERR_UNSUPPORTED;

    // slot size: the largest single row (quants + scales) any matrix has, at least 4 KB
    uint32_t max_row = 0, nbp_max = 0;
    auto row_bytes = [&](const zq_weight* w) {
        const uint32_t b = w->nbp * w->qb + w->scp * (w->type == ZQ_TYPE_Q4_1 ? 4u : 2u);
        if (b > max_row) max_row = b;
        if (w->nbp > nbp_max) nbp_max = w->nbp;
    };
    row_bytes(desc.token_embd);
    for (const GemmaDecoderLayer& L : desc.layers) {
        row_bytes(L.qkv);
        row_bytes(L.o);
        row_bytes(L.gate_up);
        row_bytes(L.down);
    }
    uint32_t slot_bytes = desc.slot_bytes ? desc.slot_bytes : (max_row < 7680u ? 7680u : max_row);
    slot_bytes = (slot_bytes + 255u) & ~255u;
    if (slot_bytes < max_row) return ZQ_ERR_UNSUPPORTED;

    GemmaDecoder* d = new (std::nothrow) GemmaDecoder;
    if (!d) return ZQ_ERR_NO_MEM;
    DParams& p = d->p;
    memset(&p, 0, sizeof(p));
    std::vector<DLayer> layers(desc.layers.size());
    bool ok = describe(&p.head, desc.token_embd, slot_bytes, false);
    uint32_t terms = 0;
    auto note_terms = [&](const DMat& m) {
        const uint32_t t = m.rows_per_unit * (m.nbp + 1);
        if (t > terms) terms = t;
    };
    note_terms(p.head);
    for (size_t l = 0; ok && l < layers.size(); ++l) {
        const GemmaDecoderLayer& s = desc.layers[l];
        DLayer& L = layers[l];
        ok = describe(&L.qkv, s.qkv, slot_bytes, false) && describe(&L.o, s.o, slot_bytes, false) &&
             describe(&L.gate_up, s.gate_up, slot_bytes, true) && describe(&L.down, s.down, slot_bytes, false);
        note_terms(L.qkv);
        note_terms(L.o);
        note_terms(L.gate_up);
        note_terms(L.down);
        L.attn_norm_w = s.attn_norm_w;
        L.post_attn_norm_w = s.post_attn_norm_w;
        L.q_norm_w = s.q_norm_w;
        L.k_norm_w = s.k_norm_w;
        L.ffn_norm_w = s.ffn_norm_w;
        L.post_ffw_norm_w = s.post_ffw_norm_w;
        L.kc = s.kc;
        L.vc = s.vc;
        L.window = s.window;
    }
    if (!ok) {
        delete d;
        return ZQ_ERR_UNSUPPORTED;
    }
    p.output_norm_w = desc.output_norm_w;
    p.freqs = desc.freqs;
    p.qkv = desc.qkv;
    p.scores = desc.scores;
    p.att = desc.att;
    p.proj = desc.proj;
    p.g = desc.g;
    p.ffn = desc.ffn_out;
    p.logits = desc.logits;
    p.state = desc.state;
    p.record = desc.record;
    p.n_layer = (uint32_t)layers.size();
    p.E = E;
    p.D = D;
    p.n_head = nh;
    p.n_kv = nkv;
    p.F = F;
    p.ctx = desc.ctx;
    p.max_len = desc.ctx;
    p.eps = desc.eps;
    p.embed_scale = desc.embed_scale;
    p.nbp_max = nbp_max;
    p.terms_per_warp = (terms + 3u) & ~3u;

    // shared-memory carve-up
    auto up = [](size_t v, size_t a) { return (v + a - 1) / a * a; };
    const size_t gemv_scratch = (size_t)nbp_max * (32 + 8) + (size_t)kConsumerWarps * p.terms_per_warp * 4;
    const size_t att_a = (size_t)(nh + nkv) * D * 4;
    const size_t att_b = (size_t)group * desc.ctx * 4 + 2 * (size_t)kVTile * 32;
    size_t scratch = gemv_scratch > att_a ? gemv_scratch : att_a;
    if (att_b > scratch) scratch = att_b;
    size_t off = 0;
    p.off_xres = (uint32_t)off;
    off = up(off + (size_t)E * 4, 128);
    p.off_xs = (uint32_t)off;
    off = up(off + (size_t)E * 4, 128);
    p.off_rope = (uint32_t)off;
    off = up(off + (size_t)D * 4, 128);
    p.off_scratch = (uint32_t)off;
    off = up(off + scratch, 128);
    p.off_ring = (uint32_t)off;
    const size_t budget = (size_t)max_smem - 2048;  // static shared memory of the kernel
    if (off + 16 * (size_t)slot_bytes > budget) {
        delete d;
        return ZQ_ERR_UNSUPPORTED;
    }
    uint32_t n_slots = (uint32_t)((budget - off) / slot_bytes);
    if (n_slots > 64) n_slots = 64;
    if (desc.n_slots && desc.n_slots >= 16 && desc.n_slots <= n_slots) n_slots = desc.n_slots;
    p.n_slots = n_slots;
    p.slot_bytes = slot_bytes;
    d->smem = off + (size_t)n_slots * slot_bytes;

    d->grid = (uint32_t)sm_count();
    cudaError_t e = cudaFuncSetAttribute(gemma3_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d->smem);
    int per_sm = 0;
    if (e == cudaSuccess)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemma3_decode_kernel, kThreads, d->smem);
    if (e != cudaSuccess || per_sm < 1) {
        delete d;
        if (e != cudaSuccess) return cuda_fail(e);
        return ZQ_ERR_UNSUPPORTED;
    }
    const size_t misc = 64 + (size_t)d->grid * 8;
    if (cudaMalloc(&d->d_layers, layers.size() * sizeof(DLayer)) != cudaSuccess ||
        cudaMalloc(&d->d_misc, misc) != cudaSuccess) {
        delete d;
        return ZQ_ERR_NO_MEM;
    }
    e = cudaMemcpy(d->d_layers, layers.data(), layers.size() * sizeof(DLayer), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemset(d->d_misc, 0, misc);
    if (e != cudaSuccess) {
        delete d;
        return cuda_fail(e);
    }
    p.layers = d->d_layers;
    p.sync = static_cast<uint32_t*>(d->d_misc);
    p.part_val = reinterpret_cast<float*>(static_cast<unsigned char*>(d->d_misc) + 64);
    p.part_idx = reinterpret_cast<uint32_t*>(p.part_val + d->grid);
    int rc = device_error_word(&p.err);
    if (rc != ZQ_OK) {
        delete d;
        return rc;
    }
    *out = d;
    return ZQ_OK;
}

int gemma_decoder_run(GemmaDecoder* d, uint32_t n_steps, int variant, cudaStream_t st) {
    if (n_steps == 0) return ZQ_OK;
    // ids 1, 2, 3, ...: the low bit picks the barrier counter, the value marks this launch's abort word
    uint32_t launch_id = d->launches + 1u;
    if (launch_id == 0u) launch_id = 2u;
    void* args[] = {&d->p, &n_steps, &variant, &launch_id};
    ZQ_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(gemma3_decode_kernel), dim3(d->grid), dim3(kThreads),
                                        args, d->smem, st));
    d->launches = launch_id;
    return ZQ_OK;
}

// One step with cycle stamps: per CTA, thread 0's clock64() at every phase boundary, in program order:
// token start; per layer 16 stamps (qkv prologue done, qkv done, barrier passed, scores done, barrier,
// softmax.V done, barrier, o prologue done, o done, barrier, ffn prologue done, gate/up done, barrier, down
// prologue done, down done, barrier); then head prologue done, head done. h_out[cta][cap].
int gemma_decoder_profile(GemmaDecoder* d, int variant, cudaStream_t st, long long* h_out, uint32_t cap,
                          uint32_t* n_ctas) {
    if (!h_out || cap == 0) return ZQ_ERR_BAD_ARG;
    const size_t bytes = (size_t)d->grid * cap * sizeof(long long);
    cudaFree(d->d_prof);
    d->d_prof = nullptr;
    if (cudaMalloc(&d->d_prof, bytes) != cudaSuccess) return ZQ_ERR_NO_MEM;
    ZQ_CUDA(cudaMemsetAsync(d->d_prof, 0, bytes, st));
    d->p.prof = d->d_prof;
    d->p.prof_cap = cap;
    int rc = gemma_decoder_run(d, 1, variant, st);
    d->p.prof = nullptr;
    if (rc != ZQ_OK) return rc;
    ZQ_CUDA(cudaMemcpyAsync(h_out, d->d_prof, bytes, cudaMemcpyDeviceToHost, st));
    ZQ_CUDA(cudaStreamSynchronize(st));
    if (n_ctas) *n_ctas = d->grid;
    return ZQ_OK;
}

}  // namespace zq
