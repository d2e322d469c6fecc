// One persistent cooperative kernel per Gemma-3 decode step (or per run of greedy steps): the whole
// token — embedding, 26 x (norm, qkv, attention, o, norm, gate/up, GeGLU, down), final norm, logits,
// argmax — runs as phases of ONE grid of one CTA per SM instead of about 270 dependent kernel launches
// (gemma3.zig:662-846; the one-encoder form of gemma3_metal.zig:189-260).
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
//     of the consumers across phase and token boundaries: HBM keeps streaming while the consumers wait
//     for an exchange, run a norm or the attention's serial chains.
//   * Small vectors (the residual stream, norms, the quantised activation image) are recomputed by every
//     CTA in its own shared memory rather than exchanged.
//   * Vectors that cross CTAs (qkv, scores, attention output, projections) are exchanged through global
//     memory as 64-bit words {value, epoch}: the consumer's load of a word is at the same time the test
//     whether its producer has written it, so an exchange costs one store and one load round trip and no
//     grid-wide barrier exists. Each exchange of a run has its own epoch number; buffers alternate with
//     the layer's parity and every CTA signs a per-layer presence word, so a buffer is rewritten only after
//     every CTA has finished the layer that read it.
//
// Every wait is bounded: a poll or slot wait that runs out records a code in the device error word,
// raises the abort flag (tagged with the launch), and every CTA drains its copies in flight and returns.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <new>
#include <vector>

#include "decode_gemma.h"
#include "decode_common.cuh"
#include "zq_internal.h"

namespace zq {
namespace {

using namespace dk;
constexpr uint32_t kVTile = 256;   // positions per V tile of the attention phase

enum { EP_VECTOR = 0, EP_GEGLU = 1, EP_LOGITS = 2 };

// A quantised matrix as the kernel walks it. Rows are taken in tiles of `rows_per_tile` (at most 8: one
// weight row per lane group of an int8 tensor-core tile); a tile whose rows do not fit a ring slot is cut
// along K into `chunks` pieces of `chunk_quads` quads (4 blocks each). One unit = one piece of one tile.
struct DMat {
    const uint8_t* qs;
    const uint8_t* sc;
    uint32_t type, n_rows, nb, nbp;
    uint32_t row_q_bytes, row_s_bytes;
    uint32_t rows_per_tile, n_tiles;
    uint32_t split;       // 1: a tile holds rows_per_tile/2 rows of the first half and the matching rows of the second
    uint32_t chunks;      // pieces per tile along K (1: whole rows, one bulk copy of quants and one of scales)
    uint32_t chunk_quads; // quads per piece (the last piece of a row may be shorter); at most 16
    uint32_t tiles_div, tiles_rem;  // n_tiles / grid and n_tiles % grid: CTA c owns tiles_div + (c < tiles_rem) tiles
    uint32_t chunk_q_pitch;         // bytes between the rows of a piece in a ring slot (chunks > 1)
    uint32_t chunks_magic;          // floor(2^32 / chunks) for fast_divmod
    uint32_t pad_;
};

struct alignas(16) DLayer {
    DMat qkv, o, gate_up, down;
    const float *attn_norm_w, *post_attn_norm_w, *q_norm_w, *k_norm_w, *ffn_norm_w, *post_ffw_norm_w;
    float *kc, *vc;
    uint32_t window;  // 0: every position (global layer)
};

// Exchange buffers, two of each (layer parity). A word is (epoch << 32) | float bits.
struct Exchange {
    unsigned long long *qkv, *scores, *att, *proj, *g, *ffn, *best;
    uint32_t qkv_n, scores_n, att_n, proj_n, g_n, ffn_n, best_n;  // words per parity
};

struct DParams {
    const DLayer* layers;
    DMat head;  // token_embd: embedding rows and the tied logits head
    const float* output_norm_w;
    const float* freqs;
    float* logits;
    uint32_t* state;   // [0] token, [1] position, [2] next slot of the greedy record
    uint32_t* record;
    uint32_t* abort_word;  // holds the id of a launch that gave up
    unsigned int* err;
    long long* prof;   // optional: per-CTA cycle stamps of one step (prof_cap per CTA); nullptr = off
    Exchange ex;
    uint32_t prof_cap;
    uint32_t n_layer, E, D, n_head, n_kv, F, ctx, max_len;
    float eps, embed_scale;
    // shared-memory carve-up (bytes from the start of dynamic shared memory)
    uint32_t n_slots, slot_magic, slot_bytes, off_ring, off_layers, off_xres, off_xs, off_rope, off_vnew, off_scratch;
    uint32_t terms_per_warp, nbp_max;
    uint32_t terms_bytes;  // bytes behind the activation image: block terms, staging of the prologues
    uint32_t deal_limit;   // a phase with at most this many units per CTA shares every unit among all warps
    uint32_t xh_off;       // second half of the activation image, in 16-byte words from the first
    uint32_t group, half_d;  // query heads per kv head; D / 2
    uint32_t magic_chunks, magic_group, magic_half, magic_nh;  // floor(2^32 / x) for fast_divmod: D / 8, group, D / 2, n_head
};

// Head of the dynamic shared memory: the launch parameters (copied once, so that device functions read them
// with shared-memory loads instead of through the parameter space), the ring's barriers and small exchange cells.
struct Shared {
    DParams p;
    unsigned long long full[64];
    unsigned long long empty[64];
    uint32_t released[64];  // per ring slot: uses consumed so far
    int abort;
    uint32_t launch_id;     // the abort word holds the id of the launch that gave up
    float part[16];         // 16 lane sums
    float bc;               // broadcast cell
    float red[32];          // per-warp partials
    float bval[kConsumerWarps];
    uint32_t bidx[kConsumerWarps];
};
constexpr uint32_t kSharedHead = (sizeof(Shared) + 127u) & ~127u;

__device__ __forceinline__ unsigned char* smem_base() {
    extern __shared__ __align__(128) unsigned char zq_decode_smem[];
    return zq_decode_smem;
}
__device__ __forceinline__ Shared& sh() { return *reinterpret_cast<Shared*>(smem_base()); }

// Per-thread view of the CTA's shared state; built (a few address computations) at the top of every device
// function rather than passed by reference, which would put it into local memory.
struct Cta {
    unsigned char* smem;
    uint32_t smem32;
    uint32_t full0, empty0;  // shared addresses of the mbarrier arrays
    volatile int* s_abort;
    float* part;
    float* bc;
    float* red;
    volatile uint32_t* released;
    int tid, lane, warp;
    uint32_t launch_id;
};
__device__ __forceinline__ Cta make_cta() {
    Shared& S = sh();
    Cta c;
    c.smem = smem_base();
    c.smem32 = (uint32_t)__cvta_generic_to_shared(c.smem);
    c.full0 = (uint32_t)__cvta_generic_to_shared(S.full);
    c.empty0 = (uint32_t)__cvta_generic_to_shared(S.empty);
    c.s_abort = &S.abort;
    c.part = S.part;
    c.bc = &S.bc;
    c.red = S.red;
    c.released = S.released;
    c.tid = threadIdx.x;
    c.lane = threadIdx.x & 31;
    c.warp = threadIdx.x >> 5;
    c.launch_id = S.launch_id;
    return c;
}

__device__ __forceinline__ void raise_abort(const Cta& c, const DParams& p, unsigned int code) {
    *c.s_abort = 1;
    if (ld_relaxed_gpu_u32(p.abort_word) != c.launch_id) atomicExch(p.err, code);
    atomicExch(p.abort_word, c.launch_id);
}

// Up to N words of an exchange buffer per thread — words first, first + stride, ... (valid below n) — with all
// loads in flight at once; words whose producer has not written yet are polled again, a bounded number of times.
template <int N>
__device__ __forceinline__ void xload_batch(const Cta& c, const DParams& p, const unsigned long long* buf,
                                            uint32_t first, uint32_t stride, uint32_t n, uint32_t epoch, float (&out)[N]) {
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
        if (missing) raise_abort(c, p, kErrExchange);
    }
#pragma unroll
    for (int u = 0; u < N; ++u) out[u] = __uint_as_float((uint32_t)w[u]);
}

// Bounded wait for a ring slot. On a timeout the abort flag is raised; the caller skips its work and the
// CTA leaves at its next uniform check.
__device__ __forceinline__ bool slot_wait(const Cta& c, const DParams& p, uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    // Not there yet: wait without flooding the shared-memory pipeline that the working warps' loads, shuffles
    // and barrier operations go through. About a second in all.
    for (uint32_t i = 0; i < (1u << 19); ++i) {
        if (mbar_try_wait_hint(bar, parity, 2000u)) return true;
        if ((i & 15u) == 15u && *c.s_abort) return false;
    }
    raise_abort(c, p, kErrUnitWait);
    return false;
}

// Sum of squares in the CPU loop's order (gemma3.zig:920-930): 16 lane accumulators, lanes added 0..15,
// then the tail. `xs` complete before the call (a cbar lies between its writes and this call).
__device__ __forceinline__ float sumsq_lanes16(const Cta& c, const float* xs, uint32_t dim) {
    const uint32_t dim16 = dim & ~15u;
    if (c.warp == kChainWarp) {
        float acc = 0.0f;
        uint32_t i = c.lane;
        if (c.lane < 16) {
            if (i + 16 * 7 < dim16) {  // loads and squares of the next eight elements run under the adds of these
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = xs[i + 16 * u];
                i += 16 * 8;
#pragma unroll 1
                for (; i + 16 * 7 < dim16; i += 16 * 8) {
                    float n[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) n[u] = xs[i + 16 * u];
#pragma unroll
                    for (int u = 0; u < 8; ++u) acc = __fadd_rn(acc, __fmul_rn(v[u], v[u]));
#pragma unroll
                    for (int u = 0; u < 8; ++u) v[u] = n[u];
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) acc = __fadd_rn(acc, __fmul_rn(v[u], v[u]));
            }
#pragma unroll 1
            for (; i < dim16; i += 16) acc = __fadd_rn(acc, __fmul_rn(xs[i], xs[i]));
        }
        // the 16 lane sums in lane order (every lane of the warp forms the same total), then the tail
        float ss = __shfl_sync(0xFFFFFFFFu, acc, 0);
#pragma unroll
        for (int l = 1; l < 16; ++l) ss = __fadd_rn(ss, __shfl_sync(0xFFFFFFFFu, acc, l));
        if (c.lane == 0) {
#pragma unroll 1
            for (uint32_t k = dim16; k < dim; ++k) ss = __fadd_rn(ss, __fmul_rn(xs[k], xs[k]));
            *c.bc = ss;
        }
    }
    cbar();
    return *c.bc;
}
// Squares added one by one (rms_norm_in_place, gemma3.zig:949-959); the next eight loads run under the adds.
__device__ __forceinline__ float sumsq_sequential(const float* xs, uint32_t dim) {
    float ss = 0.0f;
    uint32_t i = 0;
    if (dim >= 8) {
        float4 a = *reinterpret_cast<const float4*>(xs), b = *reinterpret_cast<const float4*>(xs + 4);
#pragma unroll 1
        for (i = 8; i + 8 <= dim; i += 8) {
            const float4 na = *reinterpret_cast<const float4*>(xs + i), nb = *reinterpret_cast<const float4*>(xs + i + 4);
            ss = __fadd_rn(ss, __fmul_rn(a.x, a.x)); ss = __fadd_rn(ss, __fmul_rn(a.y, a.y));
            ss = __fadd_rn(ss, __fmul_rn(a.z, a.z)); ss = __fadd_rn(ss, __fmul_rn(a.w, a.w));
            ss = __fadd_rn(ss, __fmul_rn(b.x, b.x)); ss = __fadd_rn(ss, __fmul_rn(b.y, b.y));
            ss = __fadd_rn(ss, __fmul_rn(b.z, b.z)); ss = __fadd_rn(ss, __fmul_rn(b.w, b.w));
            a = na;
            b = nb;
        }
        ss = __fadd_rn(ss, __fmul_rn(a.x, a.x)); ss = __fadd_rn(ss, __fmul_rn(a.y, a.y));
        ss = __fadd_rn(ss, __fmul_rn(a.z, a.z)); ss = __fadd_rn(ss, __fmul_rn(a.w, a.w));
        ss = __fadd_rn(ss, __fmul_rn(b.x, b.x)); ss = __fadd_rn(ss, __fmul_rn(b.y, b.y));
        ss = __fadd_rn(ss, __fmul_rn(b.z, b.z)); ss = __fadd_rn(ss, __fmul_rn(b.w, b.w));
    }
#pragma unroll 1
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
// The second half starts an odd multiple of 64 bytes behind the first (xh_off): lane groups that read the
// halves in opposite order (unit_terms) then touch different banks.
__device__ __forceinline__ XImage ximage(unsigned char* scratch, uint32_t nbp_max) {
    XImage x;
    x.xl = reinterpret_cast<uint4*>(scratch);
    x.xh = x.xl + sh().p.xh_off;
    x.xsc = reinterpret_cast<float*>(x.xl + 2 * nbp_max + 8);
    x.xsum = reinterpret_cast<int32_t*>(x.xsc + nbp_max);
    return x;
}

// quantize_row_q8 (simd_dot.zig:25-64) of the 32 values held one per lane, written into the image.
__device__ __forceinline__ void quant_block_to_image(float v, uint32_t b, int lane, const XImage& x) {
    // |v| as an unsigned integer orders like the float: one warp-wide integer maximum gives max(abs(v))
    const float amax = __uint_as_float(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(fabsf(v))));
    const float s = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, s);
    float r = roundf(__fmul_rn(v, inv));
    r = fminf(127.0f, fmaxf(-127.0f, r));
    const int qi = (int)r;
    const int acc = __reduce_add_sync(0xFFFFFFFFu, qi);
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
#pragma unroll 1
    for (uint32_t i = nb * 8 + c.tid; i < nbp * 8; i += kConsumers) {
        const uint32_t b = i >> 3, w = i & 7u;
        uint32_t* dst = reinterpret_cast<uint32_t*>(w < 4 ? x.xl : x.xh);
        dst[((b >> 2) * 4 + (w & 3u)) * 4 + (b & 3u)] = 0u;
    }
#pragma unroll 1
    for (uint32_t b = nb + c.tid; b < nbp; b += kConsumers) {
        x.xsc[b] = 1.0f;
        x.xsum[b] = 0;
    }
}

// An exchanged f32 vector (dim % 32 == 0), quantised into the image. 16 words per thread and pass, all in
// flight at once: one round trip for up to 8192 elements. The values are parked in `stage` (16 * 512 floats,
// each thread reads back only what it wrote) so that the quantiser exists once, in a rolled loop: the kernel
// runs every phase once per layer, and code size, not arithmetic, is what instruction fetch pays for.
__device__ __noinline__ void quantise_exchanged(const unsigned long long* buf,
                                                uint32_t dim, uint32_t epoch, float* stage) {
    const Cta c = make_cta();
    const DParams& p = sh().p;
    const XImage x = ximage(c.smem + p.off_scratch, p.nbp_max);
    for (uint32_t base = 0; base < dim; base += kConsumers * 16) {
        {
            float v[16];
            xload_batch<16>(c, p, buf, base + c.tid, kConsumers, dim, epoch, v);
#pragma unroll
            for (int u = 0; u < 16; ++u) stage[u * kConsumers + c.tid] = v[u];
        }
#pragma unroll 1
        for (uint32_t u = 0; u < 16; ++u) {
            const uint32_t i = base + u * kConsumers + c.tid;
            if (i - c.lane >= dim) break;  // whole warps
            quant_block_to_image(stage[u * kConsumers + c.tid], i >> 5, c.lane, x);
        }
    }
    image_padding(c, x, dim >> 5, (dim / 32 + 3u) & ~3u);
}

// xres (+)= rms_norm(src, w1) when src != nullptr; then h = rms_norm(xres, w2) quantised into the image
// (gemma3.zig:662-666, 725-737, 768-773 followed by the row quantiser of the next linear). The norm weights
// are requested (asynchronous copies into `wstage`, 2 * dim floats) together with the exchanged vector, so the
// prologue pays one memory round trip.
__device__ __noinline__ void norm_quant(const unsigned long long* src, uint32_t epoch,
                                        const float* w1, const float* w2, float* xres, float* xs, uint32_t dim,
                                        float eps, float* wstage) {
    const Cta c = make_cta();
    const DParams& p = sh().p;
    const XImage x = ximage(c.smem + p.off_scratch, p.nbp_max);
    float* w1s = wstage;
    float* w2s = wstage + dim;
    {
        const uint32_t ws32 = c.smem32 + (uint32_t)(reinterpret_cast<unsigned char*>(wstage) - c.smem);
        for (uint32_t i = c.tid * 4; i < dim; i += kConsumers * 4) {
            if (src) cp_async16(ws32 + i * 4, w1 + i);
            cp_async16(ws32 + (dim + i) * 4, w2 + i);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (src) {
#pragma unroll 1
        for (uint32_t base = 0; base < dim; base += kConsumers * 4) {
            float v[4];
            xload_batch<4>(c, p, src, base + c.tid, kConsumers, dim, epoch, v);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint32_t i = base + u * kConsumers + c.tid;
                if (i < dim) xs[i] = v[u];
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (src) {
        cbar();
        const float ss = sumsq_lanes16(c, xs, dim);
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
#pragma unroll 1
        for (uint32_t i = c.tid; i < dim; i += kConsumers)
            xres[i] = __fadd_rn(xres[i], __fmul_rn(__fmul_rn(xs[i], inv), w1s[i]));
    }
    cbar();
    const float ss = sumsq_lanes16(c, xres, dim);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)dim), eps)));
#pragma unroll 1
    for (uint32_t i = c.tid; i < dim; i += kConsumers)
        quant_block_to_image(__fmul_rn(__fmul_rn(xres[i], inv), w2s[i]), i >> 5, c.lane, x);
    image_padding(c, x, dim >> 5, (dim / 32 + 3u) & ~3u);
}

// Block terms of one unit: up to 8 rows of weights in shared memory against the activation image, for quads
// [q_lo, q_hi) of the piece (the piece starts at quad q_first of the row). Lane (g, t) holds word t (and, for
// q8_0, word 4 + t) of the four blocks of a quad of row g: one 128-bit load each; its dp4a partial dots of the
// four blocks meet the other three lanes' in a 4 x 4 transpose-and-add (three shuffles), after which lane t
// holds the exact int32 dot of block t. (The int8 mma.sync form of the same step was measured 1.5 x slower on
// this part: 56 cycles per instruction.) The eight rows of a q8_0 unit lie a multiple of 128 bytes apart, so
// odd row groups read their two halves in the opposite order (and the activation halves with them): the row
// segments of one load then cover all 32 banks. Terms land at terms[row * pitch + 4 * (q_term + q) + t].
template <int TYPE>
__device__ __forceinline__ void unit_terms(const unsigned char* slab_q, uint32_t q_pitch, const unsigned char* slab_s,
                                           uint32_t s_pitch, uint32_t rows, uint32_t q_lo, uint32_t q_hi, uint32_t q_first,
                                           uint32_t q_term, const XImage& x, float* terms, uint32_t pitch, int lane) {
    constexpr bool Q8 = TYPE == ZQ_TYPE_Q8_0;
    constexpr bool Q41 = TYPE == ZQ_TYPE_Q4_1;
    constexpr uint32_t QUAD = Q8 ? 128 : 64;
    const int t = lane & 3;
    const uint32_t g = (uint32_t)lane >> 2;
    const uint32_t gr = g < rows ? g : 0u;  // lane groups beyond the unit's rows repeat row 0 (their terms are not read)
    const uint32_t sw = Q8 ? (g & 1u) * 64u : 0u;
    const unsigned char* wrow = slab_q + (size_t)gr * q_pitch + 16 * t;
    const unsigned char* srow = slab_s + (size_t)gr * s_pitch;
    const uint4* xa = (Q8 && (g & 1u)) ? x.xh : x.xl;
    const uint4* xb = (Q8 && (g & 1u)) ? x.xl : x.xh;
    float* trow = terms + g * pitch;
#pragma unroll 2
    for (uint32_t q = q_lo; q < q_hi; ++q) {
        const uint4 wa = *reinterpret_cast<const uint4*>(wrow + q * QUAD + sw);
        uint4 wb = wa;
        if (Q8) wb = *reinterpret_cast<const uint4*>(wrow + q * QUAD + 64 - sw);
        const uint4 x0 = xa[(q_first + q) * 4 + t], x1 = xb[(q_first + q) * 4 + t];
        int part[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (Q8) {
                part[j] = __dp4a((int)pick(wa, j), (int)pick(x0, j), __dp4a((int)pick(wb, j), (int)pick(x1, j), 0));
            } else {
                const uint32_t u = pick(wa, j);
                part[j] = __dp4a((int)(u & 0x0F0F0F0Fu), (int)pick(x0, j),
                                 __dp4a((int)((u >> 4) & 0x0F0F0F0Fu), (int)pick(x1, j), 0));
            }
        }
        int idot = quad_transpose_reduce(part, t);
        const uint32_t bl = q * 4 + t, blk = (q_first + q) * 4 + t;
        float d, m = 0.0f;
        if (Q41) {
            const __half2 h = *reinterpret_cast<const __half2*>(srow + bl * 4);
            d = __low2float(h);
            m = __high2float(h);
        } else {
            d = __half2float(*reinterpret_cast<const __half*>(srow + bl * 2));
        }
        const float s = x.xsc[blk];
        const int qsum = x.xsum[blk];
        if (TYPE == ZQ_TYPE_Q4_0) idot -= 8 * qsum;
        float term = __fmul_rn(__fmul_rn(d, s), (float)idot);
        if (Q41) term = __fadd_rn(term, __fmul_rn(__fmul_rn(m, s), (float)qsum));
        trow[(q_term + q) * 4 + t] = term;
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

// Geometry of one unit (piece `ch` of tile `tile`) as both sides of the ring compute it.
struct UnitGeom {
    uint32_t rows;      // rows in the slab (both halves of a split tile together)
    uint32_t row0;      // first row (of the first half when split)
    uint32_t q_first;   // first quad of the piece
    uint32_t nqc;       // quads in the piece
    uint32_t q_pitch;   // bytes between rows of quants in the slab
    uint32_t s_pitch;   // bytes between rows of scales in the slab
    uint32_t s_off;     // byte offset of the slab's scale rows
    uint32_t s_delta;   // bytes to skip at the start of a scale row (its source was aligned down to 16)
};
__device__ __forceinline__ UnitGeom unit_geom(const DMat& m, uint32_t tile, uint32_t ch) {
    UnitGeom u;
    const uint32_t R = m.rows_per_tile, nq = m.nbp >> 2;
    const uint32_t SB = m.type == ZQ_TYPE_Q4_1 ? 4u : 2u;
    if (m.split) {
        const uint32_t half = R >> 1, n_half = m.n_rows >> 1;
        u.row0 = tile * half;
        u.rows = 2 * min(half, n_half - u.row0);
    } else {
        u.row0 = tile * R;
        u.rows = min(R, m.n_rows - u.row0);
    }
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
        u.s_off = R * u.q_pitch;
    }
    return u;
}

__device__ __forceinline__ bool unit_acquire(const Cta& c, const DParams& p, uint32_t slot, uint32_t use) {
    // The slot's previous use must have been consumed before its barrier is read: a parity wait alone cannot
    // tell fill `use` from fill `use - 2`.
    bool ready = true;
    if (use > 0) {
        uint32_t spins = 0;
        while (c.released[slot] < use && ++spins < kSlotSpinLimit) __nanosleep(64);
        ready = c.released[slot] >= use;
        if (!ready) raise_abort(c, p, kErrUnitWait);
    }
    ready = ready && slot_wait(c, p, c.full0 + slot * 8, use & 1u);
    return __all_sync(0xFFFFFFFFu, ready);  // the whole warp decides together
}
// `count` of the 16 arrivals that free a slot: a warp that consumed a unit alone signs for all of them.
__device__ __forceinline__ void unit_release(const Cta& c, uint32_t slot, uint32_t use, uint32_t count) {
    __syncwarp();
    if (c.lane == 0) {
        c.released[slot] = use + 1;
        __threadfence_block();
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(c.empty0 + slot * 8), "r"(count) : "memory");
    }
}
template <typename... A>
__device__ __forceinline__ void unit_terms_any(uint32_t type, A... a) {
    if (type == ZQ_TYPE_Q8_0) unit_terms<ZQ_TYPE_Q8_0>(a...);
    else if (type == ZQ_TYPE_Q4_0) unit_terms<ZQ_TYPE_Q4_0>(a...);
    else unit_terms<ZQ_TYPE_Q4_1>(a...);
}
// Sum of `n` terms in order, added onto `run` (tr 16-byte aligned). A dependent add takes four cycles and a
// shared-memory load about thirty: sixteen terms are added while the next sixteen are on their way, in two
// register sets that take turns (no copies between them).
__device__ __forceinline__ float ordered_sum(float run, const float* tr, uint32_t n) {
    const float4* t4 = reinterpret_cast<const float4*>(tr);
    uint32_t b = 0;
#define ZQ_ADD4(v)                  \
    run = __fadd_rn(run, (v).x);    \
    run = __fadd_rn(run, (v).y);    \
    run = __fadd_rn(run, (v).z);    \
    run = __fadd_rn(run, (v).w)
    if (n >= 16) {
        float4 a0 = t4[0], a1 = t4[1], a2 = t4[2], a3 = t4[3];  // terms [b - 16, b): loaded, not yet added
        b = 16;
#pragma unroll 1
        while (b + 32 <= n) {
            const float4 c0 = t4[(b >> 2)], c1 = t4[(b >> 2) + 1], c2 = t4[(b >> 2) + 2], c3 = t4[(b >> 2) + 3];
            ZQ_ADD4(a0);
            ZQ_ADD4(a1);
            ZQ_ADD4(a2);
            ZQ_ADD4(a3);
            a0 = t4[(b >> 2) + 4];
            a1 = t4[(b >> 2) + 5];
            a2 = t4[(b >> 2) + 6];
            a3 = t4[(b >> 2) + 7];
            ZQ_ADD4(c0);
            ZQ_ADD4(c1);
            ZQ_ADD4(c2);
            ZQ_ADD4(c3);
            b += 32;
        }
        if (b + 16 <= n) {
            const float4 c0 = t4[(b >> 2)], c1 = t4[(b >> 2) + 1], c2 = t4[(b >> 2) + 2], c3 = t4[(b >> 2) + 3];
            ZQ_ADD4(a0);
            ZQ_ADD4(a1);
            ZQ_ADD4(a2);
            ZQ_ADD4(a3);
            a0 = c0;
            a1 = c1;
            a2 = c2;
            a3 = c3;
            b += 16;
        }
        // the tail's loads (up to three vectors) go out before the last sixteen adds
        const uint32_t rest = n - b;
        float4 r0 = make_float4(0.f, 0.f, 0.f, 0.f), r1 = r0, r2 = r0;
        if (rest >= 4) r0 = t4[(b >> 2)];
        if (rest >= 8) r1 = t4[(b >> 2) + 1];
        if (rest >= 12) r2 = t4[(b >> 2) + 2];
        ZQ_ADD4(a0);
        ZQ_ADD4(a1);
        ZQ_ADD4(a2);
        ZQ_ADD4(a3);
        if (rest >= 4) { ZQ_ADD4(r0); b += 4; }
        if (rest >= 8) { ZQ_ADD4(r1); b += 4; }
        if (rest >= 12) { ZQ_ADD4(r2); b += 4; }
    } else {
#pragma unroll 1
        for (; b + 4 <= n; b += 4) {
            const float4 a = t4[b >> 2];
            ZQ_ADD4(a);
        }
    }
#undef ZQ_ADD4
#pragma unroll 1
    for (; b < n; ++b) run = __fadd_rn(run, tr[b]);
    return run;
}

// One matrix-vector phase: this CTA's tiles of `m` (tile = cta, cta + grid, ...). The activation image is
// complete (cbar) before the call. Outputs leave as exchange words (EP_VECTOR, EP_GEGLU) or as plain f32 logits
// (EP_LOGITS). Block terms are added onto a row's sum in block order, as the CPU loop does. Two forms:
//   * few units per CTA (the layer matrices): the quads of all the CTA's units, taken as one sequence, are cut
//     into 16 equal runs, one per warp; a warp touches only the one or two units its run lies in, the terms meet
//     in a CTA-wide buffer, and after a barrier one thread per row adds them up. A unit's 16 slot-release
//     arrivals are shared out among the warps that read it: a warp whose run covers quads [lo, hi) of a unit of
//     n quads (n <= 16) arrives with f(hi) - f(lo), f(x) = x below n and 16 at n, which adds up to 16 whatever
//     the cut;
//   * many tiles (the vocabulary head): one warp per tile, pieces and sums warp-private, no barrier.
// Loop counters instead of divisions throughout: a 32-bit division costs 65-95 cycles on this part.
// Returns the advanced unit counter.
__device__ __noinline__ uint32_t gemv_phase(const DMat& m, uint32_t unit_base, int ep, unsigned long long* xout,
                                            uint32_t epoch, float* out, Best* best) {
    const Cta c = make_cta();
    const DParams& p = sh().p;
    const XImage x = ximage(c.smem + p.off_scratch, p.nbp_max);
    float* terms_all = reinterpret_cast<float*>(x.xsum + p.nbp_max);
    const uint32_t G = gridDim.x, cta = blockIdx.x;
    const uint32_t C = m.chunks;
    const uint32_t mine = m.tiles_div + (cta < m.tiles_rem ? 1u : 0u);
    const uint32_t base = unit_base;
    const uint32_t type = m.type;
    const uint32_t n_slots = p.n_slots, slot_magic = p.slot_magic;
    const uint32_t row_pitch = m.nbp + 4;  // terms of a whole row
    const uint32_t nq = m.nbp >> 2, cq = m.chunk_quads;
    if (mine * C <= p.deal_limit && mine * 8 * row_pitch * 4 <= p.terms_bytes) {
        // ---- all warps share the phase's quads
        const uint32_t total = mine * nq;
        const uint32_t run_lo = ((uint32_t)c.warp * total) >> 4, run_hi = (((uint32_t)c.warp + 1u) * total) >> 4;
        uint32_t i = 0, ch = 0, us = 0;  // tile, piece, first quad of the unit in the phase's sequence
        bool live = true;
#pragma unroll 1
        for (uint32_t n = 0; n < mine * C; ++n) {
            const uint32_t q_first = ch * cq;
            const uint32_t nqc = min(cq, nq - q_first);
            const uint32_t ue = us + nqc;
            if (run_lo < ue && run_hi > us) {
                const uint32_t lo = max(run_lo, us) - us, hi = min(run_hi, ue) - us;
                uint32_t slot, use;
                fast_divmod(base + n, n_slots, slot_magic, use, slot);
                const UnitGeom u = unit_geom(m, cta + i * G, ch);
                if (!unit_acquire(c, p, slot, use)) {
                    live = false;
                    break;
                }
                const unsigned char* slab_q = c.smem + p.off_ring + (size_t)slot * p.slot_bytes;
                unit_terms_any(type, slab_q, u.q_pitch, slab_q + u.s_off + u.s_delta, u.s_pitch, u.rows, lo, hi, q_first,
                               q_first, x, terms_all + (size_t)i * 8 * row_pitch, row_pitch, c.lane);
                unit_release(c, slot, use, (hi == nqc ? (uint32_t)kConsumerWarps : hi) - lo);
            }
            us = ue;
            if (++ch == C) {
                ch = 0;
                ++i;
            }
        }
        (void)live;
        cbar();  // every term of the phase is in the buffer
        const uint32_t nb = m.nb;
#pragma unroll 1
        for (uint32_t r = (uint32_t)(c.tid >= kChainTid ? c.tid - kChainTid : c.tid + kConsumers - kChainTid); r < mine * 8;
             r += kConsumers) {  // rows start on warp 1 (kChainWarp)
            const uint32_t ti = r >> 3, g = r & 7u;
            const UnitGeom u = unit_geom(m, cta + ti * G, 0);
            const float* tr = terms_all + (size_t)r * row_pitch;
            if (ep == EP_GEGLU) {
                const uint32_t half = u.rows >> 1;
                if (g < half) {
                    const float gate = ordered_sum(0.0f, tr, nb);
                    const float up = ordered_sum(0.0f, tr + (size_t)half * row_pitch, nb);
                    xstore(xout + u.row0 + g, __fmul_rn(gelu_tanh(gate), up), epoch);
                }
            } else if (g < u.rows) {
                const float v = ordered_sum(0.0f, tr, nb);
                if (ep == EP_LOGITS) {
                    out[u.row0 + g] = v;
                    if (best) best_update(*best, v, u.row0 + g);
                } else {
                    xstore(xout + u.row0 + g, v, epoch);
                }
            }
        }
        return base + mine * C;
    }
    // ---- one warp per tile
    const uint32_t pitch = cq * 4 + 4;
    float* terms = terms_all + (size_t)c.warp * p.terms_per_warp;
    bool live = true;
#pragma unroll 1
    for (uint32_t i = c.warp; live && i < mine; i += kConsumerWarps) {
        const uint32_t tile = cta + i * G;
        float run = 0.0f;
        uint32_t rows = 0, row0 = 0;
#pragma unroll 1
        for (uint32_t ch = 0; ch < C; ++ch) {
            uint32_t slot, use;
            fast_divmod(base + i * C + ch, n_slots, slot_magic, use, slot);
            const UnitGeom u = unit_geom(m, tile, ch);
            rows = u.rows;
            row0 = u.row0;
            if (!unit_acquire(c, p, slot, use)) {
                live = false;
                break;
            }
            const unsigned char* slab_q = c.smem + p.off_ring + (size_t)slot * p.slot_bytes;
            unit_terms_any(type, slab_q, u.q_pitch, slab_q + u.s_off + u.s_delta, u.s_pitch, rows, 0u, u.nqc, u.q_first, 0u, x,
                           terms, pitch, c.lane);
            unit_release(c, slot, use, (uint32_t)kConsumerWarps);
            if ((uint32_t)c.lane < rows)
                run = ordered_sum(run, terms + c.lane * pitch, min(u.nqc * 4, m.nb - u.q_first * 4));
            __syncwarp();  // the terms are rewritten by the next piece
        }
        if (!live) break;
        if (ep == EP_GEGLU) {
            const uint32_t half = rows >> 1;
            const float up = __shfl_down_sync(0xFFFFFFFFu, run, half);
            if ((uint32_t)c.lane < half) xstore(xout + row0 + c.lane, __fmul_rn(gelu_tanh(run), up), epoch);
        } else if ((uint32_t)c.lane < rows) {
            if (ep == EP_LOGITS) {
                out[row0 + c.lane] = run;
                if (best) best_update(*best, run, row0 + c.lane);
            } else {
                xstore(xout + row0 + c.lane, run, epoch);
            }
        }
    }
    return base + mine * C;
}

// The producer's side of gemv_phase: issue this CTA's units of `m` into the ring. The whole producer warp calls
// it: lane j takes units j, j + L, ... of the phase (L = min(32, ring slots): the units of one pass lie in different
// slots, and a slot's uses follow each other in one lane). One thread doing it alone needed half a microsecond
// per unit, 110 us for the 221 units of the vocabulary head. The warp meets again at the end of a phase: a lane
// that ran ahead into the next matrix could otherwise wait on a slot whose previous use another lane has not
// issued yet, and a parity wait cannot tell those two phases apart. Returns false (to every lane) on a timeout.
__device__ __noinline__ bool produce_phase(const DMat& m, uint32_t* unit_base,
                                           uint32_t* issued) {
    const Cta c = make_cta();
    const DParams& p = sh().p;
    const uint32_t G = gridDim.x, cta = blockIdx.x;
    const uint32_t C = m.chunks;
    const uint32_t mine = m.tiles_div + (cta < m.tiles_rem ? 1u : 0u);
    const uint32_t base = *unit_base;
    *unit_base = base + mine * C;
    *issued = base + mine * C;  // (an upper bound while the phase runs; exact once it has ended)
    const uint32_t rqb = m.row_q_bytes, rsb = m.row_s_bytes, N = m.n_rows;
    const uint32_t QUAD = m.type == ZQ_TYPE_Q8_0 ? 128u : 64u, SB = m.type == ZQ_TYPE_Q4_1 ? 4u : 2u;
    const uint32_t n_slots = p.n_slots, slot_magic = p.slot_magic;
    const uint32_t lanes = n_slots < 32u ? n_slots : 32u;
    const uint8_t* qs = m.qs;
    const uint8_t* sc = m.sc;
    bool ok = true;
#pragma unroll 1
    for (uint32_t n = (uint32_t)c.lane; ok && (uint32_t)c.lane < lanes && n < mine * C; n += lanes) {
        uint32_t i, ch;
        fast_divmod(n, C, m.chunks_magic, i, ch);
        const uint32_t gi = base + n;
        uint32_t slot, use;
        fast_divmod(gi, n_slots, slot_magic, use, slot);
        const uint32_t tile = cta + i * G;
        if (use > 0 && !slot_wait(c, p, c.empty0 + slot * 8, (use - 1) & 1u)) {
            ok = false;
            break;
        }
        const uint32_t dst = c.smem32 + p.off_ring + slot * p.slot_bytes;
        const uint32_t bar = c.full0 + slot * 8;
        const UnitGeom u = unit_geom(m, tile, ch);
        if (C == 1) {
            if (m.split) {
                const uint32_t h = u.rows >> 1, n_half = N >> 1;
                const uint32_t qb = h * rqb, sb = h * rsb;
                mbar_arrive_expect_tx(bar, 2 * (qb + sb));
                bulk_copy_g2s(dst, qs + (size_t)u.row0 * rqb, qb, bar);
                bulk_copy_g2s(dst + qb, qs + (size_t)(n_half + u.row0) * rqb, qb, bar);
                bulk_copy_g2s(dst + 2 * qb, sc + (size_t)u.row0 * rsb, sb, bar);
                bulk_copy_g2s(dst + 2 * qb + sb, sc + (size_t)(n_half + u.row0) * rsb, sb, bar);
            } else {
                const uint32_t qb = u.rows * rqb, sb = u.rows * rsb;
                mbar_arrive_expect_tx(bar, qb + sb);
                bulk_copy_g2s(dst, qs + (size_t)u.row0 * rqb, qb, bar);
                bulk_copy_g2s(dst + qb, sc + (size_t)u.row0 * rsb, sb, bar);
            }
        } else {
            // a piece of a long row: one copy of quants and one of scales (from a 16-byte boundary) per row
            const uint32_t qbytes = u.nqc * QUAD;
            const uint32_t so = u.q_first * 4 * SB, sa = so & ~15u;
            const uint32_t sbytes = ((u.s_delta + u.nqc * 4 * SB + 15u) & ~15u);
            mbar_arrive_expect_tx(bar, u.rows * (qbytes + sbytes));
            const uint32_t half = u.rows >> 1;
#pragma unroll 1
            for (uint32_t r = 0; r < u.rows; ++r) {
                const size_t row = m.split ? (r < half ? u.row0 + r : (N >> 1) + u.row0 + (r - half)) : u.row0 + r;
                bulk_copy_g2s(dst + r * u.q_pitch, qs + row * rqb + (size_t)u.q_first * QUAD, qbytes, bar);
                bulk_copy_g2s(dst + u.s_off + r * u.s_pitch, sc + row * rsb + sa, sbytes, bar);
            }
        }
    }
    return __all_sync(0xFFFFFFFFu, ok);  // also where the warp meets again
}

// Embedding row of `tok`, dequantised and scaled (gemma3.zig:800-803, 855-871): q*d, then *scale.
__device__ __noinline__ void embed_row(const DMat& m, uint32_t tok, float scale, float* xres,
                                          uint32_t dim) {
    const Cta c = make_cta();
    const DParams& p = sh().p;
    (void)p;
    const unsigned char* qrow = m.qs + (size_t)tok * m.row_q_bytes;
    const unsigned char* srow = m.sc + (size_t)tok * m.row_s_bytes;
#pragma unroll 1
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

// Attention, first half (gemma3.zig:689-716, 1062-1090): every CTA takes the exchanged q|k|v row, normalises
// and rotates the query heads and this step's key heads in its own shared memory and keeps this step's value
// heads (`vnew`); the last CTA stores the key / value rows of position `pos`; the scores of the window are
// spread over the CTAs in tiles of 32 (position, head) pairs and leave as exchange words.
// Returns false (to every thread) when the CTA has to leave.
__device__ __noinline__ bool scores_phase(const DLayer& L, uint32_t pos,
                                             uint32_t kv_start, uint32_t kv_len, const float* rope, float* qn,
                                             float* vnew, const unsigned long long* qkv_in, uint32_t ep_in,
                                             unsigned long long* scores_out, uint32_t ep_out) {
    const Cta c = make_cta();
    const DParams& p = sh().p;
    (void)p;
    const uint32_t D = p.D, nh = p.n_head, nkv = p.n_kv, group = p.group, kv_dim = nkv * D;
    const uint32_t nvec = nh + nkv, nqk = nvec * D, nall = nqk + kv_dim;
    // The key rows of this CTA's first tile of (position, head) pairs are old cache rows: requested before the
    // exchange is polled, they arrive under the wait, the norms and the rotation (one round trip to L2 less).
    const uint32_t jobs = kv_len * nh, tiles = (jobs + 31) >> 5;
    const uint32_t l = c.tid & 15u, js = c.tid >> 4;
    const uint32_t dim16 = D & ~15u;
    float kpre[16];
    bool have_kpre = false;
    if (blockIdx.x < tiles && dim16 <= 256u) {
        const uint32_t job = blockIdx.x * 32 + js;
        const uint32_t jc = job < jobs ? job : jobs - 1;
        uint32_t pi, h, kvh, hrem;
        fast_divmod(jc, nh, p.magic_nh, pi, h);
        fast_divmod(h, group, p.magic_group, kvh, hrem);
        if (pi != kv_len - 1) {
            const float* kr = L.kc + (size_t)(kv_start + pi) * kv_dim + (size_t)kvh * D;
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const uint32_t d = l + 16 * u;
                kpre[u] = d < dim16 ? __ldcg(kr + d) : 0.0f;
            }
            have_kpre = true;
        }
    }
    // norm weights of the pairs this thread rotates: requested before the exchange is polled
    const uint32_t half = p.half_d, pairs = nvec * half;
    float2 nw[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const uint32_t i = c.tid + u * kConsumers;
        if (i < pairs) {
            uint32_t v, j;
            fast_divmod(i, half, p.magic_half, v, j);
            nw[u] = __ldg(reinterpret_cast<const float2*>(v < nh ? L.q_norm_w : L.k_norm_w) + j);
        } else {
            nw[u] = make_float2(0.0f, 0.0f);
        }
    }
#pragma unroll 1
    for (uint32_t base = 0; base < nall; base += kConsumers * 4) {
        float v[4];
        xload_batch<4>(c, p, qkv_in, base + c.tid, kConsumers, nall, ep_in, v);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t i = base + u * kConsumers + c.tid;
            if (i < nqk) qn[i] = v[u];
            else if (i < nall) vnew[i - nqk] = v[u];
        }
    }
    cbar();
    const bool leave = *c.s_abort != 0;  // uniform: read between two barriers that every thread passes
#pragma unroll 1
    // one chain per vector, one warp each; warps 1, 2, 3, 5, 6, 7, ... first (not on the producer's scheduler)
    for (uint32_t v = 0; v < nvec; ++v)
        if (c.lane == 0 && (uint32_t)c.warp == (v < 12 ? v + 1 + v / 3 : (v & 3u) * 4))
            c.red[v & 31u] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq_sequential(qn + v * D, D), (float)D), p.eps)));
    cbar();
    if (leave) return false;
#pragma unroll 1
    for (uint32_t i = c.tid, u = 0; i < pairs; i += kConsumers, ++u) {
        uint32_t v, j;
        fast_divmod(i, half, p.magic_half, v, j);
        float2 w;
        if (u < 2) w = u == 0 ? nw[0] : nw[1];
        else w = __ldg(reinterpret_cast<const float2*>(v < nh ? L.q_norm_w : L.k_norm_w) + j);
        float* vec = qn + v * D;
        const float inv = c.red[v & 31u];
        const float x0 = __fmul_rn(__fmul_rn(vec[2 * j], inv), w.x);
        const float x1 = __fmul_rn(__fmul_rn(vec[2 * j + 1], inv), w.y);
        const float cs = rope[2 * j], sn = rope[2 * j + 1];
        vec[2 * j] = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
        vec[2 * j + 1] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
    }
    cbar();
    if (blockIdx.x == gridDim.x - 1) {  // cache rows of this position, for the steps to come
#pragma unroll 1
        for (uint32_t i = c.tid; i < kv_dim; i += kConsumers) {
            L.kc[(size_t)pos * kv_dim + i] = qn[nh * D + i];
            L.vc[(size_t)pos * kv_dim + i] = vnew[i];
        }
    }
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)D));
#pragma unroll 1
    for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const uint32_t job = tile * 32 + js;
        const bool live = job < jobs;
        const uint32_t jc = live ? job : jobs - 1;
        uint32_t pi, h, kvh, hrem;
        fast_divmod(jc, nh, p.magic_nh, pi, h);
        fast_divmod(h, group, p.magic_group, kvh, hrem);
        const float* qh = qn + h * D;
        const bool from_smem = pi == kv_len - 1;
        const float* kr = from_smem ? qn + (nh + kvh) * D : L.kc + (size_t)(kv_start + pi) * kv_dim + (size_t)kvh * D;
        float acc = 0.0f;
#pragma unroll 1
        for (uint32_t d0 = l; d0 < dim16; d0 += 16 * 16) {
            float kv[16];
            if (have_kpre && tile == blockIdx.x) {
#pragma unroll
                for (int u = 0; u < 16; ++u) kv[u] = kpre[u];
            } else {
#pragma unroll
                for (int u = 0; u < 16; ++u) {
                    const uint32_t d = d0 + 16 * u;
                    kv[u] = d < dim16 ? (from_smem ? kr[d] : __ldcg(kr + d)) : 0.0f;
                }
            }
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const uint32_t d = d0 + 16 * u;
                if (d < dim16) acc = __fadd_rn(acc, __fmul_rn(qh[d], kv[u]));
            }
        }
        // lanes added in order 0..15 by lane 0 of the 16-lane group
        float s = __shfl_sync(0xFFFFFFFFu, acc, 0, 16);
#pragma unroll
        for (int j = 1; j < 16; ++j) s = __fadd_rn(s, __shfl_sync(0xFFFFFFFFu, acc, j, 16));
        if (l == 0 && live) {
#pragma unroll 1
            for (uint32_t d = dim16; d < D; ++d) s = __fadd_rn(s, __fmul_rn(qh[d], from_smem ? kr[d] : __ldcg(kr + d)));
            xstore(scores_out + (size_t)h * p.max_len + pi, __fmul_rn(s, scale), ep_out);
        }
    }
    return true;
}

// Attention, second half (gemma3.zig:1092-1120): a job owns 8 output dimensions of one query head. Softmax of
// the head (maximum, exp, the exponentials added one by one, times 1/sum), then out[d] += w[p] * v[p][d]
// position by position. Both are serial chains of one add (4 cycles) per position; everything else is taken
// off them: the products w[p] * v[p][d] of a tile of positions are formed by warps 1-15 (V rows straight from
// the cache, the current position's row from `vnew`) into prod[d][p], while eight threads of warp 0 add the
// previous tile's products in order. Returns false when the CTA has to leave.
__device__ __noinline__ bool softmax_v_phase(const DLayer& L, uint32_t kv_start,
                                                uint32_t kv_len, unsigned char* scratch, const float* vnew,
                                                const unsigned long long* scores_in, uint32_t ep_in,
                                                unsigned long long* att_out, uint32_t ep_out) {
    const Cta c = make_cta();
    const DParams& p = sh().p;
    const uint32_t D = p.D, nh = p.n_head, nkv = p.n_kv, kv_dim = nkv * D;
    const uint32_t chunks = D / 8, jobs = nh * chunks;
    constexpr uint32_t PITCH = kVTile + 4;                             // 4 mod 32 banks: stores and chain loads conflict-free
    float* w = reinterpret_cast<float*>(scratch);                      // [max_len]
    float* prod = w + (((size_t)p.max_len + 3u) & ~(size_t)3u);        // [2][8][PITCH]
    bool ok = true;
#pragma unroll 1
    for (uint32_t job = blockIdx.x; ok && job < jobs; job += gridDim.x) {
        uint32_t h, dc, kvh, hrem;
        fast_divmod(job, chunks, p.magic_chunks, h, dc);
        fast_divmod(h, p.group, p.magic_group, kvh, hrem);
        const float* vbase = L.vc + (size_t)kv_start * kv_dim + (size_t)kvh * D + dc * 8;
        const float* vcur = vnew + kvh * D + dc * 8;
        // products of tile `tile` by threads first, first + step, ...: (position, dimension) pairs, dimension fastest
        auto make_products = [&](uint32_t tile, uint32_t first, uint32_t step) {
            const uint32_t p0 = tile * kVTile, n = min(kVTile, kv_len - p0);
            float* dst = prod + (size_t)(tile & 1u) * 8 * PITCH;
#pragma unroll 1
            for (uint32_t i = first; i < n * 8; i += 4 * step) {
                float v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t k = i + u * step, q = p0 + (k >> 3), d = k & 7u;
                    v[u] = k < n * 8 ? (q + 1 < kv_len ? __ldcg(vbase + (size_t)q * kv_dim + d) : vcur[d]) : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t k = i + u * step, pi = k >> 3, d = k & 7u;
                    if (k < n * 8) dst[d * PITCH + pi] = __fmul_rn(w[p0 + pi], v[u]);
                }
            }
        };
        // The first tile's value rows do not depend on the scores: requested now, they arrive under the softmax.
        const uint32_t n_first = min(kVTile, kv_len);
        float vpre[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t k = (uint32_t)c.tid + u * kConsumers, q = k >> 3, d = k & 7u;
            vpre[u] = k < n_first * 8 ? (q + 1 < kv_len ? __ldcg(vbase + (size_t)q * kv_dim + d) : vcur[d]) : 0.0f;
        }
        {
            const unsigned long long* sh_ = scores_in + (size_t)h * p.max_len;
            float mx = -INFINITY;
#pragma unroll 1
            for (uint32_t base = 0; base < kv_len; base += kConsumers * 4) {
                float v[4];
                xload_batch<4>(c, p, sh_, base + c.tid, kConsumers, kv_len, ep_in, v);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t i = base + u * kConsumers + c.tid;
                    if (i < kv_len) {
                        w[i] = v[u];
                        mx = fmaxf(mx, v[u]);
                    }
                }
            }
            mx = warp_max(mx);
            if (c.lane == 0) c.red[c.warp] = mx;
            cbar();
            if (*c.s_abort) ok = false;  // uniform: read between two barriers that every thread passes
            mx = c.red[0];
#pragma unroll
            for (int k = 1; k < kConsumerWarps; ++k) mx = fmaxf(mx, c.red[k]);
            // up to two exponentials per pass, inlined: their double-precision chains overlap
#pragma unroll 1
            for (uint32_t q = c.tid; q < kv_len; q += 2 * kConsumers) {
                float e[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) e[u] = q + u * kConsumers < kv_len ? w[q + u * kConsumers] : 0.0f;
#pragma unroll
                for (int u = 0; u < 2; ++u) e[u] = (float)exp((double)__fsub_rn(e[u], mx));
#pragma unroll
                for (int u = 0; u < 2; ++u)
                    if (q + u * kConsumers < kv_len) w[q + u * kConsumers] = e[u];
            }
            cbar();
            if (c.tid == kChainTid) c.part[0] = __fdiv_rn(1.0f, ordered_sum(0.0f, w, kv_len));  // the serial sum of the head
            cbar();
            const float inv = c.part[0];
#pragma unroll 1
            for (uint32_t q = c.tid; q < kv_len; q += kConsumers) w[q] = __fmul_rn(w[q], inv);
            cbar();
        }
        const uint32_t n_tiles = (kv_len + kVTile - 1) / kVTile;
        static_assert(kVTile * 8 == 4 * kConsumers, "the first tile's products: four per thread");
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t k = (uint32_t)c.tid + u * kConsumers, pi = k >> 3, d = k & 7u;
            if (k < n_first * 8) prod[d * PITCH + pi] = __fmul_rn(w[pi], vpre[u]);
        }
        cbar();
        float acc = 0.0f;
#pragma unroll 1
        for (uint32_t tile = 0; tile < n_tiles; ++tile) {
            if ((c.warp & 3) == kChainWarp) {  // the chain has its scheduler to itself
                if (c.warp == kChainWarp && c.lane < 8) {
                    const uint32_t n = min(kVTile, kv_len - tile * kVTile);
                    acc = ordered_sum(acc, prod + (size_t)(tile & 1u) * 8 * PITCH + (size_t)c.lane * PITCH, n);
                }
            } else if (tile + 1 < n_tiles) {
                const uint32_t helper = (uint32_t)(c.warp - (c.warp >> 2) - (c.warp & 3 ? 1 : 0)) * 32u + (uint32_t)c.lane;
                make_products(tile + 1, helper, 12u * 32u);
            }
            cbar();  // the next tile's products are complete, this tile's have been added
        }
        if (c.warp == kChainWarp && c.lane < 8 && ok) xstore(att_out + (size_t)h * D + dc * 8 + c.lane, acc, ep_out);
    }
    return ok;
}

__global__ void __launch_bounds__(kThreads, 1)
gemma3_decode_kernel(const __grid_constant__ DParams p_in, uint32_t n_steps, int variant, uint32_t launch_id,
                     uint32_t epoch_base) {
    unsigned char* smem = smem_base();
    Shared& S = sh();
    {   // the launch parameters, word by word (DParams is a multiple of 4 bytes)
        const uint32_t* src = reinterpret_cast<const uint32_t*>(&p_in);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&S.p);
        for (uint32_t i = threadIdx.x; i < sizeof(DParams) / 4; i += kThreads) dst[i] = src[i];
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
    const DParams& p = S.p;
    // the layer table, once per launch: descriptors are read at every phase and must not cost a memory round trip
    DLayer* layers = reinterpret_cast<DLayer*>(smem + p_in.off_layers);
    {
        const uint4* src = reinterpret_cast<const uint4*>(p_in.layers);
        uint4* dst = reinterpret_cast<uint4*>(layers);
        for (uint32_t i = threadIdx.x; i < p_in.n_layer * (uint32_t)(sizeof(DLayer) / 16); i += kThreads) dst[i] = __ldg(src + i);
    }
    __syncthreads();
    const Cta c = make_cta();
    const bool want_logits = variant != DECODE_CACHE_ONLY;
    uint32_t unit_base = 0;

    if (c.warp == kConsumerWarps) {
        // ---------------------------------------------------------------- producer warp
        bool ok = true;
        uint32_t issued = 0;
        for (uint32_t step = 0; ok && step < n_steps; ++step) {
            for (uint32_t l = 0; ok && l < p.n_layer; ++l) {
                const DLayer& L = layers[l];
                ok = produce_phase(L.qkv, &unit_base, &issued) && produce_phase(L.o, &unit_base, &issued) &&
                     produce_phase(L.gate_up, &unit_base, &issued) &&
                     produce_phase(L.down, &unit_base, &issued);
            }
            if (ok && want_logits) ok = produce_phase(p.head, &unit_base, &issued);
        }
        if (!ok && c.lane == 0) {
            // Stopped early: copies already issued still land in this CTA's shared memory. Wait (bounded)
            // for the newest fill of every slot before the CTA may retire.
            for (uint32_t s = 0; s < p.n_slots && s < issued; ++s) {
                const uint32_t last = issued - 1 - ((issued - 1 - s) % p.n_slots);  // newest unit index in slot s
                const uint32_t use = last / p.n_slots;
                for (uint32_t i = 0; i < (1u << 16); ++i)
                    if (mbar_try_wait(c.full0 + s * 8, use & 1u)) break;
            }
        }
        __syncwarp();
        return;
    }

    // -------------------------------------------------------------------- consumer warps
    float* xres = reinterpret_cast<float*>(smem + p.off_xres);
    float* xs = reinterpret_cast<float*>(smem + p.off_xs);
    float* rope = reinterpret_cast<float*>(smem + p.off_rope);
    float* vnew = reinterpret_cast<float*>(smem + p.off_vnew);
    unsigned char* scratch = smem + p.off_scratch;
    float* terms_all = reinterpret_cast<float*>(ximage(scratch, p.nbp_max).xsum + p.nbp_max);
    const uint32_t E = p.E, D = p.D;
    const Exchange& ex = p.ex;
    uint32_t tok = __ldcg(p.state + 0), pos = __ldcg(p.state + 1), rec = __ldcg(p.state + 2);
    uint32_t epoch = epoch_base;  // the next exchange's number; every CTA counts alike
    uint32_t lc = 0;              // layers run so far in this launch: picks the buffer parity
    uint32_t n_stamp = 0;
    // cycle stamp of this CTA at a phase boundary (thread 0; profiling runs only)
#define ZQ_STAMP()                                                                              \
    do {                                                                                        \
        if (p.prof && c.tid == 0 && n_stamp < p.prof_cap) p.prof[(size_t)blockIdx.x * p.prof_cap + n_stamp++] = clock64(); \
    } while (0)
    // uniform exit: every consumer thread brings its view of the abort flag to one barrier and gets their OR
#define ZQ_CHECK_ABORT()                      \
    do {                                      \
        if (cbar_or(S.abort != 0)) return;    \
    } while (0)

    for (uint32_t step = 0; step < n_steps; ++step) {
        ZQ_STAMP();
        __threadfence();  // cache rows that the last CTA stored during earlier steps are read below
        embed_row(p.head, tok, p.embed_scale, xres, E);
        for (uint32_t j = c.tid; j < D / 2; j += kConsumers) {  // RoPE angles of this position, every layer
            const float theta = __fmul_rn((float)pos, __ldg(p.freqs + j));
            rope[2 * j] = (float)cos((double)theta);
            rope[2 * j + 1] = (float)sin((double)theta);
        }
        for (uint32_t l = 0; l < p.n_layer; ++l, ++lc) {
            const DLayer& L = layers[l];
            const uint32_t par = lc & 1u, prev = par ^ 1u;
            const uint32_t e_ffn_prev = epoch - 1;  // the previous layer's last exchange (unused for l == 0)
            const uint32_t e_qkv = epoch, e_scores = epoch + 1, e_att = epoch + 2, e_proj = epoch + 3, e_g = epoch + 4,
                           e_ffn = epoch + 5;
            epoch += 6;
            // --- attention block
            norm_quant(l ? ex.ffn + (size_t)prev * ex.ffn_n : nullptr, e_ffn_prev,
                       l ? layers[l - 1].post_ffw_norm_w : nullptr, L.attn_norm_w, xres, xs, E, p.eps, terms_all);
            if (l) {  // every CTA has finished the previous layer: its buffers of this parity may be rewritten
                for (uint32_t base = 0; base < gridDim.x; base += kConsumers) {
                    float v[1];
                    xload_batch<1>(c, p, ex.ffn + (size_t)prev * ex.ffn_n, E + base + (uint32_t)c.tid, 1u, E + gridDim.x,
                                   e_ffn_prev, v);
                }
            }
            ZQ_CHECK_ABORT();
            ZQ_STAMP();
            unit_base = gemv_phase(L.qkv, unit_base, EP_VECTOR, ex.qkv + (size_t)par * ex.qkv_n, e_qkv, nullptr, nullptr);
            ZQ_STAMP();
            cbar();  // the image region becomes attention scratch
            const uint32_t end = pos + 1;
            const uint32_t kv_len = (L.window && end > L.window) ? L.window : end;
            const uint32_t kv_start = end - kv_len;
            if (!scores_phase(L, pos, kv_start, kv_len, rope, reinterpret_cast<float*>(scratch), vnew,
                              ex.qkv + (size_t)par * ex.qkv_n, e_qkv, ex.scores + (size_t)par * ex.scores_n, e_scores))
                return;
            ZQ_STAMP();
            cbar();  // qn is overwritten by the softmax weights
            if (!softmax_v_phase(L, kv_start, kv_len, scratch, vnew, ex.scores + (size_t)par * ex.scores_n, e_scores,
                                 ex.att + (size_t)par * ex.att_n, e_att))
                return;
            ZQ_STAMP();
            cbar();
            quantise_exchanged(ex.att + (size_t)par * ex.att_n, p.n_head * D, e_att, terms_all);
            ZQ_CHECK_ABORT();
            ZQ_STAMP();
            unit_base = gemv_phase(L.o, unit_base, EP_VECTOR, ex.proj + (size_t)par * ex.proj_n, e_proj, nullptr, nullptr);
            ZQ_STAMP();
            cbar();
            // --- FFN block
            norm_quant(ex.proj + (size_t)par * ex.proj_n, e_proj, L.post_attn_norm_w, L.ffn_norm_w, xres, xs, E, p.eps, terms_all);
            ZQ_CHECK_ABORT();
            ZQ_STAMP();
            unit_base = gemv_phase(L.gate_up, unit_base, EP_GEGLU, ex.g + (size_t)par * ex.g_n, e_g, nullptr, nullptr);
            ZQ_STAMP();
            cbar();
            quantise_exchanged(ex.g + (size_t)par * ex.g_n, p.F, e_g, terms_all);
            ZQ_CHECK_ABORT();
            ZQ_STAMP();
            unit_base = gemv_phase(L.down, unit_base, EP_VECTOR, ex.ffn + (size_t)par * ex.ffn_n, e_ffn, nullptr, nullptr);
            cbar();  // every warp of this CTA is through the layer: sign the presence word
            if (c.tid == 0) xstore(ex.ffn + (size_t)par * ex.ffn_n + E + blockIdx.x, 0.0f, e_ffn);
            ZQ_STAMP();
        }
        if (want_logits) {
            const uint32_t last = (lc - 1) & 1u;
            norm_quant(ex.ffn + (size_t)last * ex.ffn_n, epoch - 1, layers[p.n_layer - 1].post_ffw_norm_w,
                       p.output_norm_w, xres, xs, E, p.eps, terms_all);
            ZQ_CHECK_ABORT();
            ZQ_STAMP();
            Best best{-INFINITY, 0xFFFFFFFFu};
            unit_base = gemv_phase(p.head, unit_base, EP_LOGITS, nullptr, 0, p.logits,
                       variant == DECODE_GREEDY ? &best : nullptr);
            ZQ_STAMP();
            if (variant == DECODE_GREEDY) {
                // first maximum wins (gpt2.zig:980-990): lanes, warps, CTAs, always preferring the lower index
                const uint32_t e_best = epoch++;
                unsigned long long* bx = ex.best + (size_t)(step & 1u) * ex.best_n;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    Best o;
                    o.v = __shfl_xor_sync(0xFFFFFFFFu, best.v, off);
                    o.i = __shfl_xor_sync(0xFFFFFFFFu, best.i, off);
                    best_update(best, o.v, o.i);
                }
                if (c.lane == 0) {
                    S.bval[c.warp] = best.v;
                    S.bidx[c.warp] = best.i;
                }
                cbar();
                if (c.tid == 0) {
                    Best b{S.bval[0], S.bidx[0]};
                    for (int wv = 1; wv < kConsumerWarps; ++wv) best_update(b, S.bval[wv], S.bidx[wv]);
                    xstore(bx + 2 * blockIdx.x, b.v, e_best);
                    xstore_u32(bx + 2 * blockIdx.x + 1, b.i, e_best);
                }
                // every CTA reads every candidate: the next token is known everywhere without another exchange
                Best b{-INFINITY, 0xFFFFFFFFu};
                for (uint32_t base = 0; base < gridDim.x; base += 32) {
                    const uint32_t k = base + c.lane;
                    float v[2];
                    xload_batch<2>(c, p, bx, 2 * k, 1u, 2 * gridDim.x, e_best, v);
                    if (k < gridDim.x) best_update(b, v[0], __float_as_uint(v[1]));
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    Best o;
                    o.v = __shfl_xor_sync(0xFFFFFFFFu, b.v, off);
                    o.i = __shfl_xor_sync(0xFFFFFFFFu, b.i, off);
                    best_update(b, o.v, o.i);
                }
                ZQ_CHECK_ABORT();
                tok = b.i;
                if (blockIdx.x == 0 && c.tid == 0) p.record[rec] = tok;
                rec += 1;
            }
        }
        pos += 1;
    }
#undef ZQ_STAMP
#undef ZQ_CHECK_ABORT
    if (blockIdx.x == 0 && c.tid == 0) {
        p.state[0] = tok;
        p.state[1] = pos;
        p.state[2] = rec;
    }
}

// ---- host side --------------------------------------------------------------------------------

// Tiles of up to 8 rows (one per lane group of the tensor-core tile). A small matrix gets smaller tiles so
// that at least half of the CTAs have one; rows that do not fit a ring slot are cut along K.
bool describe(DMat* d, const zq_weight* w, uint32_t slot_bytes, bool split, uint32_t grid) {
    d->qs = w->qs;
    d->sc = static_cast<const uint8_t*>(w->sc);
    d->type = (uint32_t)w->type;
    d->n_rows = w->out_dim;
    d->nb = w->nb;
    d->nbp = w->nbp;
    d->row_q_bytes = w->nbp * w->qb;
    d->row_s_bytes = w->scp * (w->type == ZQ_TYPE_Q4_1 ? 4u : 2u);
    d->pad_ = 0;
    d->split = split ? 1u : 0u;
    if (split && (w->out_dim & 1u)) return false;
    const uint32_t n = split ? w->out_dim / 2 : w->out_dim;  // rows to hand out (pairs of rows when split)
    auto tiles = [&](uint32_t rows) { const uint32_t per = split ? rows / 2 : rows; return (n + per - 1) / per; };
    uint32_t r = 8;
    while (r > (split ? 2u : 1u) && tiles(r) < grid / 2) r /= 2;
    d->rows_per_tile = r;
    d->n_tiles = tiles(r);
    d->tiles_div = d->n_tiles / grid;
    d->tiles_rem = d->n_tiles % grid;
    d->chunks_magic = 0xFFFFFFFFu;  // set below with the chunk count
    const uint32_t QUAD = w->qb * 4, SB = w->type == ZQ_TYPE_Q4_1 ? 4u : 2u, nq = w->nbp / 4;
    // A piece has at most 16 quads (the shared slot release of gemv_phase counts on it). Rows of a piece of a
    // 4-bit matrix lie an odd multiple of 64 bytes apart, so that the eight row segments of one load cover all banks.
    auto q_pitch = [&](uint32_t cq) { return cq * QUAD + ((QUAD == 64 && !(cq & 1u)) ? 64u : 0u); };
    auto piece_bytes = [&](uint32_t cq) { return r * (q_pitch(cq) + ((cq * 4 * SB + 15u) & ~15u) + 16u); };
    if (nq <= 16 && r * (d->row_q_bytes + d->row_s_bytes) <= slot_bytes) {
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

struct GemmaDecoder {
    DParams p;
    DLayer* d_layers = nullptr;
    void* d_misc = nullptr;  // abort word and the exchange buffers
    size_t smem = 0;
    uint32_t grid = 0;
    uint32_t launches = 0;
    uint32_t epoch = 1;      // first exchange number of the next launch (0 is what a fresh buffer holds)
    uint32_t exchanges_per_step = 0;
    size_t misc_bytes = 0;
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

    // slot size: eight q8_0 rows of 1152 weights with their scales (9.75 KB) unless the caller asks otherwise
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
    uint32_t slot_bytes = desc.slot_bytes ? desc.slot_bytes : 9856u;
    slot_bytes = (slot_bytes + 127u) & ~127u;

    GemmaDecoder* d = new (std::nothrow) GemmaDecoder;
    if (!d) return ZQ_ERR_NO_MEM;
    DParams& p = d->p;
    memset(&p, 0, sizeof(p));
    std::vector<DLayer> layers(desc.layers.size());
    memset(static_cast<void*>(layers.data()), 0, layers.size() * sizeof(DLayer));
    const uint32_t grid = (uint32_t)sm_count();
    bool ok = describe(&p.head, desc.token_embd, slot_bytes, false, grid);
    uint32_t terms = 0;
    auto note_terms = [&](const DMat& m) {
        const uint32_t t = 8 * (m.chunk_quads * 4 + 4);
        if (t > terms) terms = t;
    };
    note_terms(p.head);
    for (size_t l = 0; ok && l < layers.size(); ++l) {
        const GemmaDecoderLayer& s = desc.layers[l];
        DLayer& L = layers[l];
        ok = describe(&L.qkv, s.qkv, slot_bytes, false, grid) && describe(&L.o, s.o, slot_bytes, false, grid) &&
             describe(&L.gate_up, s.gate_up, slot_bytes, true, grid) && describe(&L.down, s.down, slot_bytes, false, grid);
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
    size_t after_image = (size_t)kConsumerWarps * p.terms_per_warp * 4;      // block terms of the dot phases
    if (after_image < (size_t)16 * kConsumers * 4) after_image = (size_t)16 * kConsumers * 4;  // staging of the quantiser
    if (after_image < (size_t)2 * E * 4) after_image = (size_t)2 * E * 4;      // norm weights
    p.terms_bytes = (uint32_t)after_image;
    const size_t gemv_scratch = (size_t)nbp_max * (32 + 8) + 128 + after_image;
    p.xh_off = nbp_max + (((nbp_max * 16u) & 127u) == 64u ? 0u : 4u);
    p.deal_limit = desc.deal_limit ? desc.deal_limit : 8u;
    auto magic = [](uint32_t d) { return d <= 1 ? 0xFFFFFFFFu : (uint32_t)(0x100000000ull / d); };
    p.group = group;
    p.half_d = D / 2;
    p.magic_chunks = magic(D / 8);
    p.magic_group = magic(group);
    p.magic_half = magic(D / 2);
    p.magic_nh = magic(nh);
    const size_t att_a = (size_t)(nh + nkv) * D * 4;
    const size_t att_b = (((size_t)desc.ctx + 3) & ~(size_t)3) * 4 + 2 * 8 * (size_t)(kVTile + 4) * 4;
    size_t scratch = gemv_scratch > att_a ? gemv_scratch : att_a;
    if (att_b > scratch) scratch = att_b;
    size_t off = kSharedHead;
    p.off_layers = (uint32_t)off;
    off = up(off + layers.size() * sizeof(DLayer), 128);
    p.off_xres = (uint32_t)off;
    off = up(off + (size_t)E * 4, 128);
    p.off_xs = (uint32_t)off;
    off = up(off + (size_t)E * 4, 128);
    p.off_rope = (uint32_t)off;
    off = up(off + (size_t)D * 4, 128);
    p.off_vnew = (uint32_t)off;
    off = up(off + (size_t)nkv * D * 4, 128);
    p.off_scratch = (uint32_t)off;
    off = up(off + scratch, 128);
    p.off_ring = (uint32_t)off;
    const size_t budget = (size_t)max_smem - 256;  // a little static shared memory of called functions
    if (off + 8 * (size_t)slot_bytes > budget) {
        delete d;
        return ZQ_ERR_UNSUPPORTED;
    }
    uint32_t n_slots = (uint32_t)((budget - off) / slot_bytes);
    if (n_slots > 64) n_slots = 64;
    if (desc.n_slots && desc.n_slots >= 8 && desc.n_slots <= n_slots) n_slots = desc.n_slots;
    p.n_slots = n_slots;
    p.slot_magic = (uint32_t)(0x100000000ull / n_slots);
    p.slot_bytes = slot_bytes;
    d->smem = off + (size_t)n_slots * slot_bytes;

    d->grid = grid;
    cudaError_t e = cudaFuncSetAttribute(gemma3_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)d->smem);
    int per_sm = 0;
    if (e == cudaSuccess)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemma3_decode_kernel, kThreads, d->smem);
    if (e != cudaSuccess || per_sm < 1) {
        delete d;
        if (e != cudaSuccess) return cuda_fail(e);
        return ZQ_ERR_UNSUPPORTED;
    }
    // exchange buffers (two of each) behind the abort word
    Exchange& ex = p.ex;
    ex.qkv_n = (nh + 2 * nkv) * D;
    ex.scores_n = nh * desc.ctx;
    ex.att_n = nh * D;
    ex.proj_n = E;
    ex.g_n = F;
    ex.ffn_n = E + d->grid;
    ex.best_n = 2 * d->grid;
    const size_t words = 2 * ((size_t)ex.qkv_n + ex.scores_n + ex.att_n + ex.proj_n + ex.g_n + ex.ffn_n + ex.best_n);
    d->misc_bytes = 256 + words * 8;
    if (cudaMalloc(&d->d_layers, layers.size() * sizeof(DLayer)) != cudaSuccess ||
        cudaMalloc(&d->d_misc, d->misc_bytes) != cudaSuccess) {
        delete d;
        return ZQ_ERR_NO_MEM;
    }
    e = cudaMemcpy(d->d_layers, layers.data(), layers.size() * sizeof(DLayer), cudaMemcpyHostToDevice);
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
    ex.g = w;
    w += 2 * (size_t)ex.g_n;
    ex.ffn = w;
    w += 2 * (size_t)ex.ffn_n;
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

int gemma_decoder_run(GemmaDecoder* d, uint32_t n_steps, int variant, cudaStream_t st) {
    if (n_steps == 0) return ZQ_OK;
    // launch ids 1, 2, 3, ... mark this launch's abort word
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
    ZQ_CUDA(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(gemma3_decode_kernel), dim3(d->grid), dim3(kThreads),
                                        args, d->smem, st));
    d->launches = launch_id;
    d->epoch += (uint32_t)need;
    return ZQ_OK;
}

// One step with cycle stamps: per CTA, thread 0's clock64() at the phase boundaries, in program order:
// token start; per layer 10 stamps (qkv prologue done, qkv done, scores done, softmax.V done, o prologue done,
// o done, ffn prologue done, gate/up done, down prologue done, down done); then head prologue done, head done.
// h_out[cta][cap].
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
