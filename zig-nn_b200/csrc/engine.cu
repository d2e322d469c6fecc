// Device-resident GPT-2 and Gemma-3 decode engines: the counterparts of zig-nn's gpt2(C)
// (src/models/gpt2.zig:198-532), gemma3(C) (src/models/gemma3.zig:243-848) and the one-encoder
// Metal engine (src/models/gemma3_metal.zig:189-260). All tensors are uploaded once; a decode step
// is a fixed sequence of kernel launches on the caller's stream with no host synchronisation.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <new>
#include <vector>

#include "decode_gemma.h"
#include "decode_gpt2.h"
#include "zq_internal.h"

namespace zq {
namespace {

struct DeviceArena {
    std::vector<void*> ptrs;
    size_t total = 0;
    ~DeviceArena() {
        for (void* p : ptrs) cudaFree(p);
    }
    int alloc(void** out, size_t bytes) {
        cudaError_t e = cudaMalloc(out, bytes ? bytes : 4);
        if (e != cudaSuccess) {
            g_last_cuda_error = (int)e;
            return e == cudaErrorMemoryAllocation ? ZQ_ERR_NO_MEM : ZQ_ERR_CUDA;
        }
        ptrs.push_back(*out);
        total += bytes;
        return ZQ_OK;
    }
    template <typename T>
    int alloc_n(T** out, size_t n) {
        return alloc(reinterpret_cast<void**>(out), n * sizeof(T));
    }
    int upload_f32(float** out, const float* host, size_t n, cudaStream_t st) {
        if (!host) return ZQ_ERR_BAD_ARG;
        int rc = alloc_n(out, n);
        if (rc != ZQ_OK) return rc;
        ZQ_CUDA(cudaMemcpyAsync(*out, host, n * sizeof(float), cudaMemcpyHostToDevice, st));
        return ZQ_OK;
    }
};

// A linear layer's weight: quantised (zq_weight) or plain f32 [out_dim][in_dim]
// (the .f32 branch of linear_forward_q, gpt2.zig:652-671).
struct Linear {
    zq_weight* qw = nullptr;
    float* f32w = nullptr;
    uint32_t out_dim = 0, in_dim = 0;
};

int upload_linear(Linear* L, const zq_tensor_ref& t, uint32_t out_dim, uint32_t in_dim,
                  DeviceArena& arena, cudaStream_t st) {
    if (!t.data || t.out_dim != out_dim || t.in_dim != in_dim) return ZQ_ERR_BAD_ARG;
    L->out_dim = out_dim;
    L->in_dim = in_dim;
    if (t.type == ZQ_TYPE_F32)
        return arena.upload_f32(&L->f32w, static_cast<const float*>(t.data), (size_t)out_dim * in_dim, st);
    if (!is_quant(t.type)) return ZQ_ERR_UNSUPPORTED;
    return zq_weight_upload(t.data, t.type, out_dim, in_dim, st, &L->qw);
}

// Step state in device memory: [0] current token, [1] its position, [2] next slot of the greedy record.
__global__ void set_state_kernel(uint32_t* state, uint32_t token, uint32_t pos, uint32_t rec) {
    state[0] = token;
    state[1] = pos;
    state[2] = rec;
}
// End of a greedy step: the argmax becomes the next token, is recorded, and the position advances.
__global__ void greedy_feed_kernel(uint32_t* state, const int32_t* arg, uint32_t* record) {
    const uint32_t tok = (uint32_t)*arg;
    record[state[2]] = tok;
    state[0] = tok;
    state[1] += 1;
    state[2] += 1;
}

// A decode step is a fixed launch sequence whose only varying inputs live in device memory, so it is
// captured once per variant and replayed. The first use of a variant runs eagerly (function
// attributes get set and launch errors surface outside capture); the second captures on the
// engine's own stream (the caller's may be the legacy default stream, which cannot capture); every
// use from then on is one graph launch on the caller's stream.
enum StepVariant { STEP_CACHE_ONLY = 0, STEP_LOGITS = 1, STEP_GREEDY = 2, STEP_BATCH = 3, STEP_VARIANTS = 4 };

struct StepGraphs {
    cudaGraphExec_t exec[STEP_VARIANTS] = {nullptr, nullptr, nullptr, nullptr};
    bool warmed[STEP_VARIANTS] = {false, false, false, false};
    cudaStream_t capture_stream = nullptr;
    bool disabled = false;
    ~StepGraphs() {
        for (cudaGraphExec_t e : exec)
            if (e) cudaGraphExecDestroy(e);
        if (capture_stream) cudaStreamDestroy(capture_stream);
    }
    template <typename Body>
    int run(int variant, cudaStream_t st, Body&& body) {
        if (disabled) return body(st);
        if (!warmed[variant]) {
            warmed[variant] = true;
            return body(st);
        }
        if (!exec[variant]) {
            if (!capture_stream) ZQ_CUDA(cudaStreamCreateWithFlags(&capture_stream, cudaStreamNonBlocking));
            ZQ_CUDA(cudaStreamBeginCapture(capture_stream, cudaStreamCaptureModeThreadLocal));
            const int rc = body(capture_stream);
            cudaGraph_t graph = nullptr;
            const cudaError_t e = cudaStreamEndCapture(capture_stream, &graph);
            if (rc != ZQ_OK || e != cudaSuccess) {
                if (graph) cudaGraphDestroy(graph);
                return rc != ZQ_OK ? rc : cuda_fail(e);
            }
            const cudaError_t ei = cudaGraphInstantiate(&exec[variant], graph, 0);
            cudaGraphDestroy(graph);
            if (ei != cudaSuccess) {
                exec[variant] = nullptr;
                return cuda_fail(ei);
            }
        }
        ZQ_CUDA(cudaGraphLaunch(exec[variant], st));
        return ZQ_OK;
    }
};

}  // namespace
}  // namespace zq

using namespace zq;

// ------------------------------------------------------------------------------ GPT-2

struct zq_gpt2 {
    zq_gpt2_config c;
    DeviceArena arena;
    StepGraphs graphs;
    float *wte = nullptr, *wpe = nullptr, *ln_f_w = nullptr, *ln_f_b = nullptr;
    struct Block {
        float *ln1_w, *ln1_b, *qkv_b, *proj_b, *ln2_w, *ln2_b, *fc_b, *mproj_b;
        Linear qkv, proj, fc, mproj;
    };
    std::vector<Block> blocks;
    std::vector<float*> k, v;  // per layer [ctx][embed]
    float *x = nullptr, *ln = nullptr, *qkv = nullptr, *att = nullptr, *hid = nullptr, *logits = nullptr;
    float* scores = nullptr;  // [head][ctx] attention scratch
    uint32_t* d_state = nullptr;
    int32_t* d_tokens = nullptr;   // token ids of a prefill chunk
    uint32_t max_rows = 1;         // rows the activation buffers hold (prefill chunk size)
    int32_t* d_arg = nullptr;
    uint32_t* d_record = nullptr;  // ctx entries for greedy decoding
    uint32_t seq_len = 0;
    GptDecoder* decoder = nullptr;  // the persistent decode kernel's view of this engine (nullptr: not available)
    int decode_mode = ZQ_DECODE_AUTO;
    ~zq_gpt2() {
        gpt_decoder_free(decoder);
        for (auto& b : blocks) {
            zq_weight_free(b.qkv.qw);
            zq_weight_free(b.proj.qw);
            zq_weight_free(b.fc.qw);
            zq_weight_free(b.mproj.qw);
        }
    }
};

// y[T][out] = W . (ln ? LayerNorm(x) : x)[T][in] + bias [gelu] [+ residual[T][out]]. Quantised weights run
// in passes of up to 16 rows through the decode kernel (every row keeps the arithmetic of a decode step);
// f32 weights (the .f32 branch of linear_forward_q, gpt2.zig:652-671) row by row with a separate epilogue.
// The norm runs as its own small launch: folded into the GEMV prologue every CTA repeats its two
// block-wide reductions before it can start, which measured 12% slower per step.
static int gpt2_linear(zq_gpt2* m, const Linear& L, const float* x, float* y, const float* bias, int gelu,
                       const float* residual, const float* ln_w, const float* ln_b, uint32_t T, cudaStream_t st) {
    int rc;
    if (ln_w) {
        if ((rc = zq_layer_norm(m->ln, x, ln_w, ln_b, T, L.in_dim, 1e-5f, st))) return rc;
        x = m->ln;
    }
    zq_epilogue ep{bias, gelu, nullptr, residual};
    if (L.qw) {
        rc = launch_gemv_mma_passes_f32(L.qw, x, y, T, &ep, st);
        if (rc == ZQ_ERR_LIMIT) rc = launch_gemv_f32(L.qw, x, y, T, &ep, st);
        return rc;
    }
    for (uint32_t r = 0; r < T; ++r) {
        float* y1 = y + (size_t)r * L.out_dim;
        rc = zq_matvec_f32(L.f32w, x + (size_t)r * L.in_dim, y1, L.out_dim, L.in_dim, st);
        if (rc == ZQ_OK && bias) rc = zq_add_broadcast(y1, y1, bias, L.out_dim, L.out_dim, st);
        if (rc == ZQ_OK && gelu) rc = zq_gelu(y1, y1, L.out_dim, st);
        if (rc == ZQ_OK && residual)
            rc = zq_add_broadcast(y1, y1, residual + (size_t)r * L.out_dim, L.out_dim, L.out_dim, st);
        if (rc != ZQ_OK) return rc;
    }
    return ZQ_OK;
}

// Forward pass over T consecutive tokens starting at position m->d_state[1] (gpt2.zig:423-509). T == 1 is a
// decode step (token in m->d_state[0]); T > 1 a batched prefill chunk (tokens in m->d_tokens). Eight
// launches per layer when decoding: ln1 | qkv | cache write + scores | softmax.V | proj + residual | ln2 |
// fc + gelu | mproj + residual. Logits are those of the last row.
static int gpt2_forward(zq_gpt2* m, uint32_t T, int variant, cudaStream_t st) {
    const zq_gpt2_config& C = m->c;
    const uint32_t E = C.embed, hd = E / C.head;
    if (T == 0 || T > m->max_rows) return ZQ_ERR_BAD_ARG;
    int rc;
    if ((rc = launch_gpt2_embed_step(m->x, m->wte, m->wpe, m->d_state, T == 1 ? nullptr : m->d_tokens, E, T, st)))
        return rc;
    for (uint32_t l = 0; l < C.layer; ++l) {
        const zq_gpt2::Block& b = m->blocks[l];
        if ((rc = gpt2_linear(m, b.qkv, m->x, m->qkv, b.qkv_b, 0, nullptr, b.ln1_w, b.ln1_b, T, st))) return rc;
        const float *k_new = m->qkv + E, *v_new = m->qkv + 2 * E;
        if (T > 1) {  // the decode step writes its cache row inside the scores kernel
            if ((rc = launch_write_kv_step(k_new, v_new, m->k[l], m->v[l], m->d_state, E, T, 3 * E, st))) return rc;
            k_new = v_new = nullptr;
        }
        if ((rc = launch_attention_step(m->qkv, m->k[l], m->v[l], k_new, v_new, m->att, nullptr, nullptr, nullptr,
                                        m->scores, C.head, C.head, hd, m->d_state, 0, C.ctx, ZQ_ATTN_GPT2_SOFTMAX, T,
                                        3 * E, nullptr, 0, nullptr, nullptr, nullptr, 0.0f, st)))
            return rc;
        if ((rc = gpt2_linear(m, b.proj, m->att, m->x, b.proj_b, 0, m->x, nullptr, nullptr, T, st))) return rc;
        if ((rc = gpt2_linear(m, b.fc, m->x, m->hid, b.fc_b, 1, nullptr, b.ln2_w, b.ln2_b, T, st))) return rc;
        if ((rc = gpt2_linear(m, b.mproj, m->hid, m->x, b.mproj_b, 0, m->x, nullptr, nullptr, T, st))) return rc;
    }
    if (variant != STEP_CACHE_ONLY) {
        const float* last = m->x + (size_t)(T - 1) * E;
        if ((rc = zq_layer_norm(m->ln, last, m->ln_f_w, m->ln_f_b, 1, E, 1e-5f, st))) return rc;
        if ((rc = launch_matvec_ln_f32(m->wte, m->ln, m->logits, C.vocab, E, nullptr, nullptr, 0.0f, st))) return rc;
    }
    if (variant == STEP_GREEDY) {
        if ((rc = zq_argmax(m->logits, C.vocab, m->d_arg, st))) return rc;
        greedy_feed_kernel<<<1, 1, 0, st>>>(m->d_state, m->d_arg, m->d_record);
        ZQ_LAUNCH_CHECK();
    }
    return ZQ_OK;
}

static bool gpt2_persistent(const zq_gpt2* m) {
    return m->decoder != nullptr && m->decode_mode != ZQ_DECODE_LAUNCH_SEQUENCE;
}

static int gpt2_run(zq_gpt2* m, int variant, cudaStream_t st) {
    if (gpt2_persistent(m)) return gpt_decoder_run(m->decoder, 1, variant, st);
    return m->graphs.run(variant, st, [&](cudaStream_t s) { return gpt2_forward(m, 1, variant, s); });
}

// The persistent decode kernel's view of the engine: built once, after every buffer exists. Engines with an f32
// linear (the .f32 branch of linear_forward_q) keep the launch sequence.
static int gpt2_make_decoder(zq_gpt2* m) {
    const zq_gpt2_config& C = m->c;
    for (const auto& b : m->blocks)
        if (!b.qkv.qw || !b.proj.qw || !b.fc.qw || !b.mproj.qw) return ZQ_OK;
    GptDecoderDesc d;
    d.embed = C.embed;
    d.n_head = C.head;
    d.ffn = C.ffn;
    d.ctx = C.ctx;
    d.vocab = C.vocab;
    d.eps = 1e-5f;
    d.wte = m->wte;
    d.wpe = m->wpe;
    d.ln_f_w = m->ln_f_w;
    d.ln_f_b = m->ln_f_b;
    for (uint32_t l = 0; l < C.layer; ++l) {
        const zq_gpt2::Block& b = m->blocks[l];
        GptDecoderLayer L;
        L.qkv = b.qkv.qw;
        L.proj = b.proj.qw;
        L.fc = b.fc.qw;
        L.mproj = b.mproj.qw;
        L.qkv_b = b.qkv_b;
        L.proj_b = b.proj_b;
        L.fc_b = b.fc_b;
        L.mproj_b = b.mproj_b;
        L.ln1_w = b.ln1_w;
        L.ln1_b = b.ln1_b;
        L.ln2_w = b.ln2_w;
        L.ln2_b = b.ln2_b;
        L.kc = m->k[l];
        L.vc = m->v[l];
        d.layers.push_back(L);
    }
    d.logits = m->logits;
    d.state = m->d_state;
    d.record = m->d_record;
    const int rc = gpt_decoder_create(d, &m->decoder);
    return rc == ZQ_ERR_UNSUPPORTED ? ZQ_OK : rc;
}

extern "C" {

int zq_gpt2_create(const zq_gpt2_config* cfg, const zq_gpt2_weights* w, zq_stream stream,
                   zq_gpt2** out) {
    if (!cfg || !w || !out || !w->blocks) return ZQ_ERR_BAD_ARG;
    *out = nullptr;
    if (!cfg->vocab || !cfg->embed || !cfg->head || !cfg->layer || !cfg->ctx || !cfg->ffn ||
        cfg->embed % cfg->head || cfg->embed % 32 || cfg->ffn % 32)
        return ZQ_ERR_BAD_ARG;
    if (cfg->ctx > 180 * 1024 / 4) return ZQ_ERR_LIMIT;  // one attention row must fit shared memory
    zq_gpt2* m = new (std::nothrow) zq_gpt2;
    if (!m) return ZQ_ERR_NO_MEM;
    m->c = *cfg;
    cudaStream_t st = as_stream(stream);
    const uint32_t E = cfg->embed, F = cfg->ffn;
    int rc = ZQ_OK;
#define TRY(expr)                  \
    do {                           \
        if ((rc = (expr)) != ZQ_OK) { \
            delete m;              \
            return rc;             \
        }                          \
    } while (0)
    TRY(m->arena.upload_f32(&m->wte, w->wte, (size_t)cfg->vocab * E, st));
    TRY(m->arena.upload_f32(&m->wpe, w->wpe, (size_t)cfg->ctx * E, st));
    TRY(m->arena.upload_f32(&m->ln_f_w, w->ln_f_weight, E, st));
    TRY(m->arena.upload_f32(&m->ln_f_b, w->ln_f_bias, E, st));
    m->blocks.resize(cfg->layer);
    m->k.resize(cfg->layer);
    m->v.resize(cfg->layer);
    for (uint32_t l = 0; l < cfg->layer; ++l) {
        const zq_gpt2_block& s = w->blocks[l];
        zq_gpt2::Block& b = m->blocks[l];
        TRY(m->arena.upload_f32(&b.ln1_w, s.ln1_weight, E, st));
        TRY(m->arena.upload_f32(&b.ln1_b, s.ln1_bias, E, st));
        TRY(m->arena.upload_f32(&b.qkv_b, s.attn_qkv_bias, 3 * (size_t)E, st));
        TRY(m->arena.upload_f32(&b.proj_b, s.attn_proj_bias, E, st));
        TRY(m->arena.upload_f32(&b.ln2_w, s.ln2_weight, E, st));
        TRY(m->arena.upload_f32(&b.ln2_b, s.ln2_bias, E, st));
        TRY(m->arena.upload_f32(&b.fc_b, s.mlp_fc_bias, F, st));
        TRY(m->arena.upload_f32(&b.mproj_b, s.mlp_proj_bias, E, st));
        TRY(upload_linear(&b.qkv, s.attn_qkv_weight, 3 * E, E, m->arena, st));
        TRY(upload_linear(&b.proj, s.attn_proj_weight, E, E, m->arena, st));
        TRY(upload_linear(&b.fc, s.mlp_fc_weight, F, E, m->arena, st));
        TRY(upload_linear(&b.mproj, s.mlp_proj_weight, E, F, m->arena, st));
        TRY(m->arena.alloc_n(&m->k[l], (size_t)cfg->ctx * E));
        TRY(m->arena.alloc_n(&m->v[l], (size_t)cfg->ctx * E));
        cudaMemsetAsync(m->k[l], 0, (size_t)cfg->ctx * E * sizeof(float), st);
        cudaMemsetAsync(m->v[l], 0, (size_t)cfg->ctx * E * sizeof(float), st);
    }
    // activation buffers hold a prefill chunk of up to 128 tokens (a decode step uses row 0)
    m->max_rows = cfg->ctx < 128 ? cfg->ctx : 128;
    const size_t R = m->max_rows;
    TRY(m->arena.alloc_n(&m->x, R * E));
    TRY(m->arena.alloc_n(&m->ln, R * (E > F ? E : F)));
    TRY(m->arena.alloc_n(&m->qkv, R * 3 * (size_t)E));
    TRY(m->arena.alloc_n(&m->att, R * E));
    TRY(m->arena.alloc_n(&m->hid, R * F));
    TRY(m->arena.alloc_n(&m->logits, cfg->vocab));
    TRY(m->arena.alloc_n(&m->scores, R * cfg->head * cfg->ctx));
    TRY(m->arena.alloc_n(&m->d_tokens, R));
    TRY(m->arena.alloc_n(&m->d_state, 4));
    TRY(m->arena.alloc_n(&m->d_arg, 1));
    TRY(m->arena.alloc_n(&m->d_record, cfg->ctx));
    TRY(gpt2_make_decoder(m));
#undef TRY
    cudaError_t e = cudaStreamSynchronize(st);  // host weight buffers may be released after create
    if (e != cudaSuccess) {
        delete m;
        return cuda_fail(e);
    }
    *out = m;
    return ZQ_OK;
}

int zq_gpt2_set_decode_mode(zq_gpt2* m, int mode) {
    if (!m || mode < ZQ_DECODE_AUTO || mode > ZQ_DECODE_PERSISTENT) return ZQ_ERR_BAD_ARG;
    if (mode == ZQ_DECODE_PERSISTENT && !m->decoder) return ZQ_ERR_UNSUPPORTED;
    m->decode_mode = mode;
    return ZQ_OK;
}

int zq_gpt2_decode_mode(const zq_gpt2* m, int* mode) {
    if (!m || !mode) return ZQ_ERR_BAD_ARG;
    *mode = gpt2_persistent(m) ? ZQ_DECODE_PERSISTENT : ZQ_DECODE_LAUNCH_SEQUENCE;
    return ZQ_OK;
}

int zq_gpt2_free(zq_gpt2* m) {
    delete m;
    return ZQ_OK;
}

int zq_gpt2_reset_cache(zq_gpt2* m) {
    if (!m) return ZQ_ERR_BAD_ARG;
    m->seq_len = 0;
    return ZQ_OK;
}

int zq_gpt2_seq_len(const zq_gpt2* m, uint32_t* seq_len) {
    if (!m || !seq_len) return ZQ_ERR_BAD_ARG;
    *seq_len = m->seq_len;
    return ZQ_OK;
}

int zq_gpt2_prefill(zq_gpt2* m, const uint32_t* h_tokens, uint32_t n, zq_stream stream,
                    const float** d_logits) {
    if (!m || !h_tokens || !d_logits) return ZQ_ERR_BAD_ARG;
    if (n == 0 || n > m->c.ctx) return ZQ_ERR_SEQUENCE;
    for (uint32_t t = 0; t < n; ++t)
        if (h_tokens[t] >= m->c.vocab) return ZQ_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    m->seq_len = 0;
    for (uint32_t t0 = 0; t0 < n; t0 += m->max_rows) {  // chunks of up to max_rows tokens
        const uint32_t T = n - t0 < m->max_rows ? n - t0 : m->max_rows;
        const bool last = t0 + T == n;
        set_state_kernel<<<1, 1, 0, st>>>(m->d_state, h_tokens[t0], t0, 0);
        ZQ_LAUNCH_CHECK();
        int rc;
        if (T == 1) {
            rc = gpt2_run(m, last ? STEP_LOGITS : STEP_CACHE_ONLY, st);
        } else {
            ZQ_CUDA(cudaMemcpyAsync(m->d_tokens, h_tokens + t0, T * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
            rc = gpt2_forward(m, T, last ? STEP_LOGITS : STEP_CACHE_ONLY, st);
            ZQ_CUDA(cudaStreamSynchronize(st));  // h_tokens is the caller's memory
        }
        if (rc != ZQ_OK) return rc;
    }
    m->seq_len = n;
    *d_logits = m->logits;
    return ZQ_OK;
}

int zq_gpt2_decode_next(zq_gpt2* m, uint32_t token, zq_stream stream, const float** d_logits) {
    if (!m || !d_logits) return ZQ_ERR_BAD_ARG;
    if (m->seq_len >= m->c.ctx) return ZQ_ERR_SEQUENCE;
    if (token >= m->c.vocab) return ZQ_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    set_state_kernel<<<1, 1, 0, st>>>(m->d_state, token, m->seq_len, 0);
    ZQ_LAUNCH_CHECK();
    int rc = gpt2_run(m, STEP_LOGITS, st);
    if (rc != ZQ_OK) return rc;
    m->seq_len += 1;
    *d_logits = m->logits;
    return ZQ_OK;
}

int zq_gpt2_decode_greedy(zq_gpt2* m, uint32_t first_token, uint32_t n_steps, zq_stream stream,
                          uint32_t* h_tokens_out) {
    if (!m || !h_tokens_out) return ZQ_ERR_BAD_ARG;
    if (n_steps == 0) return ZQ_OK;
    if ((uint64_t)m->seq_len + n_steps > m->c.ctx) return ZQ_ERR_SEQUENCE;
    if (first_token >= m->c.vocab) return ZQ_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    set_state_kernel<<<1, 1, 0, st>>>(m->d_state, first_token, m->seq_len, 0);
    ZQ_LAUNCH_CHECK();
    if (gpt2_persistent(m)) {  // every step inside one launch: the argmax feeds the next token on the device
        int rc = gpt_decoder_run(m->decoder, n_steps, DECODE_GREEDY, st);
        if (rc != ZQ_OK) return rc;
        m->seq_len += n_steps;
    } else {
        for (uint32_t s = 0; s < n_steps; ++s) {
            int rc = gpt2_run(m, STEP_GREEDY, st);
            if (rc != ZQ_OK) return rc;
            m->seq_len += 1;
        }
    }
    ZQ_CUDA(cudaMemcpyAsync(h_tokens_out, m->d_record, n_steps * sizeof(uint32_t),
                            cudaMemcpyDeviceToHost, st));
    ZQ_CUDA(cudaStreamSynchronize(st));
    return ZQ_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------ Gemma-3

struct zq_gemma3 {
    zq_gemma3_config c;
    DeviceArena arena;
    StepGraphs graphs;
    zq_weight* token_embd = nullptr;
    float* output_norm_w = nullptr;
    struct Block {
        float *attn_norm_w, *post_attn_norm_w, *q_norm_w, *k_norm_w, *ffn_norm_w, *post_ffw_norm_w;
        // q|k|v and gate|up are stored as one matrix each when their types agree (rows are independent,
        // so stacking them changes no result and saves launches); otherwise the parts stay separate.
        zq_weight *qkv, *q, *k, *v, *o, *gate_up, *gate, *up, *down;
    };
    std::vector<Block> blocks;
    std::vector<float*> k, v;  // per layer [ctx][kv_dim]
    float* freqs = nullptr;
    float *x = nullptr, *qkv = nullptr, *proj = nullptr, *gu = nullptr, *ffn = nullptr, *logits = nullptr;
    float* scores = nullptr;  // [head][ctx] attention scratch
    int8_t* xq = nullptr;     // quantised activation row, max(embed, ffn, q_dim)
    float* xscale = nullptr;
    int32_t* xsum = nullptr;
    uint32_t* d_state = nullptr;
    int32_t* d_tokens = nullptr;  // token ids of a prefill chunk / of a batched decode step
    uint32_t max_rows = 1;        // rows the activation buffers hold (prefill chunk size, >= n_seq)
    int32_t* d_arg = nullptr;
    uint32_t* d_record = nullptr;
    uint32_t seq_len = 0;
    // several independent sequences (batched decode): each has its own cache slot and position
    uint32_t n_seq = 1;
    uint32_t* d_pos = nullptr;            // [n_seq] positions of a batched decode step
    std::vector<uint32_t> seq_lens;       // host copy, [n_seq]
    float* logits_batch = nullptr;        // [n_seq][vocab]
    // One-sequence decode steps run as one persistent cooperative kernel when the model fits its plan
    // (decode_gemma.cu); otherwise, and for prefill chunks and batched sequences, as the launch sequence.
    GemmaDecoder* decoder = nullptr;
    int decode_mode = ZQ_DECODE_AUTO;
    ~zq_gemma3() {
        gemma_decoder_free(decoder);
        zq_weight_free(token_embd);
        for (auto& b : blocks) {
            zq_weight_free(b.qkv);
            zq_weight_free(b.q);
            zq_weight_free(b.k);
            zq_weight_free(b.v);
            zq_weight_free(b.o);
            zq_weight_free(b.gate_up);
            zq_weight_free(b.gate);
            zq_weight_free(b.up);
            zq_weight_free(b.down);
        }
    }
};

// Activation rows are quantised once (thread_pool.zig:111-114); any number of weights consume them.
// T rows: one exact GEMV per row, or from five rows up the exact int8 GEMM (identical results).
static int gemma_linear(zq_gemma3* m, const zq_weight* w, float* y, uint32_t y_stride, uint32_t T, cudaStream_t st) {
    if (T >= 2 && y_stride == w->out_dim) return launch_gemm_q8(w, m->xq, m->xscale, m->xsum, y, T, nullptr, st);
    for (uint32_t r = 0; r < T; ++r) {
        int rc = launch_gemv_q8(w, m->xq + (size_t)r * w->in_dim, m->xscale + (size_t)r * w->nb,
                                m->xsum + (size_t)r * w->nb, y + (size_t)r * y_stride, 1, nullptr, st);
        if (rc != ZQ_OK) return rc;
    }
    return ZQ_OK;
}

// Forward pass over T consecutive tokens starting at position m->d_state[1] (gemma3.zig:551-846).
// T == 1 is a decode step (token in m->d_state[0]); T > 1 is a batched prefill chunk (tokens in
// m->d_tokens), every row computed with exactly the arithmetic of a decode step. About ten launches per
// layer: [norm+quantise] qkv | qk-norm+rope+cache | scores | softmax.V+quantise | o |
// post-norm+residual+pre-norm+quantise | gate,up | gelu.mul+quantise | down | post-norm+residual+...
// Logits (and the argmax of a greedy step) are those of the last row.
// batch == false: the T rows are consecutive tokens of sequence `seq` (its cache slot). batch == true: row r
// is the next token of sequence r, at position m->d_pos[r], and every row's logits go to m->logits_batch.
static int gemma3_forward(zq_gemma3* m, uint32_t T, int variant, cudaStream_t st, uint32_t seq = 0,
                          bool batch = false) {
    const zq_gemma3_config& C = m->c;
    const uint32_t E = C.embed, D = C.head_dim, QD = C.head * D, KD = C.head_kv * D, F = C.ffn;
    const uint32_t QKV = QD + 2 * KD;
    if (T == 0 || T > m->max_rows || seq >= m->n_seq) return ZQ_ERR_BAD_ARG;
    const size_t cache_stride = (size_t)C.ctx * KD;
    const uint32_t* row_pos = batch ? m->d_pos : nullptr;
    const size_t slot = batch ? 0 : seq * cache_stride;
    int rc;
    const int32_t* ids = (T == 1 && !batch) ? reinterpret_cast<const int32_t*>(m->d_state) : m->d_tokens;
    if ((rc = zq_dequant_rows_scaled(m->token_embd, ids, T, sqrtf((float)E), m->x, st))) return rc;
    if ((rc = launch_norm_quant(m->x, m->blocks[0].attn_norm_w, nullptr, nullptr, E, C.rms_eps, m->xq,
                                m->xscale, m->xsum, T, E, st)))
        return rc;
    for (uint32_t l = 0; l < C.layer; ++l) {
        const zq_gemma3::Block& b = m->blocks[l];
        // attention block (gemma3.zig:662-731)
        if (b.qkv) {
            if ((rc = gemma_linear(m, b.qkv, m->qkv, QKV, T, st))) return rc;
        } else {
            if ((rc = gemma_linear(m, b.q, m->qkv, QKV, T, st))) return rc;
            if ((rc = gemma_linear(m, b.k, m->qkv + QD, QKV, T, st))) return rc;
            if ((rc = gemma_linear(m, b.v, m->qkv + QD + KD, QKV, T, st))) return rc;
        }
        const bool global = (l % C.global_every) == C.global_every - 1;
        const uint32_t window = global ? 0u : C.sliding_window;
        const uint32_t max_len = (window && window < C.ctx) ? window : C.ctx;
        // A prefill chunk needs every token's key in the cache before any score: separate launch. A decode
        // step (one row, or one row per independent sequence) normalises / rotates q and its own new key
        // inside the scores kernel, which also stores the cache row.
        const bool fused_qk = T == 1 || batch;
        if (!fused_qk) {
            if ((rc = launch_qk_norm_rope_kv(m->qkv, b.q_norm_w, b.k_norm_w, m->freqs, m->k[l] + slot, m->v[l] + slot,
                                             m->d_state, C.head, C.head_kv, D, C.rms_eps, T, QKV, row_pos,
                                             cache_stride, st)))
                return rc;
        }
        if ((rc = launch_attention_step(m->qkv, m->k[l] + slot, m->v[l] + slot, fused_qk ? m->qkv + QD : nullptr,
                                        fused_qk ? m->qkv + QD + KD : nullptr, nullptr, m->xq, m->xscale, m->xsum,
                                        m->scores, C.head, C.head_kv, D, m->d_state, window, max_len, 0, T, QKV, row_pos,
                                        cache_stride, fused_qk ? b.q_norm_w : nullptr, b.k_norm_w, m->freqs, C.rms_eps,
                                        st)))
            return rc;
        if ((rc = gemma_linear(m, b.o, m->proj, E, T, st))) return rc;
        if ((rc = launch_norm_quant(m->proj, b.post_attn_norm_w, m->x, b.ffn_norm_w, E, C.rms_eps, m->xq,
                                    m->xscale, m->xsum, T, E, st)))
            return rc;
        // FFN block (gemma3.zig:734-773)
        if (b.gate_up) {
            if ((rc = gemma_linear(m, b.gate_up, m->gu, 2 * F, T, st))) return rc;
        } else {
            if ((rc = gemma_linear(m, b.gate, m->gu, 2 * F, T, st))) return rc;
            if ((rc = gemma_linear(m, b.up, m->gu + F, 2 * F, T, st))) return rc;
        }
        if ((rc = launch_gelu_mul_quant(m->gu, m->gu + F, F, m->xq, m->xscale, m->xsum, T, 2 * F, st))) return rc;
        if ((rc = gemma_linear(m, b.down, m->ffn, E, T, st))) return rc;
        const float* next_norm = l + 1 < C.layer ? m->blocks[l + 1].attn_norm_w
                                 : (variant != STEP_CACHE_ONLY ? m->output_norm_w : nullptr);
        if (next_norm) {
            if ((rc = launch_norm_quant(m->ffn, b.post_ffw_norm_w, m->x, next_norm, E, C.rms_eps, m->xq, m->xscale,
                                        m->xsum, T, E, st)))
                return rc;
        } else if ((rc = zq_rms_norm_residual(m->ffn, b.post_ffw_norm_w, m->x, E, T, C.rms_eps, st))) {
            return rc;
        }
    }
    if (variant != STEP_CACHE_ONLY && batch) {  // every sequence's logits
        if ((rc = gemma_linear(m, m->token_embd, m->logits_batch, C.vocab, T, st))) return rc;
    } else if (variant != STEP_CACHE_ONLY) {  // the last row's logits
        const zq_weight* w = m->token_embd;
        const size_t r = T - 1;
        if ((rc = launch_gemv_q8(w, m->xq + r * w->in_dim, m->xscale + r * w->nb, m->xsum + r * w->nb, m->logits, 1,
                                 nullptr, st)))
            return rc;
    }
    if (variant == STEP_GREEDY) {
        if ((rc = zq_argmax(m->logits, C.vocab, m->d_arg, st))) return rc;
        greedy_feed_kernel<<<1, 1, 0, st>>>(m->d_state, m->d_arg, m->d_record);
        ZQ_LAUNCH_CHECK();
    }
    return ZQ_OK;
}

static bool gemma3_persistent(const zq_gemma3* m) {
    return m->decoder != nullptr && m->decode_mode != ZQ_DECODE_LAUNCH_SEQUENCE;
}

static int gemma3_run(zq_gemma3* m, int variant, cudaStream_t st) {
    if (gemma3_persistent(m)) return gemma_decoder_run(m->decoder, 1, variant, st);
    return m->graphs.run(variant, st, [&](cudaStream_t s) { return gemma3_forward(m, 1, variant, s); });
}

// The persistent decode kernel's view of the engine: built once, after every buffer exists.
static int gemma3_make_decoder(zq_gemma3* m) {
    const zq_gemma3_config& C = m->c;
    if (m->n_seq != 1) return ZQ_OK;
    for (const auto& b : m->blocks)
        if (!b.qkv || !b.gate_up) return ZQ_OK;  // mixed types inside q|k|v or gate|up: launch sequence only
    GemmaDecoderDesc d;
    d.embed = C.embed;
    d.head_dim = C.head_dim;
    d.n_head = C.head;
    d.n_kv = C.head_kv;
    d.ffn = C.ffn;
    d.ctx = C.ctx;
    d.eps = C.rms_eps;
    d.embed_scale = sqrtf((float)C.embed);
    d.token_embd = m->token_embd;
    d.output_norm_w = m->output_norm_w;
    d.freqs = m->freqs;
    for (uint32_t l = 0; l < C.layer; ++l) {
        const zq_gemma3::Block& b = m->blocks[l];
        GemmaDecoderLayer L;
        L.qkv = b.qkv;
        L.o = b.o;
        L.gate_up = b.gate_up;
        L.down = b.down;
        L.attn_norm_w = b.attn_norm_w;
        L.post_attn_norm_w = b.post_attn_norm_w;
        L.q_norm_w = b.q_norm_w;
        L.k_norm_w = b.k_norm_w;
        L.ffn_norm_w = b.ffn_norm_w;
        L.post_ffw_norm_w = b.post_ffw_norm_w;
        L.kc = m->k[l];
        L.vc = m->v[l];
        const bool global = (l % C.global_every) == C.global_every - 1;
        L.window = (global || C.sliding_window >= C.ctx) ? 0u : C.sliding_window;
        d.layers.push_back(L);
    }
    d.logits = m->logits;
    d.state = m->d_state;
    d.record = m->d_record;
    const int rc = gemma_decoder_create(d, &m->decoder);
    return rc == ZQ_ERR_UNSUPPORTED ? ZQ_OK : rc;
}

// Upload several GGUF matrices with the same in_dim and type as one matrix of stacked rows.
static int upload_stacked(zq_weight** dst, const zq_tensor_ref* const* parts, int n_parts, uint32_t in_dim,
                          cudaStream_t st) {
    size_t total_rows = 0, total_bytes = 0;
    for (int i = 0; i < n_parts; ++i) {
        total_rows += parts[i]->out_dim;
        total_bytes += zq_tensor_bytes(parts[i]->type, (size_t)parts[i]->out_dim * in_dim);
    }
    std::vector<uint8_t> host;
    try {
        host.resize(total_bytes);
    } catch (...) {
        return ZQ_ERR_NO_MEM;
    }
    size_t off = 0;
    for (int i = 0; i < n_parts; ++i) {
        const size_t nbytes = zq_tensor_bytes(parts[i]->type, (size_t)parts[i]->out_dim * in_dim);
        memcpy(host.data() + off, parts[i]->data, nbytes);
        off += nbytes;
    }
    int rc = zq_weight_upload(host.data(), parts[0]->type, (uint32_t)total_rows, in_dim, st, dst);
    if (rc != ZQ_OK) return rc;
    ZQ_CUDA(cudaStreamSynchronize(st));  // `host` is released on return
    return ZQ_OK;
}

extern "C" {

int zq_gemma3_create(const zq_gemma3_config* cfg, const zq_gemma3_weights* w, zq_stream stream,
                     zq_gemma3** out) {
    return zq_gemma3_create_batch(cfg, w, 1, stream, out);
}

int zq_gemma3_create_batch(const zq_gemma3_config* cfg, const zq_gemma3_weights* w, uint32_t n_seq,
                           zq_stream stream, zq_gemma3** out) {
    if (!cfg || !w || !out || !w->blocks || n_seq == 0 || n_seq > 1024) return ZQ_ERR_BAD_ARG;
    *out = nullptr;
    const zq_gemma3_config& C = *cfg;
    if (!C.vocab || !C.embed || !C.head || !C.head_kv || !C.head_dim || !C.layer || !C.ctx || !C.ffn ||
        !C.global_every || C.head % C.head_kv || C.embed % 32 || C.ffn % 32 || C.head_dim % 32)
        return ZQ_ERR_BAD_ARG;
    const uint32_t E = C.embed, D = C.head_dim, QD = C.head * D, KD = C.head_kv * D, F = C.ffn;
    uint32_t max_dim = E > F ? E : F;
    if (QD > max_dim) max_dim = QD;
    if (max_dim > 16384) return ZQ_ERR_LIMIT;
    if (C.ctx > 180 * 1024 / 4) return ZQ_ERR_LIMIT;  // one attention row must fit shared memory
    zq_gemma3* m = new (std::nothrow) zq_gemma3;
    if (!m) return ZQ_ERR_NO_MEM;
    m->c = C;
    m->n_seq = n_seq;
    m->seq_lens.assign(n_seq, 0);
    cudaStream_t st = as_stream(stream);
    int rc = ZQ_OK;
#define TRY(expr)                  \
    do {                           \
        if ((rc = (expr)) != ZQ_OK) { \
            delete m;              \
            return rc;             \
        }                          \
    } while (0)
    auto check_q = [&](const zq_tensor_ref& t, uint32_t od, uint32_t id) -> int {
        if (!t.data || t.out_dim != od || t.in_dim != id) return ZQ_ERR_BAD_ARG;
        if (!is_quant(t.type)) return ZQ_ERR_UNSUPPORTED;
        return ZQ_OK;
    };
    auto up_q = [&](zq_weight** dst, const zq_tensor_ref& t, uint32_t od, uint32_t id) -> int {
        int r = check_q(t, od, id);
        return r != ZQ_OK ? r : zq_weight_upload(t.data, t.type, od, id, st, dst);
    };
    TRY(up_q(&m->token_embd, w->token_embd, C.vocab, E));
    TRY(m->arena.upload_f32(&m->output_norm_w, w->output_norm_weight, E, st));
    m->blocks.assign(C.layer, zq_gemma3::Block{});
    m->k.resize(C.layer);
    m->v.resize(C.layer);
    for (uint32_t l = 0; l < C.layer; ++l) {
        const zq_gemma3_block& s = w->blocks[l];
        zq_gemma3::Block& b = m->blocks[l];
        TRY(m->arena.upload_f32(&b.attn_norm_w, s.attn_norm_weight, E, st));
        TRY(m->arena.upload_f32(&b.post_attn_norm_w, s.post_attention_norm_weight, E, st));
        TRY(m->arena.upload_f32(&b.q_norm_w, s.attn_q_norm_weight, D, st));
        TRY(m->arena.upload_f32(&b.k_norm_w, s.attn_k_norm_weight, D, st));
        TRY(m->arena.upload_f32(&b.ffn_norm_w, s.ffn_norm_weight, E, st));
        TRY(m->arena.upload_f32(&b.post_ffw_norm_w, s.post_ffw_norm_weight, E, st));
        TRY(check_q(s.attn_q_weight, QD, E));
        TRY(check_q(s.attn_k_weight, KD, E));
        TRY(check_q(s.attn_v_weight, KD, E));
        if (s.attn_q_weight.type == s.attn_k_weight.type && s.attn_q_weight.type == s.attn_v_weight.type) {
            const zq_tensor_ref* parts[3] = {&s.attn_q_weight, &s.attn_k_weight, &s.attn_v_weight};
            TRY(upload_stacked(&b.qkv, parts, 3, E, st));
        } else {
            TRY(up_q(&b.q, s.attn_q_weight, QD, E));
            TRY(up_q(&b.k, s.attn_k_weight, KD, E));
            TRY(up_q(&b.v, s.attn_v_weight, KD, E));
        }
        TRY(up_q(&b.o, s.attn_output_weight, E, QD));
        TRY(check_q(s.ffn_gate_weight, F, E));
        TRY(check_q(s.ffn_up_weight, F, E));
        if (s.ffn_gate_weight.type == s.ffn_up_weight.type) {
            const zq_tensor_ref* parts[2] = {&s.ffn_gate_weight, &s.ffn_up_weight};
            TRY(upload_stacked(&b.gate_up, parts, 2, E, st));
        } else {
            TRY(up_q(&b.gate, s.ffn_gate_weight, F, E));
            TRY(up_q(&b.up, s.ffn_up_weight, F, E));
        }
        TRY(up_q(&b.down, s.ffn_down_weight, E, F));
        TRY(m->arena.alloc_n(&m->k[l], (size_t)n_seq * C.ctx * KD));  // one cache slot per sequence
        TRY(m->arena.alloc_n(&m->v[l], (size_t)n_seq * C.ctx * KD));
        cudaMemsetAsync(m->k[l], 0, (size_t)n_seq * C.ctx * KD * sizeof(float), st);
        cudaMemsetAsync(m->v[l], 0, (size_t)n_seq * C.ctx * KD * sizeof(float), st);
    }
    {
        std::vector<float> hf(D / 2);
        zq_rope_freqs_host(D, C.rope_base, hf.data());
        TRY(m->arena.alloc_n(&m->freqs, D / 2));
        cudaError_t e = cudaMemcpyAsync(m->freqs, hf.data(), hf.size() * sizeof(float),
                                        cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);  // hf goes out of scope
        if (e != cudaSuccess) {
            delete m;
            return cuda_fail(e);
        }
    }
    // activation buffers hold a prefill chunk of up to 128 tokens (a decode step uses row 0)
    m->max_rows = C.ctx < 128 ? C.ctx : 128;
    if (m->max_rows < n_seq) m->max_rows = n_seq;
    const size_t R = m->max_rows;
    TRY(m->arena.alloc_n(&m->d_pos, n_seq));
    if (n_seq > 1) TRY(m->arena.alloc_n(&m->logits_batch, (size_t)n_seq * C.vocab));
    TRY(m->arena.alloc_n(&m->x, R * E));
    TRY(m->arena.alloc_n(&m->qkv, R * ((size_t)QD + 2 * KD)));
    TRY(m->arena.alloc_n(&m->proj, R * E));
    TRY(m->arena.alloc_n(&m->gu, R * 2 * (size_t)F));
    TRY(m->arena.alloc_n(&m->ffn, R * E));
    TRY(m->arena.alloc_n(&m->logits, C.vocab));
    TRY(m->arena.alloc_n(&m->scores, R * C.head * C.ctx));
    TRY(m->arena.alloc_n(&m->xq, R * max_dim));
    TRY(m->arena.alloc_n(&m->xscale, R * (max_dim / 32)));
    TRY(m->arena.alloc_n(&m->xsum, R * (max_dim / 32)));
    TRY(m->arena.alloc_n(&m->d_tokens, R));
    TRY(m->arena.alloc_n(&m->d_state, 4));
    TRY(m->arena.alloc_n(&m->d_arg, 1));
    TRY(m->arena.alloc_n(&m->d_record, C.ctx));
    TRY(gemma3_make_decoder(m));
#undef TRY
    cudaError_t e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        delete m;
        return cuda_fail(e);
    }
    *out = m;
    return ZQ_OK;
}

int zq_gemma3_set_decode_mode(zq_gemma3* m, int mode) {
    if (!m || mode < ZQ_DECODE_AUTO || mode > ZQ_DECODE_PERSISTENT) return ZQ_ERR_BAD_ARG;
    if (mode == ZQ_DECODE_PERSISTENT && !m->decoder) return ZQ_ERR_UNSUPPORTED;
    m->decode_mode = mode;
    return ZQ_OK;
}

int zq_gemma3_decode_mode(const zq_gemma3* m, int* mode) {
    if (!m || !mode) return ZQ_ERR_BAD_ARG;
    *mode = gemma3_persistent(m) ? ZQ_DECODE_PERSISTENT : ZQ_DECODE_LAUNCH_SEQUENCE;
    return ZQ_OK;
}

int zq_gemma3_profile_step(zq_gemma3* m, uint32_t token, zq_stream stream, long long* h_cycles, uint32_t capacity,
                           uint32_t* n_ctas) {
    if (!m || !h_cycles || !n_ctas || m->n_seq != 1) return ZQ_ERR_BAD_ARG;
    if (!m->decoder) return ZQ_ERR_UNSUPPORTED;
    if (m->seq_len >= m->c.ctx) return ZQ_ERR_SEQUENCE;
    if (token >= m->c.vocab) return ZQ_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    set_state_kernel<<<1, 1, 0, st>>>(m->d_state, token, m->seq_len, 0);
    ZQ_LAUNCH_CHECK();
    int rc = gemma_decoder_profile(m->decoder, DECODE_LOGITS, st, h_cycles, capacity, n_ctas);
    if (rc != ZQ_OK) return rc;
    m->seq_len += 1;
    m->seq_lens[0] = m->seq_len;
    return ZQ_OK;
}

int zq_gemma3_free(zq_gemma3* m) {
    delete m;
    return ZQ_OK;
}

int zq_gemma3_reset_cache(zq_gemma3* m) {
    if (!m) return ZQ_ERR_BAD_ARG;
    m->seq_len = 0;
    std::fill(m->seq_lens.begin(), m->seq_lens.end(), 0u);  // every sequence of a batch engine restarts
    return ZQ_OK;
}

int zq_gemma3_seq_len(const zq_gemma3* m, uint32_t* seq_len) {
    if (!m || !seq_len) return ZQ_ERR_BAD_ARG;
    *seq_len = m->seq_len;
    return ZQ_OK;
}

int zq_gemma3_prefill(zq_gemma3* m, const uint32_t* h_tokens, uint32_t n, zq_stream stream,
                      const float** d_logits) {
    return zq_gemma3_prefill_seq(m, 0, h_tokens, n, stream, d_logits);
}

int zq_gemma3_prefill_seq(zq_gemma3* m, uint32_t seq, const uint32_t* h_tokens, uint32_t n, zq_stream stream,
                          const float** d_logits) {
    if (!m || !h_tokens || !d_logits || seq >= m->n_seq) return ZQ_ERR_BAD_ARG;
    if (n == 0 || n > m->c.ctx) return ZQ_ERR_SEQUENCE;
    for (uint32_t t = 0; t < n; ++t)
        if (h_tokens[t] >= m->c.vocab) return ZQ_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    m->seq_lens[seq] = 0;
    if (seq == 0) m->seq_len = 0;
    // chunks of up to max_rows tokens, each a batched forward pass (every row = the arithmetic of a decode step)
    const uint32_t chunk = m->c.ctx < 128 ? m->c.ctx : 128;
    for (uint32_t t0 = 0; t0 < n; t0 += chunk) {
        const uint32_t T = n - t0 < chunk ? n - t0 : chunk;
        const bool last = t0 + T == n;
        set_state_kernel<<<1, 1, 0, st>>>(m->d_state, h_tokens[t0], t0, 0);
        ZQ_LAUNCH_CHECK();
        int rc;
        if (T == 1 && m->n_seq == 1) {
            rc = gemma3_run(m, last ? STEP_LOGITS : STEP_CACHE_ONLY, st);
        } else if (T == 1) {
            rc = gemma3_forward(m, 1, last ? STEP_LOGITS : STEP_CACHE_ONLY, st, seq);
        } else {
            ZQ_CUDA(cudaMemcpyAsync(m->d_tokens, h_tokens + t0, T * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
            rc = gemma3_forward(m, T, last ? STEP_LOGITS : STEP_CACHE_ONLY, st, seq);
            ZQ_CUDA(cudaStreamSynchronize(st));  // h_tokens is the caller's memory
        }
        if (rc != ZQ_OK) return rc;
    }
    m->seq_lens[seq] = n;
    if (seq == 0) m->seq_len = n;
    *d_logits = m->logits;
    return ZQ_OK;
}

int zq_gemma3_seq_len_of(const zq_gemma3* m, uint32_t seq, uint32_t* seq_len) {
    if (!m || !seq_len || seq >= m->n_seq) return ZQ_ERR_BAD_ARG;
    *seq_len = m->seq_lens[seq];
    return ZQ_OK;
}

// One decode step for every sequence at once: row r = sequence r, its next token h_tokens[r] at its own
// position; the linears run as exact int8 GEMMs over the n_seq rows. Logits: [n_seq][vocab].
int zq_gemma3_decode_next_batch(zq_gemma3* m, const uint32_t* h_tokens, zq_stream stream, const float** d_logits) {
    if (!m || !h_tokens || !d_logits || m->n_seq < 2) return ZQ_ERR_BAD_ARG;
    for (uint32_t r = 0; r < m->n_seq; ++r) {
        if (h_tokens[r] >= m->c.vocab) return ZQ_ERR_BAD_ARG;
        if (m->seq_lens[r] >= m->c.ctx) return ZQ_ERR_SEQUENCE;
    }
    cudaStream_t st = as_stream(stream);
    ZQ_CUDA(cudaMemcpyAsync(m->d_tokens, h_tokens, m->n_seq * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
    ZQ_CUDA(cudaMemcpyAsync(m->d_pos, m->seq_lens.data(), m->n_seq * sizeof(uint32_t), cudaMemcpyHostToDevice, st));
    ZQ_CUDA(cudaStreamSynchronize(st));  // both sources are host memory that changes below / belongs to the caller
    // tokens and positions live in device memory: the launch sequence is the same every step and is replayed
    int rc = m->graphs.run(STEP_BATCH, st, [&](cudaStream_t s2) { return gemma3_forward(m, m->n_seq, STEP_LOGITS, s2, 0, true); });
    if (rc != ZQ_OK) return rc;
    for (uint32_t r = 0; r < m->n_seq; ++r) m->seq_lens[r] += 1;
    m->seq_len = m->seq_lens[0];
    *d_logits = m->logits_batch;
    return ZQ_OK;
}

int zq_gemma3_decode_next(zq_gemma3* m, uint32_t token, zq_stream stream, const float** d_logits) {
    if (!m || !d_logits || m->n_seq != 1) return ZQ_ERR_BAD_ARG;
    if (m->seq_len >= m->c.ctx) return ZQ_ERR_SEQUENCE;
    if (token >= m->c.vocab) return ZQ_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    set_state_kernel<<<1, 1, 0, st>>>(m->d_state, token, m->seq_len, 0);
    ZQ_LAUNCH_CHECK();
    int rc = gemma3_run(m, STEP_LOGITS, st);
    if (rc != ZQ_OK) return rc;
    m->seq_len += 1;
    m->seq_lens[0] = m->seq_len;
    *d_logits = m->logits;
    return ZQ_OK;
}

int zq_gemma3_decode_greedy(zq_gemma3* m, uint32_t first_token, uint32_t n_steps, zq_stream stream,
                            uint32_t* h_tokens_out) {
    if (!m || !h_tokens_out || m->n_seq != 1) return ZQ_ERR_BAD_ARG;
    if (n_steps == 0) return ZQ_OK;
    if ((uint64_t)m->seq_len + n_steps > m->c.ctx) return ZQ_ERR_SEQUENCE;
    if (first_token >= m->c.vocab) return ZQ_ERR_BAD_ARG;
    cudaStream_t st = as_stream(stream);
    set_state_kernel<<<1, 1, 0, st>>>(m->d_state, first_token, m->seq_len, 0);
    ZQ_LAUNCH_CHECK();
    if (gemma3_persistent(m)) {  // every step inside one launch: the argmax feeds the next token on the device
        int rc = gemma_decoder_run(m->decoder, n_steps, DECODE_GREEDY, st);
        if (rc != ZQ_OK) return rc;
        m->seq_len += n_steps;
        m->seq_lens[0] = m->seq_len;
    } else {
        for (uint32_t s = 0; s < n_steps; ++s) {
            int rc = gemma3_run(m, STEP_GREEDY, st);
            if (rc != ZQ_OK) return rc;
            m->seq_len += 1;
            m->seq_lens[0] = m->seq_len;
        }
    }
    ZQ_CUDA(cudaMemcpyAsync(h_tokens_out, m->d_record, n_steps * sizeof(uint32_t),
                            cudaMemcpyDeviceToHost, st));
    ZQ_CUDA(cudaStreamSynchronize(st));
    return ZQ_OK;
}

}  // extern "C"
