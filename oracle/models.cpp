// CPU restatement of zig-nn's GPT-2 and Gemma-3 inference loops (prefill + decode_next).
// Test infrastructure only — see zq_oracle.h.
#include <cmath>
#include <cstring>
#include <vector>

#include "zq_oracle.h"

namespace {

constexpr size_t VL = 16;

inline void add_in_place(float* a, const float* b, size_t n) {
    for (size_t i = 0; i < n; ++i) a[i] += b[i];
}
inline void mul_in_place(float* a, const float* b, size_t n) {
    for (size_t i = 0; i < n; ++i) a[i] *= b[i];
}

// gpt2.linear_forward_q (gpt2.zig:632-686): per input row the f32-activation matmul, then + bias.
void gpt2_linear(const float* x, const zq_tensor_ref& w, const float* bias, float* y, size_t rows,
                 int n_threads) {
    for (size_t r = 0; r < rows; ++r) {
        float* yr = y + r * w.out_dim;
        zqo_matmul_f32(w.type, (const uint8_t*)w.data, x + r * w.in_dim, yr, w.out_dim, w.in_dim,
                       n_threads);
        for (size_t j = 0; j < w.out_dim; ++j) yr[j] += bias[j];
    }
}

// gemma3.linear_forward_q (gemma3.zig:875-902): per input row ThreadPool.matmul, no bias.
void gemma_linear(const float* x, const zq_tensor_ref& w, float* y, size_t rows, int n_threads) {
    for (size_t r = 0; r < rows; ++r)
        zqo_matmul_q8(w.type, (const uint8_t*)w.data, x + r * w.in_dim, y + r * w.out_dim,
                      w.out_dim, w.in_dim, n_threads, 1);
}

}  // namespace

struct zqo_gpt2 {
    zq_gpt2_config c;
    const zq_gpt2_weights* w;
    int n_threads;
    std::vector<std::vector<float>> k, v;  // per layer [ctx][embed]
    size_t seq_len;
    std::vector<float> logits;
};

struct zqo_gemma3 {
    zq_gemma3_config c;
    const zq_gemma3_weights* w;
    int n_threads;
    std::vector<std::vector<float>> k, v;  // per layer [ctx][kv_dim]
    std::vector<float> freqs;
    size_t seq_len;
    std::vector<float> logits;
};

extern "C" {

// ------------------------------------------------------------------ GPT-2

zqo_gpt2* zqo_gpt2_create(const zq_gpt2_config* cfg, const zq_gpt2_weights* w, int n_threads) {
    zqo_gpt2* m = new zqo_gpt2;
    m->c = *cfg;
    m->w = w;
    m->n_threads = n_threads > 0 ? n_threads : 1;
    m->k.assign(cfg->layer, std::vector<float>((size_t)cfg->ctx * cfg->embed, 0.0f));
    m->v.assign(cfg->layer, std::vector<float>((size_t)cfg->ctx * cfg->embed, 0.0f));
    m->seq_len = 0;
    m->logits.resize(cfg->vocab);
    return m;
}

void zqo_gpt2_free(zqo_gpt2* m) { delete m; }

// compute_logits (gpt2.zig:512-531): f32 dot of the hidden row with every wte row.
static void gpt2_logits(zqo_gpt2* m, const float* hidden) {
    const size_t E = m->c.embed;
    const float* wte = m->w->wte;
#pragma omp parallel for schedule(static) num_threads(m->n_threads)
    for (long v = 0; v < (long)m->c.vocab; ++v) {
        const float* row = wte + (size_t)v * E;
        float acc[VL];
        for (size_t l = 0; l < VL; ++l) acc[l] = 0.0f;
        size_t i = 0;
        for (; i + VL <= E; i += VL)
            for (size_t l = 0; l < VL; ++l) acc[l] += hidden[i + l] * row[i + l];
        float s = acc[0];
        for (size_t l = 1; l < VL; ++l) s += acc[l];
        for (; i < E; ++i) s += hidden[i] * row[i];
        m->logits[v] = s;
    }
}

int zqo_gpt2_prefill(zqo_gpt2* m, const uint32_t* tokens, size_t n, const float** logits) {
    const zq_gpt2_config& C = m->c;
    if (n == 0) return ZQ_ERR_SEQUENCE;
    if (n > C.ctx) return ZQ_ERR_SEQUENCE;
    const size_t E = C.embed, F = C.ffn, hd = E / C.head;
    m->seq_len = 0;
    std::vector<float> x(n * E), ln(n * E), qkv(n * 3 * E), att(n * E), proj(n * E), hid(n * F),
        mlp(n * E), scores(n);
    for (size_t t = 0; t < n; ++t)
        for (size_t i = 0; i < E; ++i)
            x[t * E + i] = m->w->wte[(size_t)tokens[t] * E + i] + m->w->wpe[t * E + i];
    for (size_t l = 0; l < C.layer; ++l) {  // prefill_layer, gpt2.zig:357-420
        const zq_gpt2_block& b = m->w->blocks[l];
        zqo_layer_norm_rows(x.data(), b.ln1_weight, b.ln1_bias, ln.data(), n, E);
        gpt2_linear(ln.data(), b.attn_qkv_weight, b.attn_qkv_bias, qkv.data(), n, m->n_threads);
        for (size_t t = 0; t < n; ++t) {
            memcpy(&m->k[l][t * E], &qkv[t * 3 * E + E], E * sizeof(float));
            memcpy(&m->v[l][t * E], &qkv[t * 3 * E + 2 * E], E * sizeof(float));
        }
        zqo_causal_self_attention(qkv.data(), att.data(), scores.data(), n, C.head, hd, E);
        gpt2_linear(att.data(), b.attn_proj_weight, b.attn_proj_bias, proj.data(), n,
                    m->n_threads);
        add_in_place(x.data(), proj.data(), n * E);
        zqo_layer_norm_rows(x.data(), b.ln2_weight, b.ln2_bias, ln.data(), n, E);
        gpt2_linear(ln.data(), b.mlp_fc_weight, b.mlp_fc_bias, hid.data(), n, m->n_threads);
        zqo_gelu_in_place(hid.data(), n * F);
        gpt2_linear(hid.data(), b.mlp_proj_weight, b.mlp_proj_bias, mlp.data(), n, m->n_threads);
        add_in_place(x.data(), mlp.data(), n * E);
    }
    m->seq_len = n;
    // The reference normalises every row and keeps the last; rows are independent.
    zqo_layer_norm_rows(&x[(n - 1) * E], m->w->ln_f_weight, m->w->ln_f_bias, ln.data(), 1, E);
    gpt2_logits(m, ln.data());
    *logits = m->logits.data();
    return ZQ_OK;
}

int zqo_gpt2_decode_next(zqo_gpt2* m, uint32_t token, const float** logits) {
    const zq_gpt2_config& C = m->c;
    const size_t pos = m->seq_len;
    if (pos >= C.ctx) return ZQ_ERR_SEQUENCE;
    const size_t E = C.embed, F = C.ffn, hd = E / C.head;
    std::vector<float> x(E), ln(E), qkv(3 * E), att(E), proj(E), hid(F), mlp(E), scores(pos + 1);
    for (size_t i = 0; i < E; ++i)
        x[i] = m->w->wte[(size_t)token * E + i] + m->w->wpe[pos * E + i];
    for (size_t l = 0; l < C.layer; ++l) {  // gpt2.zig:464-504
        const zq_gpt2_block& b = m->w->blocks[l];
        zqo_layer_norm_rows(x.data(), b.ln1_weight, b.ln1_bias, ln.data(), 1, E);
        gpt2_linear(ln.data(), b.attn_qkv_weight, b.attn_qkv_bias, qkv.data(), 1, m->n_threads);
        memcpy(&m->k[l][pos * E], &qkv[E], E * sizeof(float));
        memcpy(&m->v[l][pos * E], &qkv[2 * E], E * sizeof(float));
        zqo_cached_attention(qkv.data(), m->k[l].data(), m->v[l].data(), att.data(),
                             scores.data(), pos + 1, C.head, hd, E);
        gpt2_linear(att.data(), b.attn_proj_weight, b.attn_proj_bias, proj.data(), 1,
                    m->n_threads);
        add_in_place(x.data(), proj.data(), E);
        zqo_layer_norm_rows(x.data(), b.ln2_weight, b.ln2_bias, ln.data(), 1, E);
        gpt2_linear(ln.data(), b.mlp_fc_weight, b.mlp_fc_bias, hid.data(), 1, m->n_threads);
        zqo_gelu_in_place(hid.data(), F);
        gpt2_linear(hid.data(), b.mlp_proj_weight, b.mlp_proj_bias, mlp.data(), 1, m->n_threads);
        add_in_place(x.data(), mlp.data(), E);
    }
    m->seq_len = pos + 1;
    zqo_layer_norm_rows(x.data(), m->w->ln_f_weight, m->w->ln_f_bias, ln.data(), 1, E);
    gpt2_logits(m, ln.data());
    *logits = m->logits.data();
    return ZQ_OK;
}

// ------------------------------------------------------------------ Gemma-3

zqo_gemma3* zqo_gemma3_create(const zq_gemma3_config* cfg, const zq_gemma3_weights* w,
                              int n_threads) {
    zqo_gemma3* m = new zqo_gemma3;
    m->c = *cfg;
    m->w = w;
    m->n_threads = n_threads > 0 ? n_threads : 1;
    const size_t kv_dim = (size_t)cfg->head_kv * cfg->head_dim;
    m->k.assign(cfg->layer, std::vector<float>((size_t)cfg->ctx * kv_dim, 0.0f));
    m->v.assign(cfg->layer, std::vector<float>((size_t)cfg->ctx * kv_dim, 0.0f));
    m->freqs.resize(cfg->head_dim / 2);
    zqo_rope_freqs(cfg->head_dim, cfg->rope_base, m->freqs.data());
    m->seq_len = 0;
    m->logits.resize(cfg->vocab);
    return m;
}

void zqo_gemma3_free(zqo_gemma3* m) { delete m; }

static inline bool gemma_is_global(const zq_gemma3_config& C, size_t layer) {
    return (layer % C.global_every) == (size_t)C.global_every - 1;  // gemma3.zig:1123-1125
}

// dequant_row (gemma3.zig:855-871) followed by the sqrt(EMBED) scale (gemma3.zig:353-356).
static void gemma_embed(const zqo_gemma3* m, uint32_t token, float* dst) {
    const zq_tensor_ref& t = m->w->token_embd;
    const size_t row_bytes = zqo_tensor_bytes(t.type, t.in_dim);
    zqo_dequantize(t.type, (const uint8_t*)t.data + (size_t)token * row_bytes, dst, t.in_dim);
    const float s = std::sqrt((float)m->c.embed);
    for (size_t i = 0; i < t.in_dim; ++i) dst[i] *= s;
}

int zqo_gemma3_prefill(zqo_gemma3* m, const uint32_t* tokens, size_t n, const float** logits) {
    const zq_gemma3_config& C = m->c;
    if (n == 0) return ZQ_ERR_SEQUENCE;
    if (n > C.ctx) return ZQ_ERR_SEQUENCE;
    const size_t E = C.embed, F = C.ffn, D = C.head_dim;
    const size_t QD = (size_t)C.head * D, KD = (size_t)C.head_kv * D;
    const int T = m->n_threads;
    m->seq_len = 0;
    std::vector<float> x(n * E), h(n * E), q(n * QD), k(n * KD), v(n * KD), att(n * QD),
        proj(n * E), gate(n * F), up(n * F), ffn(n * E), nrm(n * E);
    for (size_t t = 0; t < n; ++t) gemma_embed(m, tokens[t], &x[t * E]);
    for (size_t l = 0; l < C.layer; ++l) {
        const zq_gemma3_block& b = m->w->blocks[l];
        // prefill_attention_block, gemma3.zig:407-455
        zqo_rms_norm_rows(x.data(), b.attn_norm_weight, h.data(), n, E, C.rms_eps);
        gemma_linear(h.data(), b.attn_q_weight, q.data(), n, T);
        gemma_linear(h.data(), b.attn_k_weight, k.data(), n, T);
        gemma_linear(h.data(), b.attn_v_weight, v.data(), n, T);
        for (size_t t = 0; t < n; ++t) {  // prefill_qk_norm_rope, gemma3.zig:361-404
            for (size_t hd = 0; hd < C.head; ++hd)
                zqo_rms_norm_in_place(&q[t * QD + hd * D], b.attn_q_norm_weight, D, C.rms_eps);
            zqo_rms_norm_in_place(&k[t * KD], b.attn_k_norm_weight, D, C.rms_eps);
            for (size_t hd = 0; hd < C.head; ++hd)
                zqo_rope(&q[t * QD + hd * D], t, m->freqs.data(), D / 2);
            zqo_rope(&k[t * KD], t, m->freqs.data(), D / 2);
            memcpy(&m->k[l][t * KD], &k[t * KD], KD * sizeof(float));
            memcpy(&m->v[l][t * KD], &v[t * KD], KD * sizeof(float));
        }
        const size_t window = gemma_is_global(C, l) ? n : C.sliding_window;
        zqo_gqa_causal_attention_prefill(q.data(), m->k[l].data(), m->v[l].data(), att.data(), n,
                                         C.head, D, QD, KD, window);
        gemma_linear(att.data(), b.attn_output_weight, proj.data(), n, T);
        zqo_rms_norm_rows(proj.data(), b.post_attention_norm_weight, nrm.data(), n, E, C.rms_eps);
        add_in_place(x.data(), nrm.data(), n * E);
        // prefill_ffn_block, gemma3.zig:495-535
        zqo_rms_norm_rows(x.data(), b.ffn_norm_weight, h.data(), n, E, C.rms_eps);
        gemma_linear(h.data(), b.ffn_gate_weight, gate.data(), n, T);
        zqo_gelu_in_place(gate.data(), n * F);
        gemma_linear(h.data(), b.ffn_up_weight, up.data(), n, T);
        mul_in_place(gate.data(), up.data(), n * F);
        gemma_linear(gate.data(), b.ffn_down_weight, ffn.data(), n, T);
        zqo_rms_norm_rows(ffn.data(), b.post_ffw_norm_weight, nrm.data(), n, E, C.rms_eps);
        add_in_place(x.data(), nrm.data(), n * E);
    }
    m->seq_len = n;
    zqo_rms_norm_rows(&x[(n - 1) * E], m->w->output_norm_weight, h.data(), 1, E, C.rms_eps);
    const zq_tensor_ref& te = m->w->token_embd;  // compute_logits, gemma3.zig:830-846
    zqo_matmul_q8(te.type, (const uint8_t*)te.data, h.data(), m->logits.data(), C.vocab, E, T, 1);
    *logits = m->logits.data();
    return ZQ_OK;
}

int zqo_gemma3_decode_next(zqo_gemma3* m, uint32_t token, const float** logits) {
    const zq_gemma3_config& C = m->c;
    const size_t pos = m->seq_len;
    if (pos >= C.ctx) return ZQ_ERR_SEQUENCE;
    const size_t E = C.embed, F = C.ffn, D = C.head_dim;
    const size_t QD = (size_t)C.head * D, KD = (size_t)C.head_kv * D;
    const int T = m->n_threads;
    std::vector<float> x(E), h(E), q(QD), k(KD), v(KD), att(QD), proj(E), gate(F), up(F), ffn(E),
        nrm(E), scores(pos + 1);
    gemma_embed(m, token, x.data());
    for (size_t l = 0; l < C.layer; ++l) {
        const zq_gemma3_block& b = m->w->blocks[l];
        // decode_attention_block, gemma3.zig:662-731
        zqo_rms_norm_rows(x.data(), b.attn_norm_weight, h.data(), 1, E, C.rms_eps);
        gemma_linear(h.data(), b.attn_q_weight, q.data(), 1, T);
        gemma_linear(h.data(), b.attn_k_weight, k.data(), 1, T);
        gemma_linear(h.data(), b.attn_v_weight, v.data(), 1, T);
        for (size_t hd = 0; hd < C.head; ++hd) {  // decode_qk_norm_rope, gemma3.zig:629-659
            zqo_rms_norm_in_place(&q[hd * D], b.attn_q_norm_weight, D, C.rms_eps);
            zqo_rope(&q[hd * D], pos, m->freqs.data(), D / 2);
        }
        zqo_rms_norm_in_place(k.data(), b.attn_k_norm_weight, D, C.rms_eps);
        zqo_rope(k.data(), pos, m->freqs.data(), D / 2);
        memcpy(&m->k[l][pos * KD], k.data(), KD * sizeof(float));
        memcpy(&m->v[l][pos * KD], v.data(), KD * sizeof(float));
        const size_t kv_len = pos + 1;
        const size_t window =
            gemma_is_global(C, l) ? kv_len : (kv_len < C.sliding_window ? kv_len : C.sliding_window);
        const size_t kv_start = kv_len > window ? kv_len - window : 0;
        zqo_gqa_cached_attention(q.data(), m->k[l].data(), m->v[l].data(), att.data(),
                                 scores.data(), kv_start, kv_len, C.head, D, QD, KD);
        gemma_linear(att.data(), b.attn_output_weight, proj.data(), 1, T);
        zqo_rms_norm_rows(proj.data(), b.post_attention_norm_weight, nrm.data(), 1, E, C.rms_eps);
        add_in_place(x.data(), nrm.data(), E);
        // decode_ffn_block, gemma3.zig:734-773
        zqo_rms_norm_rows(x.data(), b.ffn_norm_weight, h.data(), 1, E, C.rms_eps);
        gemma_linear(h.data(), b.ffn_gate_weight, gate.data(), 1, T);
        zqo_gelu_in_place(gate.data(), F);
        gemma_linear(h.data(), b.ffn_up_weight, up.data(), 1, T);
        mul_in_place(gate.data(), up.data(), F);
        gemma_linear(gate.data(), b.ffn_down_weight, ffn.data(), 1, T);
        zqo_rms_norm_rows(ffn.data(), b.post_ffw_norm_weight, nrm.data(), 1, E, C.rms_eps);
        add_in_place(x.data(), nrm.data(), E);
    }
    zqo_rms_norm_rows(x.data(), m->w->output_norm_weight, h.data(), 1, E, C.rms_eps);
    m->seq_len = pos + 1;
    const zq_tensor_ref& te = m->w->token_embd;
    zqo_matmul_q8(te.type, (const uint8_t*)te.data, h.data(), m->logits.data(), C.vocab, E, T, 1);
    *logits = m->logits.data();
    return ZQ_OK;
}

}  // extern "C"
