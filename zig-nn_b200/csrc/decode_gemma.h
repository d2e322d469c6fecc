// Host interface of the persistent Gemma-3 decode kernel (decode_gemma.cu), used by the engine.
#pragma once

#include <vector>

#include "zq_internal.h"

namespace zq {

enum { DECODE_CACHE_ONLY = 0, DECODE_LOGITS = 1, DECODE_GREEDY = 2 };

struct GemmaDecoderLayer {
    const zq_weight *qkv, *o, *gate_up, *down;  // q|k|v rows stacked; gate rows then up rows stacked
    const float *attn_norm_w, *post_attn_norm_w, *q_norm_w, *k_norm_w, *ffn_norm_w, *post_ffw_norm_w;
    float *kc, *vc;   // [ctx][n_kv * head_dim]
    uint32_t window;  // 0: global layer
};

struct GemmaDecoderDesc {
    uint32_t embed, head_dim, n_head, n_kv, ffn, ctx;
    float eps, embed_scale;
    const zq_weight* token_embd;
    const float* output_norm_w;
    const float* freqs;
    std::vector<GemmaDecoderLayer> layers;
    // engine-owned device buffers: logits [vocab]; state [3] = token, position, record index; record [ctx]
    float* logits;
    uint32_t *state, *record;
    uint32_t slot_bytes = 0, n_slots = 0;  // 0: chosen by the decoder
    uint32_t deal_limit = 0;               // units per CTA and phase up to which all warps share every unit (0: default)
};

struct GemmaDecoder;

// ZQ_ERR_UNSUPPORTED when the model does not fit the kernel's plan (the engine then keeps its launch
// sequence): a row larger than a ring slot, head groups that do not divide 16 warps, no cooperative launch.
int gemma_decoder_create(const GemmaDecoderDesc& desc, GemmaDecoder** out);
void gemma_decoder_free(GemmaDecoder* d);
// n_steps tokens in one launch. The token, its position and the record index are read from state[0..2];
// DECODE_GREEDY feeds each argmax back as the next token and appends it to the record.
int gemma_decoder_run(GemmaDecoder* d, uint32_t n_steps, int variant, cudaStream_t st);
// One step with per-CTA cycle stamps at the phase boundaries (token start; ten per layer; two for the head);
// h_out[grid][cap], *n_ctas = grid.
int gemma_decoder_profile(GemmaDecoder* d, int variant, cudaStream_t st, long long* h_out, uint32_t cap,
                          uint32_t* n_ctas);
uint32_t gemma_decoder_grid(const GemmaDecoder* d);

}  // namespace zq
