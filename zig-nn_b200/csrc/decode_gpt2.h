// Host interface of the persistent GPT-2 decode kernel (decode_gpt2.cu), used by the engine.
#pragma once

#include <vector>

#include "decode_gemma.h"  // DECODE_CACHE_ONLY / DECODE_LOGITS / DECODE_GREEDY
#include "zq_internal.h"

namespace zq {

struct GptDecoderLayer {
    const zq_weight *qkv, *proj, *fc, *mproj;             // quantised (q4_0 / q4_1 / q8_0)
    const float *qkv_b, *proj_b, *fc_b, *mproj_b;         // biases
    const float *ln1_w, *ln1_b, *ln2_w, *ln2_b;
    float *kc, *vc;                                       // [ctx][embed]
};

struct GptDecoderDesc {
    uint32_t embed, n_head, ffn, ctx, vocab;
    float eps;
    const float *wte, *wpe, *ln_f_w, *ln_f_b;             // wte doubles as the f32 vocabulary head
    std::vector<GptDecoderLayer> layers;
    // engine-owned device buffers: logits [vocab]; state [3] = token, position, record index; record [ctx]
    float* logits;
    uint32_t *state, *record;
};

struct GptDecoder;

// ZQ_ERR_UNSUPPORTED when the model does not fit the kernel's plan (the engine then keeps its launch sequence).
int gpt_decoder_create(const GptDecoderDesc& desc, GptDecoder** out);
void gpt_decoder_free(GptDecoder* d);
// n_steps tokens in one launch; the token, its position and the record index are read from state[0..2];
// DECODE_GREEDY feeds each argmax back as the next token and appends it to the record.
int gpt_decoder_run(GptDecoder* d, uint32_t n_steps, int variant, cudaStream_t st);

}  // namespace zq
