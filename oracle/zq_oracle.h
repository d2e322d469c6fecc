/*
 * zq_oracle.h — CPU restatement of zig-nn's quantised-inference path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links, loads or calls this
 * code; it exists so the tests, the smoke check and the benchmark's CPU-baseline leg have
 * an independent statement of the arithmetic to compare the CUDA kernels against.
 *
 * The reference is Zig 0.16 and cannot be compiled where this repository is built, so
 * each function restates the Zig source it cites (paths inside the zig-nn tree). The
 * block-level functions are pinned by the reference's own in-file known-answer tests
 * (see tests/test_oracle_kat.py); model-level outputs are not pinned by any reference
 * test or fixture ("parity unpinned" above the block level).
 *
 * Floating-point conventions kept from the reference:
 *   - SIMD vector length `vl` = 16 f32 lanes (std.simd.suggestVectorLength on an AVX-512
 *     host); lane accumulators, then an in-order reduction lane 0..15.
 *   - mul and add are separate roundings (build with -ffp-contract=off).
 *   - round() is round-half-away-from-zero (std.math.round).
 *   - exp / tanh / cos / sin are computed in double and rounded once to f32 (see ops.cpp); the
 *     reference's own f32 routines may differ from that in the last bit.
 */
#ifndef ZQ_ORACLE_H
#define ZQ_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#include "../include/zq.h" /* zq_type ids and the model weight structs */

#ifdef __cplusplus
extern "C" {
#endif

/* Q8Block — src/gguf/simd_dot.zig:17-21 */
typedef struct zqo_q8_block {
    int8_t q[32];
    float scale;
    int32_t sum;
} zqo_q8_block;

/* block geometry — src/gguf/dequant.zig:23-61 */
size_t zqo_block_size(int type);
size_t zqo_bytes_per_block(int type);
size_t zqo_tensor_bytes(int type, size_t num_elements);

/* f16 <-> f32 (IEEE binary16, round-to-nearest-even on narrowing) */
float zqo_f16_to_f32(uint16_t h);
uint16_t zqo_f32_to_f16(float f);

/* Encoders. The reference has no weight quantiser in library code; these produce the test
 * inputs and never take part in a parity comparison (both sides read the same bytes).
 *   q4_0: d = signed-absmax / -8, q = clamp(round(x/d) + 8, 0, 15)    (benchmark config text)
 *   q8_0: scale = absmax/127, q = round(x/scale) clamped to [-128,127]
 *         (test-local encoder, src/diff/mps_runtime_test.zig:649-674)
 *   q4_1: m = min, d = (max-min)/15, q = clamp(round((x-m)/d), 0, 15)  (from the decode rule,
 *         src/gguf/dequant.zig:191-207) */
void zqo_quantize_q4_0(const float* x, uint8_t* out, size_t n);
void zqo_quantize_q4_1(const float* x, uint8_t* out, size_t n);
void zqo_quantize_q8_0(const float* x, uint8_t* out, size_t n);
int zqo_quantize(int type, const float* x, uint8_t* out, size_t n);

/* dequantize — src/gguf/dequant.zig:68-123,191-207,406-420. Returns non-zero for an
 * unsupported type (error.UnsupportedQuantType). */
int zqo_dequantize(int type, const uint8_t* src, float* dst, size_t n);

/* f32-activation dots and matmuls — src/gguf/dequant.zig:133-309 */
float zqo_dot_f32(int type, const uint8_t* row, const float* x, size_t in_dim);
int zqo_matmul_f32(int type, const uint8_t* w, const float* x, float* y, size_t out_dim,
                   size_t in_dim, int n_threads);

/* Q8 activation path — src/gguf/simd_dot.zig:25-152, src/gguf/thread_pool.zig:96-181.
 * zqo_matmul_q8 returns non-zero when in_dim > 8192 (MAX_Q8_BLOCKS, thread_pool.zig:21) unless
 * allow_long is set (the limit is a buffer size in the reference, not part of the arithmetic). */
void zqo_quantize_row_q8(const float* x, zqo_q8_block* out, size_t n);
float zqo_dot_q8(int type, const uint8_t* row, const zqo_q8_block* xq, size_t n_blocks);
int zqo_matmul_q8(int type, const uint8_t* w, const float* x, float* y, size_t out_dim,
                  size_t in_dim, int n_threads, int allow_long);

/* Batched rows: y[m] = matmul(x[m]) for m in 0..m_rows, the way linear_forward_q loops
 * (src/models/gpt2.zig:640-686, src/models/gemma3.zig:889-901). act_mode: 0 f32, 1 q8. */
/* grad_x[m][k] (+)= sum_j grad_out[m][j] * W[j][k] (nn_training_kernels.metal:1149-1242) */
int zqo_matmul_transposed(int type, const uint8_t* w, const float* grad_out, float* grad_x, size_t m_rows,
                          size_t out_dim, size_t in_dim, int accumulate, int n_threads);
int zqo_linear(int type, const uint8_t* w, const float* x, float* y, size_t m_rows,
               size_t out_dim, size_t in_dim, int act_mode, int n_threads);

/* small ops */
void zqo_layer_norm_rows(const float* x, const float* w, const float* b, float* out, size_t rows,
                         size_t dim); /* gpt2.zig:541-596, eps 1e-5 */
void zqo_layer_norm_forward(const float* x, float* out, const float* gamma, const float* beta,
                            size_t rows, size_t dim, float eps); /* runtime_kernels.zig:148-213 */
void zqo_rms_norm_rows(const float* x, const float* w, float* out, size_t rows, size_t dim,
                       float eps);                                  /* gemma3.zig:906-946 */
void zqo_rms_norm_in_place(float* x, const float* w, size_t dim, float eps); /* gemma3.zig:949-959 */
void zqo_gelu_in_place(float* x, size_t n);           /* gpt2.zig:690-697, gemma3.zig:1148-1155 */
void zqo_softmax_gpt2(float* x, size_t n);            /* gpt2.zig:700-731 */
void zqo_softmax_gemma(float* x, size_t n);           /* gemma3.zig:1158-1172 */
void zqo_softmax_forward(float* data, size_t rows, size_t cols); /* runtime_kernels.zig:40-81 */
void zqo_rope_freqs(size_t head_dim, float base, float* freqs); /* gemma3.zig:1128-1135 */
void zqo_rope(float* x, size_t pos, const float* freqs, size_t n_freqs); /* gemma3.zig:962-973 */
uint32_t zqo_argmax(const float* logits, size_t n);   /* gpt2.zig:980-990 */
void zqo_cached_attention(const float* q, const float* k_cache, const float* v_cache, float* out,
                          float* scores, size_t kv_len, size_t n_head, size_t head_dim,
                          size_t embed); /* gpt2.zig:796-849 */
void zqo_causal_self_attention(const float* qkv, float* out, float* scores, size_t seq_len,
                               size_t n_head, size_t head_dim, size_t embed); /* gpt2.zig:736-792 */
void zqo_gqa_cached_attention(const float* q, const float* k_cache, const float* v_cache,
                              float* out, float* scores, size_t kv_start, size_t kv_end,
                              size_t n_head, size_t head_dim, size_t q_dim,
                              size_t kv_dim); /* gemma3.zig:1062-1120 */
void zqo_gqa_causal_attention_prefill(const float* q, const float* k_cache, const float* v_cache,
                                      float* out, size_t seq_len, size_t n_head, size_t head_dim,
                                      size_t q_dim, size_t kv_dim,
                                      size_t window); /* gemma3.zig:992-1059 */

/* models: gpt2(C) (gpt2.zig:198-532) and gemma3(C) (gemma3.zig:243-848). Weight pointers are
 * borrowed and must outlive the model. Logits buffers are owned by the model. */
typedef struct zqo_gpt2 zqo_gpt2;
typedef struct zqo_gemma3 zqo_gemma3;

/* n_threads only splits output rows of the linears; results do not depend on it. The reference
 * runs GPT-2 on one thread and Gemma-3 on min(cpu_count, 8) (gemma3.zig:285-286). */
zqo_gpt2* zqo_gpt2_create(const zq_gpt2_config* cfg, const zq_gpt2_weights* w, int n_threads);
void zqo_gpt2_free(zqo_gpt2* m);
int zqo_gpt2_prefill(zqo_gpt2* m, const uint32_t* tokens, size_t n, const float** logits);
int zqo_gpt2_decode_next(zqo_gpt2* m, uint32_t token, const float** logits);

zqo_gemma3* zqo_gemma3_create(const zq_gemma3_config* cfg, const zq_gemma3_weights* w,
                              int n_threads);
void zqo_gemma3_free(zqo_gemma3* m);
int zqo_gemma3_prefill(zqo_gemma3* m, const uint32_t* tokens, size_t n, const float** logits);
int zqo_gemma3_decode_next(zqo_gemma3* m, uint32_t token, const float** logits);

#ifdef __cplusplus
}
#endif
#endif
