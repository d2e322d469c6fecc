/*
 * zq.h — C ABI of libzq: sm_100a CUDA kernels for the GGUF Q4_0 / Q4_1 / Q8_0
 * linear layers (and the small ops between them) that zig-nn runs for GPT-2 and
 * Gemma-3 inference.
 *
 * Conventions
 *   - Every function returns a zq_status (0 = ok). Nothing aborts or throws.
 *   - `stream` is the caller's CUstream / cudaStream_t (NULL = default stream);
 *     kernels are launched asynchronously on it in the current CUDA context and
 *     nothing synchronises unless the comment says so.
 *   - Pointers named d_* are device pointers, h_* are host pointers.
 *   - Quantised weights are row-major [out_dim][in_dim/32 blocks], exactly the
 *     GGUF tensor bytes (src/gguf/dequant.zig:23-61; src/gguf/gguf.zig:155-176).
 *   - Activations and outputs are row-major f32: x [m_rows][in_dim],
 *     y [m_rows][out_dim]  (src/backend/shaders/nn_kernels.metal:491-528).
 *
 * Citations are paths inside the zig-nn source tree.
 */
#ifndef ZQ_H
#define ZQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status */

typedef enum zq_status {
    ZQ_OK = 0,
    ZQ_ERR_BAD_ARG = 1,      /* null pointer, in_dim % 32 != 0, m_rows out of range ... */
    ZQ_ERR_UNSUPPORTED = 2,  /* GGML type other than f32/f16/q4_0/q4_1/q8_0
                                (error.UnsupportedQuantType, src/gguf/dequant.zig:418) */
    ZQ_ERR_CUDA = 3,         /* a CUDA runtime call failed; see zq_last_cuda_error() */
    ZQ_ERR_NO_MEM = 4,
    ZQ_ERR_LIMIT = 5,        /* a documented size limit was exceeded */
    ZQ_ERR_SEQUENCE = 6,     /* empty prompt, prompt longer than ctx, or context full
                                (error.EmptySequence / SequenceTooLong / ContextFull,
                                src/models/gpt2.zig:425-426,445) */
    ZQ_ERR_TIMEOUT = 7,      /* a bounded device-side wait gave up */
    ZQ_ERR_PEER = 8          /* peer (multi-GPU) set-up failed: a peer's buffer or flag pointer is missing */
} zq_status;

const char* zq_status_string(int status);
/* cudaError_t of the most recent failing CUDA call on this thread (0 if none). */
int zq_last_cuda_error(void);
/* ABI version of this header; bumped on incompatible change. */
int zq_abi_version(void);
/* Device-side waits (on async-copy barriers) are bounded; a wait that ran out sets a flag in device
 * memory instead of hanging. *out receives the flag (0 = never happened); clear != 0 resets it.
 * Synchronises the device. */
int zq_device_error(unsigned int* out, int clear);
/* The same as a status: ZQ_ERR_TIMEOUT when a bounded device-side wait has run out since the word was last
 * cleared (the result buffers of that call then hold stale data), ZQ_OK otherwise. Synchronises the device.
 * Callers of the peer exchanges check it at their own synchronisation points. */
int zq_device_check(int clear);
/* Number of polls a device-side wait on a PEER's flag makes before it gives up (zq_peer_gather*,
 * zq_matmul_gather); 0 restores the kernels' own defaults (about a second). Process-wide; takes effect with the
 * next launch. Lets a host fail fast, and lets a test make a wait run out without hanging anything. */
int zq_set_wait_limit(unsigned int polls);
/* The many-row tensor-core GEMM runs on pairs of CTAs (thread-block clusters of two, tcgen05 cta_group::2) where
 * that is the faster form. enabled = 0 keeps it on single CTAs (about 0.8 of the speed), as the library does by
 * itself when a cluster launch is refused; for GPUs partitioned so that pairs of SMs cannot be scheduled, and for
 * tests of that route. Process-wide; default 1. */
int zq_set_cluster_launch(int enabled);

/* GGML tensor type ids — src/gguf/dequant.zig:9-20. */
typedef enum zq_type {
    ZQ_TYPE_F32 = 0,
    ZQ_TYPE_F16 = 1,
    ZQ_TYPE_Q4_0 = 2,
    ZQ_TYPE_Q4_1 = 3,
    ZQ_TYPE_Q8_0 = 8
} zq_type;

/* How the activation row is treated before the dot products.
 *   ZQ_ACT_F32: f32 activations times weights dequantised on the fly — the GPT-2
 *               path (src/models/gpt2.zig:632-686 -> src/gguf/dequant.zig:133-309).
 *               Up to 16 rows per call the activations keep 22 mantissa bits (results agree
 *               with the f32 CPU path to about 1e-7 relative L2). From 49 rows on the call is a
 *               tensor-core GEMM with fp16 operands, as ZQ_ACT_F16: about 3e-4 relative L2
 *               (inside the path's 1e-3 bar), and it NEEDS the workspace of
 *               zq_matmul_workspace_bytes(); without one the call returns ZQ_ERR_BAD_ARG (it is
 *               not served by the slower small-batch kernel behind the caller's back).
 *               17 to 48 rows: zq_matmul_workspace_bytes() is non-zero for matrices of 12 288 rows
 *               and more, and a call that brings that workspace runs the weight-streaming
 *               tensor-core form (fp16 operands, 3e-4, 2-3 x faster); a call without workspace,
 *               or on a smaller matrix, runs passes of the 16-row kernel (1e-7).
 *   ZQ_ACT_Q8 : each activation row is first quantised to 32-wide int8 blocks and
 *               the dots are exact int8 x int8 -> int32 — the Gemma-3 path
 *               (src/gguf/thread_pool.zig:96-160 -> src/gguf/simd_dot.zig:25-152).
 *               Outputs are bit-identical to that CPU path. in_dim <= 16384.
 *   ZQ_ACT_F16: tensor-core path (m_rows >= 1): activations and dequantised weights
 *               are rounded to fp16, products accumulate in f32. Faster for m_rows > 1;
 *               rel-L2 vs. ZQ_ACT_F32 about 3e-4.
 */
typedef enum zq_act_mode { ZQ_ACT_F32 = 0, ZQ_ACT_Q8 = 1, ZQ_ACT_F16 = 2 } zq_act_mode;

typedef void* zq_stream;

/* Block geometry — src/gguf/dequant.zig:23-61. Return 0 for unsupported types. */
size_t zq_block_size(int type);       /* elements per block: 1 or 32 */
size_t zq_bytes_per_block(int type);  /* 4, 2, 18, 20, 34 */
size_t zq_tensor_bytes(int type, size_t num_elements);

/* ------------------------------------------------------------- weights */

/* A quantised weight resident on the device. Counterpart of QuantizedWeight
 * (src/models/gpt2.zig:35-40) / DiffMpsRuntime.QuantWeight (src/diff/mps_runtime.zig:1164-1169).
 * The library owns a re-laid-out device copy (quants 16-byte aligned, scales in their
 * own array); values are unchanged, and zq_weight_download_raw returns the original bytes. */
typedef struct zq_weight zq_weight;

/* Copy raw GGUF bytes from the host and lay them out for the kernels. The host bytes may
 * be freed once the call returns (it synchronises `stream`). Types: q4_0, q4_1, q8_0.
 * Replaces MetalContext.create_buffer_with_data + the borrowed slice in QuantizedWeight
 * (src/models/gemma3_metal.zig:105-108,145-157). */
int zq_weight_upload(const void* h_raw, int type, uint32_t out_dim, uint32_t in_dim,
                     zq_stream stream, zq_weight** out);
/* Same, from raw GGUF bytes that are already on the device (asynchronous on `stream`). */
int zq_weight_from_device(const void* d_raw, int type, uint32_t out_dim, uint32_t in_dim,
                          zq_stream stream, zq_weight** out);
int zq_weight_free(zq_weight* w);
int zq_weight_info(const zq_weight* w, int* type, uint32_t* out_dim, uint32_t* in_dim);
/* Bytes the weight occupies on the device. */
size_t zq_weight_device_bytes(const zq_weight* w);
/* Rebuild the raw GGUF bytes into d_raw (zq_tensor_bytes(type, out_dim*in_dim) bytes). */
int zq_weight_download_raw(const zq_weight* w, void* d_raw, zq_stream stream);

/* dequantize_q4_0 / q4_1 / q8_0 (src/gguf/dequant.zig:88-123,191-207): whole tensor to
 * d_out [out_dim][in_dim] f32. Bit-exact with the CPU code. */
int zq_dequantize(const zq_weight* w, float* d_out, zq_stream stream);
/* dequant_row + scale (src/models/gemma3.zig:800-803,855-871;
 * MetalContext.dispatch_dequant_q8_row_scaled, src/backend/metal.zig:1007): rows picked by
 * d_token_ids[0..n_rows) -> d_out [n_rows][in_dim], each value dequantised then multiplied by
 * `scale` as a separate f32 multiply. */
int zq_dequant_rows_scaled(const zq_weight* w, const int32_t* d_token_ids, uint32_t n_rows,
                           float scale, float* d_out, zq_stream stream);

/* ------------------------------------------------------------- matmul */

/* Optional work fused after the dot products, applied in this order:
 *   v = dot (+ bias[j]) ; if gelu: v = gelu(v) ; if mul: v *= mul[m][j] ; if residual: v += residual[m][j]
 * bias: gpt2.zig:675-684; gelu: gpt2.zig:690-697; mul (GeGLU): gemma3.zig:749-752,
 * nn_kernels.metal:377-388; residual: gpt2.zig:852-863. `residual` and `mul` may alias y. */
typedef struct zq_epilogue {
    const float* d_bias;      /* [out_dim] or NULL */
    int gelu;                 /* 0 / 1 */
    const float* d_mul;       /* [m_rows][out_dim] or NULL */
    const float* d_residual;  /* [m_rows][out_dim] or NULL */
} zq_epilogue;

/* Scratch needed by zq_matmul for (w, m_rows, act_mode); 0 when none is needed. */
size_t zq_matmul_workspace_bytes(const zq_weight* w, uint32_t m_rows, int act_mode);

/* y[m][j] = sum_k x[m][k] * W[j][k] (+ epilogue).
 * Replaces matmul_q4_0_f32 / matmul_q4_1_f32 / matmul_q8_0_f32 (src/gguf/dequant.zig:170-309),
 * ThreadPool.matmul (src/gguf/thread_pool.zig:96-160), MetalContext.dispatch_matmul and
 * dispatch_matmul_batched (src/backend/metal.zig:729-846).
 * m_rows <= 16 runs the bandwidth-bound decode kernels; larger m_rows the tiled kernels.
 * d_workspace: zq_matmul_workspace_bytes() bytes, 256-byte aligned, or NULL when that is 0.
 * d_y may also be page-locked host memory that the device can address (cudaHostAlloc, cudaHostRegister):
 * the kernels only write y (unless an epilogue pointer aliases it), so a caller that wants the result on
 * the host — the reference's matmuls return into host slices — saves the device-to-host copy; the rows
 * leave over PCIe while the weights are still streaming. */
int zq_matmul(const zq_weight* w, const float* d_x, float* d_y, uint32_t m_rows, int act_mode,
              const zq_epilogue* epilogue, void* d_workspace, size_t workspace_bytes,
              zq_stream stream);

/* zq_matmul in ZQ_ACT_Q8 mode without a workspace argument and without any allocation: the scratch
 * for the quantised activations is a fixed 320 KiB array inside the library's device image (every GPU
 * that loads libzq holds it until the process exits). This entry point has no counterpart in the
 * reference. It is for hosts that cannot allocate device memory at call time — a runtime that owns
 * all device memory through its own pool, or a decode loop that must not risk cudaMalloc's implicit
 * synchronisation or an out-of-memory error mid-request.
 *   Limits: m_rows <= 16 and in_dim <= 16384, otherwise ZQ_ERR_LIMIT. Results are bit-identical to
 *   zq_matmul(..., ZQ_ACT_Q8, ...).
 *   First call on a device looks up the array's device address (cudaGetSymbolAddress) with that
 *   device current; make that first call outside any stream capture.
 *   All calls on a device share the one array: calls that may overlap on the GPU (different streams,
 *   no ordering between them) race on it. Calls on one stream are safe. Nothing needs clearing
 *   between calls: each call overwrites every entry it later reads.
 *   Calls no cudaMalloc / cudaFree or other allocating routine. */
int zq_matmul_q8_static(const zq_weight* w, const float* d_x, float* d_y, uint32_t m_rows,
                        const zq_epilogue* epilogue, zq_stream stream);

/* Scratch needed by zq_matmul_transposed for (w, m_rows): the fp16 copy of grad_out and its row scales; for many
 * rows on a large matrix also W^T as fp16 tiles (2 bytes per weight), which that form lays out on every call. */
size_t zq_matmul_transposed_workspace_bytes(const zq_weight* w, uint32_t m_rows);

/* grad_x[m][k] (+)= sum_j grad_out[m][j] * W[j][k]: the backward of zq_matmul with respect to its
 * activations, weights decoded on the fly. Replaces matmul_q4_0_trans_batched / matmul_q4_1_trans_batched /
 * matmul_q8_0_trans_batched (src/backend/shaders/nn_training_kernels.metal:1149-1242) behind
 * MetalContext.dispatch_quant_trans_batched, which backward_quant_matmul calls
 * (src/diff/mps_runtime.zig:1212-1230).
 * d_grad_out: [m_rows][out_dim] f32; d_grad_x: [m_rows][in_dim] f32, 8-byte aligned.
 * accumulate != 0 adds to d_grad_x (what the reference's kernels do); 0 overwrites it.
 * out_dim must be a multiple of 8 (ZQ_ERR_UNSUPPORTED otherwise).
 * d_workspace: zq_matmul_transposed_workspace_bytes() bytes, 256-byte aligned.
 * Tensor-core product of fp16 copies (one rounding each for weights and gradients), f32 accumulation:
 * about 3e-4 relative L2 against the f32 statement. On small shapes the sums over the weight rows may be split
 * over CTAs and meet through atomic adds, so the last bits depend on the schedule there; more than 256 rows on a
 * matrix of 1024 weight rows and more run the tcgen05 GEMM on W^T (deterministic). */
int zq_matmul_transposed(const zq_weight* w, const float* d_grad_out, float* d_grad_x, uint32_t m_rows,
                         int accumulate, void* d_workspace, size_t workspace_bytes, zq_stream stream);

/* quantize_row_q8 (src/gguf/simd_dot.zig:25-64) for m_rows rows of in_dim floats.
 * d_q: int8 [m_rows][in_dim]; d_scale: f32 [m_rows][in_dim/32]; d_sum: int32 [m_rows][in_dim/32]. */
int zq_quantize_rows_q8(const float* d_x, uint32_t m_rows, uint32_t in_dim, int8_t* d_q,
                        float* d_scale, int32_t* d_sum, zq_stream stream);

/* f32 weight [out_dim][in_dim] times one f32 row — GPT-2's vocabulary head
 * (compute_logits, src/models/gpt2.zig:512-531). */
int zq_matvec_f32(const float* d_w, const float* d_x, float* d_y, uint32_t out_dim,
                  uint32_t in_dim, zq_stream stream);

/* argmax with first-maximum-wins ties (src/models/gpt2.zig:980-990). Result in d_index[0]. */
int zq_argmax(const float* d_logits, uint32_t n, int32_t* d_index, zq_stream stream);

/* ------------------------------------------------ row sharding over GPUs */

/* All-gather of the output slices of a row-sharded linear over NVLink peer memory. The reference
 * splits a matmul's rows over CPU threads that share one output buffer
 * (ThreadPool.matmul, src/gguf/thread_pool.zig:96-181); across GPUs every rank has its own copy of the
 * output, so after computing y[slice_offset .. slice_offset + slice_len) into its own buffer a rank
 * calls this to copy that range into the same place of every peer's buffer (plain peer stores) and to
 * wait until every peer has done the same for the current round.
 *   h_y_peers[r]    device pointer, valid on this GPU, to rank r's result buffer (entry `rank` = own)
 *   h_flag_peers[r] device pointer, valid on this GPU, to rank r's counters: `world` uint32, zeroed once
 *   round           1, 2, 3, ... — the same value on every rank for the same call, growing by one per call
 * The caller alternates two result buffers between rounds (a peer may run one round ahead). Ranks
 * must reach the call within about a second of each other: the wait is bounded and records a timeout
 * in the word zq_device_error() reads instead of hanging. The two host arrays are read before return. */
int zq_peer_gather(float* const* h_y_peers, uint32_t* const* h_flag_peers, uint32_t world, uint32_t rank,
                   size_t slice_offset, size_t slice_len, uint32_t round, zq_stream stream);

/* The same exchange with the round number kept in device memory (*d_round, zeroed once by the caller,
 * incremented by this call on the stream) and the two alternating result buffers passed together: odd
 * rounds use h_y_peers_odd, even rounds h_y_peers_even. Nothing in the launch depends on host state
 * that changes between calls, so a stream capture that contains an even number of these calls can be
 * replayed. The caller writes its slice into its own odd / even buffer accordingly. */
int zq_peer_gather_step(float* const* h_y_peers_odd, float* const* h_y_peers_even,
                        uint32_t* const* h_flag_peers, uint32_t world, uint32_t rank, size_t slice_offset,
                        size_t slice_len, uint32_t* d_round, zq_stream stream);

/* Several activation rows: this rank owns the columns [col_offset, col_offset + cols) of the row-major
 * [m_rows][n_total] result and holds them as a contiguous [m_rows][cols] block `d_local`. The block is stored to
 * that place of every rank's result buffer (this rank's own included), so each rank ends up with the row-major
 * result itself; counters and rounds as for zq_peer_gather_step (these counters count 32 arrivals per round:
 * give this entry point flags of its own). Result buffers: [m_rows][n_total] floats, odd / even rounds. */
int zq_peer_gather_cols_step(float* const* h_y_peers_odd, float* const* h_y_peers_even,
                             uint32_t* const* h_flag_peers, uint32_t world, uint32_t rank, const float* d_local,
                             uint32_t m_rows, size_t n_total, size_t col_offset, uint32_t cols, uint32_t* d_round,
                             zq_stream stream);

/* One activation row times a row-sharded weight with the exchange inside the GEMV kernel: every output
 * row is stored into this rank's result buffer and, in the same epilogue, into every peer's (plain peer
 * stores), so the all-gather overlaps the weight stream; the grid's last CTA then publishes a counter on
 * every peer and waits (bounded, as above) for theirs. f32 activations.
 *   w            this rank's rows [row_offset, row_offset + out_dim) of the whole matrix
 *   h_y_peers_*  as for zq_peer_gather_step: whole result rows, odd / even rounds
 *   h_flag_peers counters used by this entry point only (`world` uint32 per rank, zeroed once)
 *   d_sync       two uint32 on this GPU, zeroed once: completed rounds, CTA arrivals
 * Returns ZQ_ERR_UNSUPPORTED when the shard has too few rows for this kernel; the caller then uses
 * zq_matmul followed by zq_peer_gather_step. */
int zq_matmul_gather(const zq_weight* w, const float* d_x, const zq_epilogue* epilogue,
                     float* const* h_y_peers_odd, float* const* h_y_peers_even, uint32_t* const* h_flag_peers,
                     uint32_t world, uint32_t rank, uint32_t row_offset, uint32_t* d_sync, zq_stream stream);

/* The same product and exchange with nothing after the peer stores: what travels is one 64-bit word per
 * output row, the round number above the float's bits, stored into the peer's inbox. A word tells by itself
 * whether it belongs to the round, so the sender issues no fence and publishes no counter; each rank's kernel
 * ends by polling (bounded, zq_set_wait_limit) its own inbox for the other ranks' rows and storing the floats
 * into its result row. Every rank owns the same number of rows (w->out_dim, even): rank r's rows are
 * [r * out_dim, (r + 1) * out_dim) of the result.
 *   h_inbox_peers_*  `world` pointers (host array): every rank's inbox of world * out_dim 64-bit words, zeroed
 *                    once, entry `rank` being this GPU's own; odd / even rounds use different inboxes
 *   d_y_*            this GPU's result rows (world * out_dim floats) of odd / even rounds
 *   d_sync           two uint32 on this GPU, zeroed once: completed rounds, CTA arrivals
 * Returns ZQ_ERR_UNSUPPORTED when the shard has too few rows for this kernel or an odd number of them. */
int zq_matmul_gather_tagged(const zq_weight* w, const float* d_x, const zq_epilogue* epilogue,
                            unsigned long long* const* h_inbox_peers_odd, unsigned long long* const* h_inbox_peers_even,
                            float* d_y_odd, float* d_y_even, uint32_t world, uint32_t rank, uint32_t* d_sync,
                            zq_stream stream);

/* Greedy decoding over a (row-sharded) vocabulary head: one activation row times this rank's rows, and only the
 * index of the first largest output over ALL ranks leaves the kernel (argmax of src/models/gpt2.zig:980-990: strict
 * `>`, so the lowest index among equal values; all values NaN or -inf: index 0). Every CTA reduces its rows, the
 * grid's last CTA reduces the CTAs, sends this rank's (value, row) to every peer as two 64-bit words carrying the
 * round number (16 bytes per peer instead of the row of zq_matmul_gather_tagged), polls (bounded,
 * zq_set_wait_limit) for theirs and takes the best in rank order, which is row order. f32 activations.
 *   w            this rank's rows [rank * out_dim, (rank + 1) * out_dim) of the head (every rank owns as many)
 *   d_y_local    optional: this rank's out_dim outputs are stored there too
 *   h_inbox_*    world > 1: `world` pointers (host array) to every rank's inbox of 2 * world 64-bit words, zeroed
 *                once, odd / even rounds; world = 1: may be null
 *   d_index      the index (every rank computes the same); d_value, optional, its value
 *   d_sync       4096 uint32 on this GPU, zeroed once, 8-byte aligned: rounds, arrivals, one slot per CTA
 * Returns ZQ_ERR_UNSUPPORTED when this rank has too few rows for the kernel (the caller then uses zq_matmul and
 * zq_argmax). */
int zq_matmul_argmax(const zq_weight* w, const float* d_x, const zq_epilogue* epilogue, float* d_y_local,
                     unsigned long long* const* h_inbox_peers_odd, unsigned long long* const* h_inbox_peers_even,
                     int32_t* d_index, float* d_value, uint32_t world, uint32_t rank, uint32_t* d_sync,
                     zq_stream stream);

/* --------------------------------------------------- small ops (inference) */

/* rms_norm_rows (src/models/gemma3.zig:906-946; MetalContext.dispatch_rms_norm,
 * src/backend/metal.zig:848): out = x * (1/sqrt(mean(x^2) + eps)) * w, per row. */
int zq_rms_norm(const float* d_x, const float* d_w, float* d_out, uint32_t dim, uint32_t rows,
                float eps, zq_stream stream);
/* dispatch_rms_norm_residual (src/backend/metal.zig:940; gemma3.zig:718-729):
 * residual[r] += rms_norm(x[r]) * w. */
int zq_rms_norm_residual(const float* d_x, const float* d_w, float* d_residual, uint32_t dim,
                         uint32_t rows, float eps, zq_stream stream);
/* rms_norm_in_place over consecutive heads (src/models/gemma3.zig:949-959;
 * dispatch_rms_norm_in_place, src/backend/metal.zig:875): n_vec vectors of `dim` floats. */
int zq_rms_norm_in_place(float* d_x, const float* d_w, uint32_t dim, uint32_t n_vec, float eps,
                         zq_stream stream);
/* apply_rope_precomputed (src/models/gemma3.zig:962-973; dispatch_rope, metal.zig:898):
 * interleaved pairs (2i, 2i+1) rotated by pos * freqs[i], for n_heads heads of 2*half_dim. */
int zq_rope(float* d_x, const float* d_freqs, uint32_t half_dim, uint32_t n_heads, float pos,
            zq_stream stream);
/* compute_rope_freqs (src/models/gemma3.zig:1128-1135), evaluated on the host with powf. */
int zq_rope_freqs_host(uint32_t head_dim, float rope_base, float* h_freqs);
/* gelu_in_place then mul_in_place (src/models/gemma3.zig:1148-1155,1189-1200;
 * dispatch_gelu_mul, metal.zig:926): gate[i] = gelu(gate[i]) * up[i]. */
int zq_gelu_mul(float* d_gate, const float* d_up, size_t n, zq_stream stream);
/* dispatch_write_kv_cache (metal.zig:1078): copy k,v [kv_dim] to row `pos` of the caches. */
int zq_write_kv_cache(const float* d_k, const float* d_v, float* d_k_cache, float* d_v_cache,
                      uint32_t pos, uint32_t kv_dim, zq_stream stream);
/* gqa_cached_attention / cached_attention (src/models/gemma3.zig:1062-1120;
 * src/models/gpt2.zig:796-849; dispatch_attention_decode, metal.zig:1025).
 * q [n_head*head_dim]; caches [ctx][kv_dim]; out [n_head*head_dim]. Query head h reads the
 * KV head h / (n_head / n_kv_head). Positions kv_start <= p < kv_end (at most 12288 of them).
 * d_scores: scratch of n_head*(kv_end-kv_start) floats, as the Metal dispatcher's `scores` buffer.
 * The arithmetic order is the CPU loops' (16-lane dot products, exponentials summed one by one,
 * values accumulated position by position), so results are bit-identical to them when exp is
 * taken as the correctly rounded f32 exponential. flags: ZQ_ATTN_GPT2_SOFTMAX selects the GPT-2
 * softmax, whose last (n % 16) weights are divided by the sum rather than multiplied by 1/sum. */
#define ZQ_ATTN_GPT2_SOFTMAX 1
int zq_attention_decode(const float* d_q, const float* d_k_cache, const float* d_v_cache,
                        float* d_out, float* d_scores, uint32_t n_head, uint32_t n_kv_head,
                        uint32_t head_dim, uint32_t kv_start, uint32_t kv_end, int flags,
                        zq_stream stream);

/* ----------------------- forward kernels behind src/cuda_ops.zig dispatchers */

/* dispatch_softmax (cuda_ops.zig:88) / dispatch_softmax_out (:518); runtime_kernels.zig:40-81. */
int zq_softmax(float* d_data, uint32_t rows, uint32_t cols, zq_stream stream);
int zq_softmax_out(float* d_out, const float* d_x, uint32_t rows, uint32_t cols, zq_stream stream);
/* dispatch_layer_norm (cuda_ops.zig:113); two-pass statistics as layer_norm_rows
 * (src/models/gpt2.zig:541-596) and layernorm_kernel (kernels/forward_structured.cu:154-198). */
int zq_layer_norm(float* d_out, const float* d_x, const float* d_gamma, const float* d_beta,
                  uint32_t rows, uint32_t cols, float eps, zq_stream stream);
/* dispatch_elementwise with gelu_kernel (cuda_ops.zig:65; forward_elementwise.cu:22-30). */
int zq_gelu(float* d_out, const float* d_x, size_t n, zq_stream stream);
/* dispatch_broadcast_binop with add_broadcast / mul_broadcast (cuda_ops.zig:36;
 * forward_elementwise.cu:4-20): out[i] = a[i] (+|*) b[i % b_total]. */
int zq_add_broadcast(float* d_out, const float* d_a, const float* d_b, size_t a_total,
                     size_t b_total, zq_stream stream);
int zq_mul_broadcast(float* d_out, const float* d_a, const float* d_b, size_t a_total,
                     size_t b_total, zq_stream stream);
/* dispatch_gather (cuda_ops.zig:207; forward_structured.cu:225): out[i] = table[idx[i]]. */
int zq_gather(float* d_out, const float* d_table, const int32_t* d_idx, uint32_t num_indices,
              uint32_t embed_dim, zq_stream stream);
/* dispatch_scale (cuda_ops.zig:236): out[i] = x[i] * s. */
int zq_scale(float* d_out, const float* d_x, float s, size_t n, zq_stream stream);
/* d_dst[i] = src[i], n floats, as a kernel. `src` may be page-locked host memory that the device can
 * address: staging a host activation row this way (instead of a copy-engine transfer) lets the matmul
 * that follows on the stream start streaming its weights while the row is still on its way. No
 * counterpart in the reference, whose CUDA path uploads with cuMemcpyHtoD (src/backend/cuda_context.zig:176). */
int zq_copy_f32(float* d_dst, const float* src, size_t n, zq_stream stream);

/* ------------------------------------------------------------- models */

/* One tensor as the GGUF loader hands it over — RawTensorRef (src/gguf/gguf.zig:147-176). */
typedef struct zq_tensor_ref {
    const void* data; /* host bytes */
    int32_t type;     /* zq_type */
    uint32_t out_dim;
    uint32_t in_dim;
} zq_tensor_ref;

/* GPT2Small / GPT2Medium (src/models/gpt2.zig:10-28). head_dim = embed / head. */
typedef struct zq_gpt2_config {
    uint32_t vocab, embed, head, layer, ctx, ffn;
} zq_gpt2_config;

/* transformer_block_weights (src/models/gpt2.zig:42-59). f32 vectors are host pointers. */
typedef struct zq_gpt2_block {
    const float* ln1_weight;
    const float* ln1_bias;
    zq_tensor_ref attn_qkv_weight; /* [3*embed][embed] */
    const float* attn_qkv_bias;
    zq_tensor_ref attn_proj_weight; /* [embed][embed] */
    const float* attn_proj_bias;
    const float* ln2_weight;
    const float* ln2_bias;
    zq_tensor_ref mlp_fc_weight; /* [ffn][embed] */
    const float* mlp_fc_bias;
    zq_tensor_ref mlp_proj_weight; /* [embed][ffn] */
    const float* mlp_proj_bias;
} zq_gpt2_block;

/* gpt2_weights (src/models/gpt2.zig:61-70). */
typedef struct zq_gpt2_weights {
    const float* wte; /* [vocab][embed] */
    const float* wpe; /* [ctx][embed] */
    const float* ln_f_weight;
    const float* ln_f_bias;
    const zq_gpt2_block* blocks; /* [layer] */
} zq_gpt2_weights;

/* Gemma3_1B (src/models/gemma3.zig:15-29). */
typedef struct zq_gemma3_config {
    uint32_t vocab, embed, head, head_kv, head_dim, layer, ctx, ffn;
    float rope_base;
    uint32_t sliding_window;
    float rms_eps;
    uint32_t global_every; /* layer l is global when l % global_every == global_every-1
                              (is_global_layer, gemma3.zig:1123-1125: 6) */
} zq_gemma3_config;

/* GemmaBlockWeights (src/models/gemma3.zig:100-114). */
typedef struct zq_gemma3_block {
    const float* attn_norm_weight;
    const float* post_attention_norm_weight;
    zq_tensor_ref attn_q_weight;      /* [head*head_dim][embed] */
    zq_tensor_ref attn_k_weight;      /* [head_kv*head_dim][embed] */
    zq_tensor_ref attn_v_weight;      /* [head_kv*head_dim][embed] */
    zq_tensor_ref attn_output_weight; /* [embed][head*head_dim] */
    const float* attn_q_norm_weight;  /* [head_dim] */
    const float* attn_k_norm_weight;  /* [head_dim] */
    const float* ffn_norm_weight;
    const float* post_ffw_norm_weight;
    zq_tensor_ref ffn_gate_weight; /* [ffn][embed] */
    zq_tensor_ref ffn_up_weight;   /* [ffn][embed] */
    zq_tensor_ref ffn_down_weight; /* [embed][ffn] */
} zq_gemma3_block;

/* gemma3_weights (src/models/gemma3.zig:116-123). token_embd doubles as the output head. */
typedef struct zq_gemma3_weights {
    zq_tensor_ref token_embd; /* [vocab][embed], q8_0 or q4_0 or q4_1 */
    const float* output_norm_weight;
    const zq_gemma3_block* blocks; /* [layer] */
} zq_gemma3_weights;

/* Decode engines: device-resident counterparts of gpt2(C) (src/models/gpt2.zig:198-532) and
 * gemma3(C) / gemma3_metal(C) (src/models/gemma3.zig:243-848; gemma3_metal.zig:189-260).
 * create() uploads every tensor and allocates KV cache and scratch once; prefill() and
 * decode_next() allocate nothing. Logits pointers returned are device pointers owned by the
 * engine, valid until the next call; the calls are asynchronous on `stream`. */
typedef struct zq_gpt2 zq_gpt2;
typedef struct zq_gemma3 zq_gemma3;

int zq_gpt2_create(const zq_gpt2_config* cfg, const zq_gpt2_weights* weights, zq_stream stream,
                   zq_gpt2** out);
int zq_gpt2_free(zq_gpt2* m);
int zq_gpt2_reset_cache(zq_gpt2* m);
int zq_gpt2_seq_len(const zq_gpt2* m, uint32_t* seq_len);
/* prefill (gpt2.zig:423-440): resets the cache, processes the prompt, logits of the last token. */
int zq_gpt2_prefill(zq_gpt2* m, const uint32_t* h_tokens, uint32_t n_tokens, zq_stream stream,
                    const float** d_logits);
/* decode_next (gpt2.zig:443-509). */
int zq_gpt2_decode_next(zq_gpt2* m, uint32_t token, zq_stream stream, const float** d_logits);
/* n_steps greedy steps on the device: token <- argmax(logits) each step, no host round trip
 * between steps. h_tokens_out[n_steps] receives the chosen tokens; synchronises `stream`. */
int zq_gpt2_decode_greedy(zq_gpt2* m, uint32_t first_token, uint32_t n_steps, zq_stream stream,
                          uint32_t* h_tokens_out);

int zq_gemma3_create(const zq_gemma3_config* cfg, const zq_gemma3_weights* weights,
                     zq_stream stream, zq_gemma3** out);
int zq_gemma3_free(zq_gemma3* m);
int zq_gemma3_reset_cache(zq_gemma3* m);
int zq_gemma3_seq_len(const zq_gemma3* m, uint32_t* seq_len);
/* prefill (gemma3.zig:551-595). */
int zq_gemma3_prefill(zq_gemma3* m, const uint32_t* h_tokens, uint32_t n_tokens,
                      zq_stream stream, const float** d_logits);
/* decode_next (gemma3.zig:789-827). */
int zq_gemma3_decode_next(zq_gemma3* m, uint32_t token, zq_stream stream,
                          const float** d_logits);
int zq_gemma3_decode_greedy(zq_gemma3* m, uint32_t first_token, uint32_t n_steps,
                            zq_stream stream, uint32_t* h_tokens_out);

/* Several independent sequences in one engine (batched decode). The reference decodes one sequence at a
 * time (gemma3.zig:789-827); here n_seq sequences share the weights, each with its own KV-cache slot and
 * position, and one call advances all of them: the linears run as exact int8 GEMMs over the n_seq rows
 * (weights read once per step instead of once per sequence), every row with the arithmetic of a
 * single-sequence decode step, so each sequence's logits are bit-identical to decoding it alone.
 *   zq_gemma3_create_batch      n_seq cache slots (1 <= n_seq <= 1024); n_seq == 1 is zq_gemma3_create
 *   zq_gemma3_prefill_seq       prefill of sequence `seq`; *d_logits = its last token's logits [vocab]
 *   zq_gemma3_decode_next_batch h_tokens[n_seq] = next token of every sequence; *d_logits = [n_seq][vocab]
 *   zq_gemma3_seq_len_of        tokens held by sequence `seq`
 * zq_gemma3_decode_next / _decode_greedy need n_seq == 1. */
int zq_gemma3_create_batch(const zq_gemma3_config* cfg, const zq_gemma3_weights* w, uint32_t n_seq,
                           zq_stream stream, zq_gemma3** out);
int zq_gemma3_prefill_seq(zq_gemma3* m, uint32_t seq, const uint32_t* h_tokens, uint32_t n, zq_stream stream,
                          const float** d_logits);
int zq_gemma3_decode_next_batch(zq_gemma3* m, const uint32_t* h_tokens, zq_stream stream, const float** d_logits);
int zq_gemma3_seq_len_of(const zq_gemma3* m, uint32_t seq, uint32_t* seq_len);

/* How a one-sequence decode step runs on the device. The reference's Metal engine encodes a whole token
 * into one command buffer (gemma3_metal.zig:189-260); the counterpart here is ONE persistent cooperative
 * kernel per token (or per run of greedy tokens), its phases separated by grid barriers, weights streamed
 * ahead of the phases by bulk copies. Results are bit-identical in both modes.
 *   ZQ_DECODE_AUTO             the persistent kernel when the model fits its plan, else the launch sequence
 *   ZQ_DECODE_LAUNCH_SEQUENCE  always the captured sequence of about ten launches per layer
 *   ZQ_DECODE_PERSISTENT       the persistent kernel; ZQ_ERR_UNSUPPORTED when the model does not fit it
 *                              (mixed types inside q|k|v or gate|up, a weight row above a ring slot,
 *                              batched engines)
 * zq_gemma3_decode_mode reports the mode the next decode step will use (never AUTO). Prefill chunks and
 * batched steps always use the launch sequence. */
#define ZQ_DECODE_AUTO 0
#define ZQ_DECODE_LAUNCH_SEQUENCE 1
#define ZQ_DECODE_PERSISTENT 2
int zq_gemma3_set_decode_mode(zq_gemma3* m, int mode);
int zq_gemma3_decode_mode(const zq_gemma3* m, int* mode);
/* The same choice for the GPT-2 engine (gpt2.zig:423-509). Its persistent kernel computes with f32 multiply-adds
 * and tree reductions in a fixed order: results agree with the launch sequence within this path's tolerance
 * (about 1e-6 relative L2 on logits, identical greedy tokens), not bit for bit. ZQ_ERR_UNSUPPORTED for
 * ZQ_DECODE_PERSISTENT when a linear layer of the model is f32 or a row does not fit a ring slot. */
int zq_gpt2_set_decode_mode(zq_gpt2* m, int mode);
int zq_gpt2_decode_mode(const zq_gpt2* m, int* mode);
/* Per-phase timing of one decode step, the device-side counterpart of gemma3.ProfileStats
 * (gemma3.zig:35-92, filled at :417-491): the persistent kernel runs one step (like decode_next) and every
 * CTA records its SM cycle counter at each phase boundary. h_cycles[n_ctas][capacity] receives the stamps of
 * CTA c at h_cycles[c * capacity ...], in program order: token start; per layer 10 stamps (qkv prologue done,
 * qkv done, scores done, softmax.V done, o prologue done, o done, ffn prologue done, gate/up done, down prologue
 * done, down done); head prologue done, head done. A prologue includes the wait for the vector it consumes.
 * Unused entries are 0. capacity >= 3 + 10 * layers holds all of them. ZQ_ERR_UNSUPPORTED without the
 * persistent kernel. */
int zq_gemma3_profile_step(zq_gemma3* m, uint32_t token, zq_stream stream, long long* h_cycles, uint32_t capacity,
                           uint32_t* n_ctas);

#ifdef __cplusplus
}
#endif
#endif /* ZQ_H */
