// Internal declarations shared by the libzq translation units (not part of the C ABI).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "zq.h"

// Device-resident quantised weight. Values are those of the GGUF blocks; only the arrangement
// differs so that the kernels can use aligned 128-bit loads that feed tensor-core fragments directly:
//   qs : quant words of each row, in groups of 4 consecutive blocks ("quads"). Inside a quad the 32-bit
//        words are interleaved so that words with the same index t of the 4 blocks are adjacent:
//          q4_0 / q4_1 (4 words per block):  quad = 64 bytes,  word w of block j at (w*4 + j)*4
//          q8_0 (8 words per block):         quad = 128 bytes, word w of block j at
//                                            ((w/4)*16 + (w%4)*4 + j)*4
//        A lane that needs word t of every block (the K footprint of an MMA A fragment) reads 16
//        contiguous bytes per quad. Rows are padded to nbp = roundup(nb, 4) blocks (zero quants).
//   sc : q4_0 / q8_0: f16 d [out_dim][scp];  q4_1: (f16 d, f16 m) pairs [out_dim][scp].
//        scp >= nb is the row pitch in scale elements, padded with zeros to a multiple of 8 so that
//        every row starts on a 16-byte boundary.
struct zq_weight {
    int type;
    uint32_t out_dim;
    uint32_t in_dim;
    uint32_t nb;       // blocks per row = in_dim / 32
    uint32_t nbp;      // blocks per row in the qs array (nb rounded up to a multiple of 4)
    uint32_t qb;       // quant bytes per block
    uint32_t scp;      // scale elements per row (pitch), multiple of 8 (f16) or 4 (f16 pairs)
    uint8_t* qs;       // device
    void* sc;          // device
    void* base;        // the single allocation holding qs and sc
    size_t bytes;      // size of that allocation
    int device;        // ordinal of the device that holds it
};

namespace zq {

extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return ZQ_ERR_CUDA;
}

#define ZQ_CUDA(call)                                   \
    do {                                                \
        cudaError_t e__ = (call);                       \
        if (e__ != cudaSuccess) return zq::cuda_fail(e__); \
    } while (0)

// Check the launch that was just issued.
#define ZQ_LAUNCH_CHECK() ZQ_CUDA(cudaGetLastError())

inline cudaStream_t as_stream(zq_stream s) { return reinterpret_cast<cudaStream_t>(s); }

// Byte offset of 32-bit word `w` of block `blk` inside a row of the interleaved qs array.
__host__ __device__ inline size_t qs_word_offset(uint32_t qb, uint32_t blk, uint32_t w) {
    const uint32_t quad = blk >> 2, j = blk & 3u;
    if (qb == 16) return (size_t)quad * 64 + (size_t)(w * 4 + j) * 4;
    return (size_t)quad * 128 + (size_t)((w >> 2) * 16 + (w & 3u) * 4 + j) * 4;
}

// ---- programmatic dependent launch -----------------------------------------------------------
// Decode-step kernels are launched with the programmatic-serialisation attribute: a kernel may start
// while its predecessor in the stream is still running. Each such kernel first calls
// pdl_launch_dependents() (so its own successor can be scheduled early), may prefetch data that no
// earlier kernel writes (weights), and must call pdl_wait() before it touches anything an earlier
// kernel produces or still reads: pdl_wait() returns only when every earlier grid has completed and
// its writes are visible. Without the launch attribute both calls do nothing.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Ask L2 to fetch `bytes` (a multiple of 16, 16-byte aligned address) without waiting for them.
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
__device__ __forceinline__ void prefetch_l2_line(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// Exponent e of the power-of-two row scale 2^-e that brings a row's largest magnitude `amax` just under 2^14
// (fp16 operands keep full precision, no overflow). Rows that are zero, not finite, or so small that 2^-e
// would overflow f32 (amax below 2^-100: vanishing gradients) are left unscaled.
__host__ __device__ inline int row_scale_exponent(float amax) {
    if (!(amax > 7.8886090522101181e-31f) || !(amax < INFINITY)) return 0;
    return ilogbf(amax) - 13;
}

inline bool is_quant(int t) { return t == ZQ_TYPE_Q4_0 || t == ZQ_TYPE_Q4_1 || t == ZQ_TYPE_Q8_0; }

int sm_count();  // multiprocessors of the current device (cached per device)
// Polls a device-side wait on a peer's flag makes before it gives up (zq_set_wait_limit; 0 = the kernel's default).
uint32_t wait_limit();
// Device address of the word zq_device_error() reads; kernels with bounded waits record a timeout there.
int device_error_word(unsigned int** out);
// ZQ_OK when the weight lives on the current device, ZQ_ERR_BAD_ARG otherwise.
int check_weight_device(const zq_weight* w);

// ---- launchers implemented in gemv.cu and used by the engines -------------------------

// Prologue applied to the activation row before the dot products (engine fusions).
enum Prologue { PRO_NONE = 0 };

int launch_gemv_f32(const zq_weight* w, const float* x, float* y, uint32_t m_rows,
                    const zq_epilogue* ep, cudaStream_t st);
// Tensor-core f32-activation GEMV for m_rows <= 16 (gemv_mma.cu); x must be 16-byte aligned.
int launch_gemv_mma_f32(const zq_weight* w, const float* x, float* y, uint32_t m_rows,
                        const zq_epilogue* ep, cudaStream_t st);
// Any row count: passes of up to 16 rows, the pass height chosen so that its activation image fits.
int launch_gemv_mma_passes_f32(const zq_weight* w, const float* x, float* y, uint32_t m_rows,
                               const zq_epilogue* ep, cudaStream_t st);
// The same with LayerNorm(x) computed in the kernel's prologue (one activation row; gpt2.zig:541-596).
int launch_gemv_mma_ln_f32(const zq_weight* w, const float* x, float* y, uint32_t m_rows, const zq_epilogue* ep,
                           const float* ln_gamma, const float* ln_beta, float ln_eps, cudaStream_t st);
// f32-activation GEMV for one row with the all-gather of row-sharded outputs fused in (gemv_mma.cu).
int launch_gemv_gather_tagged_f32(const zq_weight* w, const float* x, const zq_epilogue* ep,
                                  unsigned long long* const* inbox_odd, unsigned long long* const* inbox_even,
                                  float* y_odd, float* y_even, uint32_t world, uint32_t rank, uint32_t* d_sync,
                                  cudaStream_t st);
int launch_gemv_argmax_f32(const zq_weight* w, const float* x, const zq_epilogue* ep, float* y_local,
                           unsigned long long* const* inbox_odd, unsigned long long* const* inbox_even,
                           int32_t* out_index, float* out_value, uint32_t world, uint32_t rank, uint32_t* d_sync,
                           cudaStream_t st);
int launch_gemv_gather_f32(const zq_weight* w, const float* x, const zq_epilogue* ep, float* const* y_odd,
                           float* const* y_even, uint32_t* const* flags, uint32_t world, uint32_t rank,
                           uint32_t row_off, uint32_t* d_sync, cudaStream_t st);
int launch_gemv_q8(const zq_weight* w, const int8_t* xq, const float* xscale, const int32_t* xsum,
                   float* y, uint32_t m_rows, const zq_epilogue* ep, cudaStream_t st);
int launch_quantize_rows_q8(const float* x, uint32_t m_rows, uint32_t in_dim, int8_t* q,
                            float* scale, int32_t* sum, cudaStream_t st);
// Exact int8 tensor-core GEMM for many Q8-quantised activation rows; bit-identical to launch_gemv_q8 (gemm_q8.cu).
int launch_gemm_q8(const zq_weight* w, const int8_t* xq, const float* xscale, const int32_t* xsum, float* y,
                   uint32_t m_rows, const zq_epilogue* ep, cudaStream_t st);
constexpr uint32_t kGemmMinRows = 49;  // below this, passes of the 16-row decode kernel are faster
// x16[m][k] = fp16(x[m][k] * 2^-e_m), post[m] = 2^e_m (gemm.cu).
int launch_convert_rows_f16(const float* x, __half* x16, float* post, uint32_t m_rows, uint32_t in_dim,
                            cudaStream_t st);
// Tensor-core GEMM for many activation rows: tcgen05.mma, fp16 operands, accumulator in tensor memory
// (gemm_tc.cu). `workspace` holds gemm_tc_workspace_bytes() bytes, 256-byte aligned.
int launch_gemm_tc(const zq_weight* w, const float* x, float* y, uint32_t m_rows, const zq_epilogue* ep,
                   void* workspace, cudaStream_t st);
size_t gemm_tc_workspace_bytes(const zq_weight* w, uint32_t m_rows);
// True when the weight-streaming form of the tensor-core GEMM (up to 128 activation rows, matrices of 12 288 rows
// and more) serves the call.
bool gemm_stream_takes(const zq_weight* w, uint32_t m_rows);
// The transposed product on pairs of CTAs (gemm_tc.cu): whether it takes the call, its workspace, the launch.
bool gemm_trans_pair_takes(const zq_weight* w, uint32_t m_rows);
size_t gemm_trans_pair_workspace_bytes(const zq_weight* w, uint32_t m_rows);
int launch_gemm_trans_pair(const zq_weight* w, const float* grad_out, float* grad_x, uint32_t m_rows, int accumulate,
                           void* workspace, cudaStream_t st);
constexpr uint32_t kStreamMinRowsF32 = 17;  // f32-activation calls from this many rows on take it when they bring a workspace

// ---- fused decode-step launchers (ops.cu). `state` is device memory: state[0] = current token,
// state[1] = its position. Kernels read the position there, so a captured launch sequence can be
// replayed for every step.

// `rows` > 1: row r is token r of a prefill chunk at position state[1] + r, or — row_pos != nullptr — one
// of several independent sequences at position row_pos[r] with its own cache cache_stride floats
// further. Inputs of row r start r * <stride> floats further, quantised outputs are dense [rows][dim].
// res == nullptr: quantise rms_norm(src, w1).  Otherwise res += rms_norm(src, w1) and quantise
// rms_norm(res, w2).
int launch_norm_quant(const float* src, const float* w1, float* res, const float* w2, uint32_t dim, float eps,
                      int8_t* q, float* scale, int32_t* sum, uint32_t rows, uint32_t src_stride, cudaStream_t st);
// qkv = [q heads | k heads | v heads]; q is normalised and rotated in place, k and v go to the caches.
int launch_qk_norm_rope_kv(float* qkv, const float* q_norm_w, const float* k_norm_w, const float* freqs,
                           float* kc, float* vc, const uint32_t* state, uint32_t n_head, uint32_t n_kv_head,
                           uint32_t head_dim, float eps, uint32_t rows, uint32_t qkv_stride, const uint32_t* row_pos,
                           size_t cache_stride, cudaStream_t st);
int launch_gelu_mul_quant(const float* gate, const float* up, uint32_t n, int8_t* q, float* scale,
                          int32_t* sum, uint32_t rows, uint32_t in_stride, cudaStream_t st);
// Single-query attention over positions [max(0, pos + 1 - window), pos] (window 0 = all); max_len is the
// largest window any step can have. k_new / v_new (optional, rows == 1): this step's key / value rows,
// stored into row `pos` of the caches by the same launch. `out` (f32) and `oq/oscale/osum` (quantised)
// are each optional. scores holds rows * n_head * max_len floats. q_norm_w != nullptr: q and k_new are raw
// projection outputs; per-head RMSNorm + RoPE (gemma3.zig:689-716) is applied inside the scores kernel.
int launch_attention_step(const float* q, float* kc, float* vc, const float* k_new, const float* v_new,
                          float* out, int8_t* oq, float* oscale, int32_t* osum, float* scores, uint32_t n_head,
                          uint32_t n_kv_head, uint32_t head_dim, const uint32_t* state, uint32_t window,
                          uint32_t max_len, int flags, uint32_t rows, uint32_t q_stride, const uint32_t* row_pos,
                          size_t cache_stride, const float* q_norm_w, const float* k_norm_w, const float* freqs,
                          float norm_eps, cudaStream_t st);
// f32 matvec (GPT-2 vocabulary head) with an optional LayerNorm of x in the prologue (gemv.cu).
int launch_matvec_ln_f32(const float* w, const float* x, float* y, uint32_t out_dim, uint32_t in_dim,
                         const float* ln_gamma, const float* ln_beta, float ln_eps, cudaStream_t st);
int launch_gpt2_embed_step(float* x, const float* wte, const float* wpe, const uint32_t* state,
                           const int32_t* tokens, uint32_t embed, uint32_t rows, cudaStream_t st);
int launch_write_kv_step(const float* k, const float* v, float* kc, float* vc, const uint32_t* state,
                         uint32_t kv_dim, uint32_t rows, uint32_t in_stride, cudaStream_t st);

}  // namespace zq
