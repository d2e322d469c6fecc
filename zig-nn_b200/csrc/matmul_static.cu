// zq_matmul_q8_static: the Q8-activation matmul for callers that must not allocate.
//
// zq_matmul in ZQ_ACT_Q8 mode needs scratch for the quantised activation rows (int8 values, per-block
// scales and sums) and asks the caller to bring it. Some callers cannot: a host runtime that took all
// of its device memory up front and hands out slices of it (there is nothing left to cudaMalloc from,
// and its own pool may not be reachable from where the call is made), or a latency-critical decode
// loop that cannot afford cudaMalloc's implicit device-wide synchronisation or the possibility of an
// out-of-memory failure in the middle of a request. For them the scratch lives in this library's
// image: a fixed array in device global memory, present on every GPU that loads the library for as
// long as the process runs.
#include <mutex>

#include "zq_internal.h"

namespace {

constexpr uint32_t kMaxRows = 16;       // activation rows per call
constexpr uint32_t kMaxInDim = 16384;   // in_dim limit of the Q8-activation path
constexpr size_t kQuantBytes = (size_t)kMaxRows * kMaxInDim;                       // int8 values
constexpr size_t kBlockBytes = (size_t)kMaxRows * (kMaxInDim / 32) * sizeof(float);  // scales; sums alike
constexpr size_t kScratchBytes = kQuantBytes + 2 * kBlockBytes;                    // 320 KiB

// In host code this name is only a handle for the runtime, never a device address: the address the
// kernels get comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

std::mutex g_mutex;
void* g_scratch_ptr[64] = {nullptr};  // per device ordinal, filled on first use

// Device address of the scratch array on the current device; looked up once per device.
int static_scratch(void** out) {
    int dev = 0;
    ZQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return ZQ_ERR_LIMIT;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        ZQ_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) return ZQ_ERR_CUDA;
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return ZQ_OK;
}

}  // namespace

extern "C" int zq_matmul_q8_static(const zq_weight* w, const float* d_x, float* d_y, uint32_t m_rows,
                                   const zq_epilogue* epilogue, zq_stream stream) {
    if (!w) return ZQ_ERR_BAD_ARG;
    if (m_rows == 0) return ZQ_OK;
    if (!d_x || !d_y) return ZQ_ERR_BAD_ARG;
    if (m_rows > kMaxRows || w->in_dim > kMaxInDim) return ZQ_ERR_LIMIT;  // beyond the built-in scratch
    // the scratch of the CURRENT device is used: the weight has to live there too
    if (zq::check_weight_device(w) != ZQ_OK) return ZQ_ERR_BAD_ARG;
    void* base = nullptr;
    int rc = static_scratch(&base);
    if (rc != ZQ_OK) return rc;
    // Fixed carve-up (independent of the call's sizes), every part 256-byte aligned. Each call rewrites
    // exactly the entries it reads, so nothing has to be cleared between calls.
    int8_t* q = static_cast<int8_t*>(base);
    float* scale = reinterpret_cast<float*>(static_cast<unsigned char*>(base) + kQuantBytes);
    int32_t* sum = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(base) + kQuantBytes + kBlockBytes);
    cudaStream_t st = zq::as_stream(stream);
    rc = zq::launch_quantize_rows_q8(d_x, m_rows, w->in_dim, q, scale, sum, st);
    if (rc != ZQ_OK) return rc;
    // same kernels as zq_matmul in ZQ_ACT_Q8 mode (neither allocates): the exact int8 GEMM from two rows on
    if (m_rows >= 2) return zq::launch_gemm_q8(w, q, scale, sum, d_y, m_rows, epilogue, st);
    return zq::launch_gemv_q8(w, q, scale, sum, d_y, m_rows, epilogue, st);
}
