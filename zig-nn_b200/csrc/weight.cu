// Weight handles: upload + re-layout of GGUF quant blocks, bit-exact dequantisation.
#include <new>

#include <atomic>
#include <mutex>

#include "zq_internal.h"

namespace zq {

thread_local int g_last_cuda_error = 0;

// Set by a kernel whose bounded device-side wait ran out; read with zq_device_error().
__device__ unsigned int g_device_error = 0;

// Device address of the error word, for kernels in other translation units (passed as a parameter).
static std::atomic<uint32_t> g_wait_limit{0};
uint32_t wait_limit() { return g_wait_limit.load(std::memory_order_relaxed); }

int check_weight_device(const zq_weight* w) {
    int dev = -1;
    ZQ_CUDA(cudaGetDevice(&dev));
    return w && w->device == dev ? ZQ_OK : ZQ_ERR_BAD_ARG;
}

int device_error_word(unsigned int** out) {
    static unsigned int* cached[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    ZQ_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return ZQ_ERR_LIMIT;
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[dev]) {
        void* p = nullptr;
        ZQ_CUDA(cudaGetSymbolAddress(&p, g_device_error));
        cached[dev] = static_cast<unsigned int*>(p);
    }
    *out = cached[dev];
    return ZQ_OK;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

namespace {

__host__ __device__ inline uint32_t raw_bpb(int type) {
    return type == ZQ_TYPE_Q4_0 ? 18u : type == ZQ_TYPE_Q4_1 ? 20u : 34u;
}

// One thread per block: split the GGUF block into its scale word(s) and its quant bytes.
__global__ void repack_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ qs,
                              uint8_t* __restrict__ sc, int type, size_t n_blocks, uint32_t nb,
                              uint32_t scp) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const uint32_t bpb = raw_bpb(type);
    const uint32_t hdr = type == ZQ_TYPE_Q4_1 ? 4u : 2u;
    const uint32_t qb = bpb - hdr;
    const uint8_t* src = raw + b * bpb;
    const size_t row = b / nb;
    const uint32_t blk = (uint32_t)(b % nb);
    const size_t sb = row * scp + blk;  // scale slot in the padded row
    for (uint32_t i = 0; i < hdr; ++i) sc[sb * hdr + i] = src[i];
    const uint32_t nbp = (nb + 3u) & ~3u;
    uint8_t* qrow = qs + row * (size_t)nbp * qb;
    for (uint32_t i = 0; i < qb; ++i) qrow[qs_word_offset(qb, blk, i >> 2) + (i & 3u)] = src[hdr + i];
}

__global__ void unpack_kernel(uint8_t* __restrict__ raw, const uint8_t* __restrict__ qs,
                              const uint8_t* __restrict__ sc, int type, size_t n_blocks, uint32_t nb,
                              uint32_t scp) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const uint32_t bpb = raw_bpb(type);
    const uint32_t hdr = type == ZQ_TYPE_Q4_1 ? 4u : 2u;
    const uint32_t qb = bpb - hdr;
    uint8_t* dst = raw + b * bpb;
    const size_t row = b / nb;
    const uint32_t blk = (uint32_t)(b % nb);
    const size_t sb = row * scp + blk;
    for (uint32_t i = 0; i < hdr; ++i) dst[i] = sc[sb * hdr + i];
    const uint32_t nbp = (nb + 3u) & ~3u;
    const uint8_t* qrow = qs + row * (size_t)nbp * qb;
    for (uint32_t i = 0; i < qb; ++i) dst[hdr + i] = qrow[qs_word_offset(qb, blk, i >> 2) + (i & 3u)];
}

// One thread per element. `row_map` (optional) selects source rows; `scale_mode` multiplies the
// dequantised value by `scale` as a second, separately rounded multiply.
template <int TYPE>
__global__ void dequant_kernel(const uint8_t* __restrict__ qs, const void* __restrict__ sc,
                               float* __restrict__ out, uint32_t nb, uint32_t scp, size_t n_rows,
                               const int32_t* __restrict__ row_map, int scale_mode, float scale) {
    const size_t K = (size_t)nb * 32;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * K) return;
    const size_t r = idx / K;
    const uint32_t k = (uint32_t)(idx - r * K);
    const size_t src_row = row_map ? (size_t)row_map[r] : r;
    const uint32_t blk = k >> 5;
    const size_t sblk = src_row * scp + blk;
    const uint32_t j = k & 31;
    const uint32_t nbp = (nb + 3u) & ~3u;
    const uint8_t* qrow = qs + src_row * (size_t)nbp * (TYPE == ZQ_TYPE_Q8_0 ? 32 : 16);
    float v;
    if (TYPE == ZQ_TYPE_Q8_0) {
        const float d = __half2float(reinterpret_cast<const __half*>(sc)[sblk]);
        const int8_t q = (int8_t)qrow[qs_word_offset(32, blk, j >> 2) + (j & 3u)];
        v = __fmul_rn((float)q, d);
    } else {
        const uint32_t jb = j & 15u;
        const uint8_t byte = qrow[qs_word_offset(16, blk, jb >> 2) + (jb & 3u)];
        const int nib = (j < 16) ? (byte & 0x0F) : (byte >> 4);
        if (TYPE == ZQ_TYPE_Q4_0) {
            const float d = __half2float(reinterpret_cast<const __half*>(sc)[sblk]);
            v = __fmul_rn((float)(nib - 8), d);
        } else {
            const __half2 dm = reinterpret_cast<const __half2*>(sc)[sblk];
            // nibble*d then +m: two roundings, never contracted into an FMA
            v = __fadd_rn(__fmul_rn((float)nib, __low2float(dm)), __high2float(dm));
        }
    }
    if (scale_mode) v = __fmul_rn(v, scale);
    out[idx] = v;
}

int make_weight(int type, uint32_t out_dim, uint32_t in_dim, zq_weight** out) {
    if (!out) return ZQ_ERR_BAD_ARG;
    *out = nullptr;
    if (type != ZQ_TYPE_Q4_0 && type != ZQ_TYPE_Q4_1 && type != ZQ_TYPE_Q8_0)
        return ZQ_ERR_UNSUPPORTED;
    if (out_dim == 0 || in_dim == 0 || (in_dim % 32) != 0) return ZQ_ERR_BAD_ARG;
    zq_weight* w = new (std::nothrow) zq_weight;
    if (!w) return ZQ_ERR_NO_MEM;
    w->type = type;
    w->out_dim = out_dim;
    w->in_dim = in_dim;
    w->nb = in_dim / 32;
    w->qb = type == ZQ_TYPE_Q8_0 ? 32 : 16;
    w->nbp = (w->nb + 3u) & ~3u;
    const size_t qs_bytes = (size_t)out_dim * w->nbp * w->qb;
    const size_t qs_pad = (qs_bytes + 255) & ~(size_t)255;
    w->scp = type == ZQ_TYPE_Q4_1 ? ((w->nb + 3) & ~3u) : ((w->nb + 7) & ~7u);
    const size_t sc_bytes = (size_t)out_dim * w->scp * (type == ZQ_TYPE_Q4_1 ? 4 : 2);
    w->bytes = qs_pad + ((sc_bytes + 255) & ~(size_t)255);
    cudaError_t e = cudaMalloc(&w->base, w->bytes);
    if (e != cudaSuccess) {
        delete w;
        g_last_cuda_error = (int)e;
        return e == cudaErrorMemoryAllocation ? ZQ_ERR_NO_MEM : ZQ_ERR_CUDA;
    }
    w->qs = static_cast<uint8_t*>(w->base);
    w->sc = w->qs + qs_pad;
    w->device = 0;
    cudaGetDevice(&w->device);
    *out = w;
    return ZQ_OK;
}

}  // namespace
}  // namespace zq

using namespace zq;

extern "C" {

const char* zq_status_string(int s) {
    switch (s) {
        case ZQ_OK: return "ok";
        case ZQ_ERR_BAD_ARG: return "bad argument";
        case ZQ_ERR_UNSUPPORTED: return "unsupported quant type";
        case ZQ_ERR_CUDA: return "CUDA error";
        case ZQ_ERR_NO_MEM: return "out of memory";
        case ZQ_ERR_LIMIT: return "size limit exceeded";
        case ZQ_ERR_SEQUENCE: return "empty sequence, sequence too long or context full";
        case ZQ_ERR_TIMEOUT: return "device-side wait timed out";
        case ZQ_ERR_PEER: return "peer set-up failed";
        default: return "unknown status";
    }
}

int zq_last_cuda_error(void) { return g_last_cuda_error; }

int zq_device_error(unsigned int* out, int clear) {
    if (!out) return ZQ_ERR_BAD_ARG;
    unsigned int v = 0;
    ZQ_CUDA(cudaMemcpyFromSymbol(&v, zq::g_device_error, sizeof(v)));
    *out = v;
    if (clear && v) {
        const unsigned int z = 0;
        ZQ_CUDA(cudaMemcpyToSymbol(zq::g_device_error, &z, sizeof(z)));
    }
    return ZQ_OK;
}
int zq_device_check(int clear) {
    unsigned int v = 0;
    const int rc = zq_device_error(&v, clear);
    if (rc != ZQ_OK) return rc;
    return v ? ZQ_ERR_TIMEOUT : ZQ_OK;
}
int zq_set_wait_limit(unsigned int polls) {
    zq::g_wait_limit.store(polls, std::memory_order_relaxed);
    return ZQ_OK;
}
int zq_abi_version(void) { return 1; }

size_t zq_block_size(int t) {
    switch (t) {
        case ZQ_TYPE_F32:
        case ZQ_TYPE_F16: return 1;
        case ZQ_TYPE_Q4_0:
        case ZQ_TYPE_Q4_1:
        case ZQ_TYPE_Q8_0: return 32;
        default: return 0;
    }
}

size_t zq_bytes_per_block(int t) {
    switch (t) {
        case ZQ_TYPE_F32: return 4;
        case ZQ_TYPE_F16: return 2;
        case ZQ_TYPE_Q4_0: return 18;
        case ZQ_TYPE_Q4_1: return 20;
        case ZQ_TYPE_Q8_0: return 34;
        default: return 0;
    }
}

size_t zq_tensor_bytes(int t, size_t n) {
    const size_t bs = zq_block_size(t);
    return bs ? (n / bs) * zq_bytes_per_block(t) : 0;
}

int zq_weight_from_device(const void* d_raw, int type, uint32_t out_dim, uint32_t in_dim,
                          zq_stream stream, zq_weight** out) {
    if (!d_raw) return ZQ_ERR_BAD_ARG;
    int rc = make_weight(type, out_dim, in_dim, out);
    if (rc != ZQ_OK) return rc;
    zq_weight* w = *out;
    const size_t n_blocks = (size_t)out_dim * w->nb;
    const unsigned threads = 256;
    const unsigned blocks = (unsigned)((n_blocks + threads - 1) / threads);
    // padding blocks of the quant rows and padding slots of the scale rows read as zero
    cudaError_t e = cudaSuccess;
    if (w->nbp != w->nb) e = cudaMemsetAsync(w->qs, 0, (size_t)out_dim * w->nbp * w->qb, as_stream(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(w->sc, 0, (size_t)out_dim * w->scp * (type == ZQ_TYPE_Q4_1 ? 4 : 2),
                                    as_stream(stream));
    if (e == cudaSuccess) {
        repack_kernel<<<blocks, threads, 0, as_stream(stream)>>>(static_cast<const uint8_t*>(d_raw), w->qs,
                                                                 static_cast<uint8_t*>(w->sc), type, n_blocks,
                                                                 w->nb, w->scp);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        zq_weight_free(w);
        *out = nullptr;
        return cuda_fail(e);
    }
    return ZQ_OK;
}

int zq_weight_upload(const void* h_raw, int type, uint32_t out_dim, uint32_t in_dim,
                     zq_stream stream, zq_weight** out) {
    if (!h_raw || !out) return ZQ_ERR_BAD_ARG;
    *out = nullptr;
    if (!is_quant(type)) return ZQ_ERR_UNSUPPORTED;
    if (out_dim == 0 || in_dim == 0 || (in_dim % 32) != 0) return ZQ_ERR_BAD_ARG;
    const size_t raw_bytes = zq_tensor_bytes(type, (size_t)out_dim * in_dim);
    void* staging = nullptr;
    cudaError_t e = cudaMalloc(&staging, raw_bytes);
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        return e == cudaErrorMemoryAllocation ? ZQ_ERR_NO_MEM : ZQ_ERR_CUDA;
    }
    cudaStream_t st = as_stream(stream);
    int rc = ZQ_OK;
    e = cudaMemcpyAsync(staging, h_raw, raw_bytes, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) rc = cuda_fail(e);
    if (rc == ZQ_OK) rc = zq_weight_from_device(staging, type, out_dim, in_dim, stream, out);
    e = cudaStreamSynchronize(st);
    if (rc == ZQ_OK && e != cudaSuccess) rc = cuda_fail(e);
    cudaFree(staging);
    if (rc != ZQ_OK && *out) {
        zq_weight_free(*out);
        *out = nullptr;
    }
    return rc;
}

int zq_weight_free(zq_weight* w) {
    if (!w) return ZQ_OK;
    cudaError_t e = cudaFree(w->base);
    delete w;
    if (e != cudaSuccess) return cuda_fail(e);
    return ZQ_OK;
}

int zq_weight_info(const zq_weight* w, int* type, uint32_t* out_dim, uint32_t* in_dim) {
    if (!w) return ZQ_ERR_BAD_ARG;
    if (type) *type = w->type;
    if (out_dim) *out_dim = w->out_dim;
    if (in_dim) *in_dim = w->in_dim;
    return ZQ_OK;
}

size_t zq_weight_device_bytes(const zq_weight* w) { return w ? w->bytes : 0; }

int zq_weight_download_raw(const zq_weight* w, void* d_raw, zq_stream stream) {
    if (!w || !d_raw) return ZQ_ERR_BAD_ARG;
    const size_t n_blocks = (size_t)w->out_dim * w->nb;
    const unsigned threads = 256;
    const unsigned blocks = (unsigned)((n_blocks + threads - 1) / threads);
    unpack_kernel<<<blocks, threads, 0, as_stream(stream)>>>(
        static_cast<uint8_t*>(d_raw), w->qs, static_cast<const uint8_t*>(w->sc), w->type, n_blocks, w->nb,
        w->scp);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

static int dequant_launch(const zq_weight* w, float* d_out, size_t n_rows, const int32_t* row_map,
                          int scale_mode, float scale, zq_stream stream) {
    const size_t total = n_rows * (size_t)w->in_dim;
    if (total == 0) return ZQ_OK;
    const unsigned threads = 256;
    const size_t blocks64 = (total + threads - 1) / threads;
    if (blocks64 > 0x7FFFFFFFull) return ZQ_ERR_LIMIT;
    const unsigned blocks = (unsigned)blocks64;
    cudaStream_t st = as_stream(stream);
    switch (w->type) {
        case ZQ_TYPE_Q4_0:
            dequant_kernel<ZQ_TYPE_Q4_0><<<blocks, threads, 0, st>>>(w->qs, w->sc, d_out, w->nb, w->scp,
                                                                    n_rows, row_map, scale_mode, scale);
            break;
        case ZQ_TYPE_Q4_1:
            dequant_kernel<ZQ_TYPE_Q4_1><<<blocks, threads, 0, st>>>(w->qs, w->sc, d_out, w->nb, w->scp,
                                                                    n_rows, row_map, scale_mode, scale);
            break;
        case ZQ_TYPE_Q8_0:
            dequant_kernel<ZQ_TYPE_Q8_0><<<blocks, threads, 0, st>>>(w->qs, w->sc, d_out, w->nb, w->scp,
                                                                    n_rows, row_map, scale_mode, scale);
            break;
        default: return ZQ_ERR_UNSUPPORTED;
    }
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

int zq_dequantize(const zq_weight* w, float* d_out, zq_stream stream) {
    if (!w || !d_out) return ZQ_ERR_BAD_ARG;
    return dequant_launch(w, d_out, w->out_dim, nullptr, 0, 1.0f, stream);
}

int zq_dequant_rows_scaled(const zq_weight* w, const int32_t* d_token_ids, uint32_t n_rows,
                           float scale, float* d_out, zq_stream stream) {
    if (!w || !d_token_ids || !d_out) return ZQ_ERR_BAD_ARG;
    return dequant_launch(w, d_out, n_rows, d_token_ids, 1, scale, stream);
}

}  // extern "C"
