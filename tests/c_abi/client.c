/* A plain-C client of libzq: what a compiled host (zig-nn's Zig, through the same C ABI) does with a
 * quantised linear layer. No Python, no torch: cudaMalloc'd buffers, a q8_0 matrix built by hand whose
 * product is known in closed form, both activation modes, the error paths.
 *
 * Weight: N rows x K columns, every block has scale d = 0.5 (f16 0x3800) and quants q[i] = (row % 7) - 3.
 * x = all ones  ->  y[row] = K * 0.5 * ((row % 7) - 3), exact in both modes (the Q8 quantiser maps 1.0 to
 * 127 with scale 1/127; (0.5 * (1/127)) * float(127 * 32 * q) per block is not exactly K*0.5*q, so that
 * mode is compared with a tolerance). Exit code 0 = pass. */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "zq.h"

#define CHECK(call)                                                        \
    do {                                                                   \
        int rc__ = (call);                                                 \
        if (rc__ != 0) {                                                   \
            fprintf(stderr, "%s:%d: %s -> %d (%s)\n", __FILE__, __LINE__, #call, rc__, zq_status_string(rc__)); \
            return 1;                                                      \
        }                                                                  \
    } while (0)
#define CUDA(call)                                                         \
    do {                                                                   \
        cudaError_t e__ = (call);                                          \
        if (e__ != cudaSuccess) {                                          \
            fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e__)); \
            return 1;                                                      \
        }                                                                  \
    } while (0)

int main(void) {
    const uint32_t N = 300, K = 256, M = 3;
    const size_t nb = K / 32, row_bytes = nb * 34;
    if (zq_tensor_bytes(ZQ_TYPE_Q8_0, (size_t)N * K) != N * row_bytes) return 2;
    if (zq_block_size(ZQ_TYPE_Q4_0) != 32 || zq_bytes_per_block(ZQ_TYPE_Q4_1) != 20) return 2;

    uint8_t* raw = (uint8_t*)malloc(N * row_bytes);
    for (uint32_t r = 0; r < N; ++r)
        for (size_t b = 0; b < nb; ++b) {
            uint8_t* blk = raw + r * row_bytes + b * 34;
            blk[0] = 0x00; blk[1] = 0x38;                       /* f16 0.5, little endian */
            memset(blk + 2, (uint8_t)(int8_t)((int)(r % 7) - 3), 32);
        }

    zq_weight* w = NULL;
    CHECK(zq_weight_upload(raw, ZQ_TYPE_Q8_0, N, K, NULL, &w));
    int type = 0; uint32_t od = 0, id = 0;
    CHECK(zq_weight_info(w, &type, &od, &id));
    if (type != ZQ_TYPE_Q8_0 || od != N || id != K) return 3;

    float *d_x = NULL, *d_y = NULL, *h_x = (float*)malloc(sizeof(float) * M * K), *h_y = (float*)malloc(sizeof(float) * M * N);
    for (uint32_t i = 0; i < M * K; ++i) h_x[i] = 1.0f;
    CUDA(cudaMalloc((void**)&d_x, sizeof(float) * M * K));
    CUDA(cudaMalloc((void**)&d_y, sizeof(float) * M * N));
    CUDA(cudaMemcpy(d_x, h_x, sizeof(float) * M * K, cudaMemcpyHostToDevice));

    /* f32 activations: exact */
    CHECK(zq_matmul(w, d_x, d_y, M, ZQ_ACT_F32, NULL, NULL, 0, NULL));
    CUDA(cudaMemcpy(h_y, d_y, sizeof(float) * M * N, cudaMemcpyDeviceToHost));
    for (uint32_t m = 0; m < M; ++m)
        for (uint32_t r = 0; r < N; ++r) {
            const float want = (float)K * 0.5f * (float)((int)(r % 7) - 3);
            if (h_y[m * N + r] != want) {
                fprintf(stderr, "f32 mode: y[%u][%u] = %g, want %g\n", m, r, h_y[m * N + r], want);
                return 4;
            }
        }

    /* Q8 activations: needs the workspace the library asks for */
    const size_t ws_bytes = zq_matmul_workspace_bytes(w, M, ZQ_ACT_Q8);
    void* d_ws = NULL;
    if (ws_bytes == 0) return 5;
    CUDA(cudaMalloc(&d_ws, ws_bytes));
    if (zq_matmul(w, d_x, d_y, M, ZQ_ACT_Q8, NULL, NULL, 0, NULL) != ZQ_ERR_BAD_ARG) return 5; /* no workspace */
    CHECK(zq_matmul(w, d_x, d_y, M, ZQ_ACT_Q8, NULL, d_ws, ws_bytes, NULL));
    CUDA(cudaMemcpy(h_y, d_y, sizeof(float) * M * N, cudaMemcpyDeviceToHost));
    for (uint32_t r = 0; r < N; ++r) {
        const float want = (float)K * 0.5f * (float)((int)(r % 7) - 3);
        if (fabsf(h_y[r] - want) > 1e-3f * (fabsf(want) + 1.0f)) {
            fprintf(stderr, "q8 mode: y[%u] = %g, want %g\n", r, h_y[r], want);
            return 6;
        }
    }

    /* epilogue: bias + residual */
    float *d_bias = NULL, *h_b = (float*)malloc(sizeof(float) * N);
    for (uint32_t r = 0; r < N; ++r) h_b[r] = (float)r;
    CUDA(cudaMalloc((void**)&d_bias, sizeof(float) * N));
    CUDA(cudaMemcpy(d_bias, h_b, sizeof(float) * N, cudaMemcpyHostToDevice));
    zq_epilogue ep;
    memset(&ep, 0, sizeof(ep));
    ep.d_bias = d_bias;
    CHECK(zq_matmul(w, d_x, d_y, 1, ZQ_ACT_F32, &ep, NULL, 0, NULL));
    CUDA(cudaMemcpy(h_y, d_y, sizeof(float) * N, cudaMemcpyDeviceToHost));
    for (uint32_t r = 0; r < N; ++r)
        if (h_y[r] != (float)K * 0.5f * (float)((int)(r % 7) - 3) + (float)r) return 7;

    /* argmax, first maximum wins: rows 6, 13, ... all hold the maximum 3 * K / 2 */
    int32_t* d_idx = NULL; int32_t h_idx = -1;
    CUDA(cudaMalloc((void**)&d_idx, sizeof(int32_t)));
    CHECK(zq_matmul(w, d_x, d_y, 1, ZQ_ACT_F32, NULL, NULL, 0, NULL));
    CHECK(zq_argmax(d_y, N, d_idx, NULL));
    CUDA(cudaMemcpy(&h_idx, d_idx, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (h_idx != 6) return 8;

    /* errors are statuses, not aborts */
    zq_weight* bad = NULL;
    if (zq_weight_upload(raw, 6 /* q5_0 */, N, K, NULL, &bad) != ZQ_ERR_UNSUPPORTED) return 9;
    if (zq_weight_upload(raw, ZQ_TYPE_Q8_0, N, 48, NULL, &bad) != ZQ_ERR_BAD_ARG) return 9;
    unsigned int dev_err = 1;
    CHECK(zq_device_error(&dev_err, 0));
    if (dev_err != 0) return 10;
    if (zq_abi_version() < 1) return 11;

    CHECK(zq_weight_free(w));
    cudaFree(d_x); cudaFree(d_y); cudaFree(d_ws); cudaFree(d_bias); cudaFree(d_idx);
    free(raw); free(h_x); free(h_y); free(h_b);
    printf("c abi client ok\n");
    return 0;
}
