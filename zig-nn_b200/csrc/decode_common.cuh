// Helpers shared by the persistent decode kernels (decode_gemma.cu, decode_gpt2.cu): the consumers' named
// barrier, mbarrier and bulk-copy wrappers, the exchange words CTAs pass values in, reciprocal division.
// Everything is `static`-like (in an unnamed namespace of the including file's namespace zq::dk).
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace zq {
namespace dk {
namespace {

constexpr int kConsumerWarps = 16;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;           // + the producer warp
constexpr unsigned int kErrExchange = 0x58434847u;  // 'XCHG'
constexpr unsigned int kErrUnitWait = 0x554E4954u;  // 'UNIT'
constexpr uint32_t kPollLimit = 1u << 21;
constexpr uint32_t kSlotSpinLimit = 1u << 22;
// Serial chains (ordered sums) run on warp 1, not warp 0: the producer warp (16) shares warp 0's scheduler, and
// its polling takes issue slots that a chain of dependent adds feels one for one.
constexpr int kChainWarp = 1;
constexpr int kChainTid = kChainWarp * 32;

// ---- small device helpers --------------------------------------------------------------------

__device__ __forceinline__ void cbar() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }
// The consumers' barrier with an OR over a flag of every thread: all get the same answer from one barrier.
__device__ __forceinline__ bool cbar_or(bool v) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)v), "n"(kConsumers)
        : "memory");
    return r != 0;
}

__device__ __noinline__ float exp_f32(float x) { return (float)exp((double)x); }
__device__ __noinline__ float gelu_tanh(float v) {
    const float cube = __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, v), v), v);
    const float inner = __fmul_rn(0.7978845608f, __fadd_rn(v, cube));
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, (float)tanh((double)inner)));
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
    return v;
}
__device__ __forceinline__ uint32_t pick(const uint4& v, int j) {
    return j == 0 ? v.x : j == 1 ? v.y : j == 2 ? v.z : v.w;
}
// n / d and n % d with magic = floor(2^32 / d) (0xFFFFFFFF for d = 1) from the host: the product's high word is
// the quotient or one less; a 32-bit division instruction sequence costs 65-95 cycles on this part.
__device__ __forceinline__ void fast_divmod(uint32_t n, uint32_t d, uint32_t magic, uint32_t& q, uint32_t& r) {
    q = __umulhi(n, magic);
    r = n - q * d;
    if (r >= d) {
        r -= d;
        q += 1;
    }
}
__device__ __forceinline__ int quad_transpose_reduce(const int (&p)[4], int t) {
    const bool upper = t & 2;
    const int keep0 = upper ? p[2] : p[0], keep1 = upper ? p[3] : p[1];
    const int send0 = upper ? p[0] : p[2], send1 = upper ? p[1] : p[3];
    const int a0 = keep0 + __shfl_xor_sync(0xFFFFFFFFu, send0, 2);
    const int a1 = keep1 + __shfl_xor_sync(0xFFFFFFFFu, send1, 2);
    const bool odd = t & 1;
    const int keep = odd ? a1 : a0, send = odd ? a0 : a1;
    return keep + __shfl_xor_sync(0xFFFFFFFFu, send, 1);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}
// The same with a suspend-time hint (nanoseconds): the thread may sleep in hardware until the phase completes
// or the time has passed, instead of occupying the shared-memory pipeline with polls.
__device__ __forceinline__ uint32_t mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_gpu_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// One exchange word: a naturally aligned 64-bit store / load is a single memory operation.
__device__ __forceinline__ void xstore(unsigned long long* p, float v, uint32_t epoch) {
    const unsigned long long w = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void xstore_u32(unsigned long long* p, uint32_t v, uint32_t epoch) {
    const unsigned long long w = ((unsigned long long)epoch << 32) | (unsigned long long)v;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long xload(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}

}  // namespace
}  // namespace dk
}  // namespace zq
