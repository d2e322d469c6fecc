// All-gather of the output slices of a row-sharded linear, written as plain peer stores over NVLink.
//
// Each rank owns rows [lo, hi) of the weight and therefore the slice y[:, lo:hi] of the result
// (zig-nn's CPU pool splits rows the same way, src/gguf/thread_pool.zig:96-181). Instead of handing the
// slices to a library collective, the rank copies its slice into every peer's result buffer itself
// (128-bit stores to peer-mapped memory), publishes a counter on the peer, and waits — bounded — until
// every peer's counter for this round has reached it. One launch, (world - 1) x kCtasPerPeer CTAs.
//
// Protocol. flags[r] on rank q counts the CTAs of rank r that have finished writing into q's buffer:
// after its stores a CTA executes a system-scope fence and adds 1 to the peer's counter, so round e is
// complete on q when flags[r] >= e * kCtasPerPeer for every r. Counters only grow; nothing is reset.
// The caller alternates two result buffers between rounds, so a peer that is one round ahead never
// overwrites a buffer that is still being read. No multicast, no loads from peer memory.
#include "zq_internal.h"

namespace zq {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kCtasPerPeer = 8;
constexpr uint32_t kSpinLimit = 1u << 20;              // polls of a flag before giving up (about a second)
constexpr unsigned int kErrGatherTimeout = 0x47415448u;  // 'GATH'

struct PeerTable {
    float* y[2][kMaxWorld];  // two result buffers, used by odd / even rounds
    uint32_t* flags[kMaxWorld];
};

// The round number lives in device memory so that a captured launch sequence can be replayed.
__global__ void bump_round_kernel(uint32_t* round_ctr) { *round_ctr += 1; }

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256)
peer_gather_kernel(PeerTable tab, uint32_t world, uint32_t rank, size_t slice_off, size_t slice_len,
                   uint32_t round_arg, const uint32_t* __restrict__ round_ctr, unsigned int* err_word,
                   uint32_t spin_limit) {
    const uint32_t round = round_ctr ? *round_ctr : round_arg;
    const uint32_t pi = blockIdx.x / kCtasPerPeer, chunk = blockIdx.x % kCtasPerPeer;
    const uint32_t peer = pi < rank ? pi : pi + 1;  // the peers in rank order, skipping this rank
    const float* src = tab.y[round & 1u][rank] + slice_off;
    float* dst = tab.y[round & 1u][peer] + slice_off;

    // this CTA's share of the slice, in 16-byte units where alignment allows
    const size_t per = (slice_len + kCtasPerPeer - 1) / kCtasPerPeer;
    const size_t per4 = (per + 3) & ~(size_t)3;
    const size_t lo = min(slice_len, (size_t)chunk * per4), hi = min(slice_len, lo + per4);
    const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0;
    if (vec) {
        const size_t n4 = (hi - lo) / 4;
        const float4* s4 = reinterpret_cast<const float4*>(src + lo);
        float4* d4 = reinterpret_cast<float4*>(dst + lo);
        for (size_t i = threadIdx.x; i < n4; i += blockDim.x) d4[i] = s4[i];
        for (size_t i = lo + n4 * 4 + threadIdx.x; i < hi; i += blockDim.x) dst[i] = src[i];
    } else {
        for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) dst[i] = src[i];
    }
    __threadfence_system();  // the stores above are visible system-wide before the counter moves
    __syncthreads();
    if (threadIdx.x == 0) {
        atomicAdd_system(tab.flags[peer] + rank, 1u);
        if (chunk == 0) {
            // wait for this peer's CTAs of the same round to have written into our buffer
            const uint32_t want = round * kCtasPerPeer;
            const uint32_t* f = tab.flags[rank] + peer;
            bool ok = false;
            for (uint32_t i = 0; i < spin_limit; ++i) {
                if ((int32_t)(ld_acquire_sys(f) - want) >= 0) {
                    ok = true;
                    break;
                }
                __nanosleep(64);
            }
            if (!ok) atomicExch(err_word, kErrGatherTimeout);
        }
    }
}

// Several activation rows: rank r owns the COLUMNS [col_off, col_off + per) of the [m_rows][n_total] result. Its
// [m_rows][per] block goes straight to that place in every rank's result buffer (its own included), so what a
// rank holds afterwards is the row-major result itself, not [world][m_rows][per] to be permuted.
// kColCtas CTAs per destination share the rows; the counters work as above with kColCtas arrivals per round.
constexpr int kColCtas = 32;

__global__ void __launch_bounds__(512)
peer_gather_cols_kernel(PeerTable tab, uint32_t world, uint32_t rank, const float* __restrict__ local, uint32_t m_rows,
                        size_t n_total, size_t col_off, uint32_t per, uint32_t round_arg,
                        const uint32_t* __restrict__ round_ctr, unsigned int* err_word, uint32_t spin_limit) {
    const uint32_t round = round_ctr ? *round_ctr : round_arg;
    const uint32_t dest = blockIdx.x / kColCtas, chunk = blockIdx.x % kColCtas;
    float* dst = tab.y[round & 1u][dest] + col_off;
    const uint32_t rows_per = (m_rows + kColCtas - 1) / kColCtas;
    const uint32_t r0 = min(m_rows, chunk * rows_per), r1 = min(m_rows, r0 + rows_per);
    const bool vec = ((reinterpret_cast<uintptr_t>(local) | reinterpret_cast<uintptr_t>(dst)) & 15u) == 0 &&
                     (per & 3u) == 0 && (n_total & 3u) == 0;
    if (vec) {
        const uint32_t per4 = per / 4;
        const size_t total = (size_t)(r1 - r0) * per4;
        for (size_t i = threadIdx.x; i < total; i += blockDim.x) {
            const size_t r = r0 + i / per4, c = (i % per4) * 4;
            *reinterpret_cast<float4*>(dst + r * n_total + c) = *reinterpret_cast<const float4*>(local + r * per + c);
        }
    } else {
        const size_t total = (size_t)(r1 - r0) * per;
        for (size_t i = threadIdx.x; i < total; i += blockDim.x) {
            const size_t r = r0 + i / per, c = i % per;
            dst[r * n_total + c] = local[r * per + c];
        }
    }
    if (dest == rank) return;  // this GPU's own copy needs no publication
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        atomicAdd_system(tab.flags[dest] + rank, 1u);
        if (chunk == 0) {
            const uint32_t want = round * kColCtas;
            const uint32_t* f = tab.flags[rank] + dest;
            bool ok = false;
            for (uint32_t i = 0; i < spin_limit; ++i) {
                if ((int32_t)(ld_acquire_sys(f) - want) >= 0) {
                    ok = true;
                    break;
                }
                __nanosleep(64);
            }
            if (!ok) atomicExch(err_word, kErrGatherTimeout);
        }
    }
}

}  // namespace
}  // namespace zq

using namespace zq;

static int peer_gather_launch(float* const* y_odd, float* const* y_even, uint32_t* const* h_flag_peers,
                              uint32_t world, uint32_t rank, size_t slice_offset, size_t slice_len, uint32_t round,
                              uint32_t* d_round, cudaStream_t st) {
    PeerTable tab{};
    for (uint32_t r = 0; r < world; ++r) {
        if (!y_odd[r] || !y_even[r] || !h_flag_peers[r]) return ZQ_ERR_PEER;  // a peer's buffer was never mapped
        tab.y[1][r] = y_odd[r];
        tab.y[0][r] = y_even[r];
        tab.flags[r] = h_flag_peers[r];
    }
    unsigned int* err_word = nullptr;
    int rc = device_error_word(&err_word);
    if (rc != ZQ_OK) return rc;
    if (d_round) {
        bump_round_kernel<<<1, 1, 0, st>>>(d_round);
        ZQ_LAUNCH_CHECK();
    }
    peer_gather_kernel<<<(world - 1) * kCtasPerPeer, 256, 0, st>>>(tab, world, rank, slice_offset, slice_len, round,
                                                                    d_round, err_word, wait_limit() ? wait_limit() : kSpinLimit);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}

extern "C" int zq_peer_gather(float* const* h_y_peers, uint32_t* const* h_flag_peers, uint32_t world,
                              uint32_t rank, size_t slice_offset, size_t slice_len, uint32_t round,
                              zq_stream stream) {
    if (!h_y_peers || !h_flag_peers || world == 0 || world > (uint32_t)kMaxWorld || rank >= world || round == 0)
        return ZQ_ERR_BAD_ARG;
    if (world == 1) return ZQ_OK;
    return peer_gather_launch(h_y_peers, h_y_peers, h_flag_peers, world, rank, slice_offset, slice_len, round,
                              nullptr, as_stream(stream));
}

extern "C" int zq_peer_gather_step(float* const* h_y_peers_odd, float* const* h_y_peers_even,
                                   uint32_t* const* h_flag_peers, uint32_t world, uint32_t rank,
                                   size_t slice_offset, size_t slice_len, uint32_t* d_round, zq_stream stream) {
    if (!h_y_peers_odd || !h_y_peers_even || !h_flag_peers || !d_round || world == 0 ||
        world > (uint32_t)kMaxWorld || rank >= world)
        return ZQ_ERR_BAD_ARG;
    if (world == 1) return ZQ_OK;
    return peer_gather_launch(h_y_peers_odd, h_y_peers_even, h_flag_peers, world, rank, slice_offset, slice_len, 0,
                              d_round, as_stream(stream));
}

extern "C" int zq_peer_gather_cols_step(float* const* h_y_peers_odd, float* const* h_y_peers_even,
                                        uint32_t* const* h_flag_peers, uint32_t world, uint32_t rank,
                                        const float* d_local, uint32_t m_rows, size_t n_total, size_t col_offset,
                                        uint32_t cols, uint32_t* d_round, zq_stream stream) {
    if (!h_y_peers_odd || !h_y_peers_even || !h_flag_peers || !d_local || !d_round || world == 0 ||
        world > (uint32_t)kMaxWorld || rank >= world || m_rows == 0 || cols == 0 || col_offset + cols > n_total)
        return ZQ_ERR_BAD_ARG;
    PeerTable tab{};
    for (uint32_t r = 0; r < world; ++r) {
        if (!h_y_peers_odd[r] || !h_y_peers_even[r] || !h_flag_peers[r]) return ZQ_ERR_PEER;
        tab.y[1][r] = h_y_peers_odd[r];
        tab.y[0][r] = h_y_peers_even[r];
        tab.flags[r] = h_flag_peers[r];
    }
    unsigned int* err_word = nullptr;
    int rc = device_error_word(&err_word);
    if (rc != ZQ_OK) return rc;
    cudaStream_t st = as_stream(stream);
    bump_round_kernel<<<1, 1, 0, st>>>(d_round);
    ZQ_LAUNCH_CHECK();
    peer_gather_cols_kernel<<<world * kColCtas, 512, 0, st>>>(tab, world, rank, d_local, m_rows, n_total, col_offset, cols, 0,
                                                             d_round, err_word, wait_limit() ? wait_limit() : kSpinLimit);
    ZQ_LAUNCH_CHECK();
    return ZQ_OK;
}
