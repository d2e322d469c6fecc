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
