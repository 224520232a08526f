// Carry exchange between sequence shards through peer memory (NVLink), without a collective.
//
// Every rank owns an inbox in its own memory: for each of four slots (direction x parity of the
// call counter) one (first, second) aggregate pair per rank, plus one flag word per rank and slot.
// After its aggregate kernel a rank PUSHES its pair into the inbox of every rank with plain stores
// through peer pointers and then sets its flag there to the call's epoch (release at system scope).
// The kernel that computes a rank's carry-in waits - bounded - until the flags of ALL ranks show the
// epoch (acquire at system scope) and folds the pairs of the ranks it depends on in rank order with
// the scan's combine, the same expression carry_fold_kernel evaluates after an all-gather, so both
// ways of exchanging give bit-identical carries.
//
// A slot is reused two calls later.  A rank that pushes call e+2 has passed the wait of call e+1,
// which needed every rank's push of call e+1, and a rank issues that push (same stream) only after
// its own fold of call e has finished reading the slot: no rank can overwrite data that is still
// being read, whatever mix of forward and backward calls the ranks make (waiting only for the ranks
// a fold depends on would let the first rank of a forward-only loop run ahead of its readers).
//
// Only loads and stores on peer memory; no bulk-copy engine, no multicast.
#pragma once
#include "qssm_tile.cuh"

namespace qssm {

constexpr int MAX_PEERS = 16;
constexpr int PEER_SLOTS = 4;

struct PeerPushParams {
    const float* first;   // [n_chan]
    const float* second;  // [n_chan]
    float* inbox[MAX_PEERS];  // base of every rank's inbox  [PEER_SLOTS][world][2][n_chan]
    int* flags[MAX_PEERS];    // base of every rank's flags  [PEER_SLOTS][world]
    unsigned int* counters;   // [world] local arrival counters, zero between calls
    long long n_chan;
    int rank, world, slot, epoch;
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// grid (ctas_per_peer, world): the CTAs of column `peer` copy this rank's pair into that rank's inbox;
// the last of them to finish publishes the flag.
static __global__ void carry_push_kernel(const PeerPushParams p) {
    const int peer = blockIdx.y;
    float* dst = p.inbox[peer] + (((long long)p.slot * p.world + p.rank) * 2) * p.n_chan;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < p.n_chan;
         i += (long long)gridDim.x * blockDim.x) {
        dst[i] = p.first[i];
        dst[p.n_chan + i] = p.second[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(p.counters + peer, 1u);
        if (prev == gridDim.x - 1) {
            p.counters[peer] = 0;
            __threadfence_system();
            st_release_sys(p.flags[peer] + p.slot * p.world + p.rank, p.epoch);
        }
    }
}

// carry[c] = the pairs of the ranks before (reverse: after) `rank`, folded in rank order onto seed[c]
static __global__ void carry_wait_fold_kernel(const float* inbox, const int* flags, long long n_chan, int rank, int world,
                                              int slot, int epoch, int reverse, const float* seed, float* carry,
                                              unsigned long long wait_ns, int* status) {
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        bool good = true;
        const unsigned long long start = global_timer_ns();
        for (int k = 0; k < world && good; ++k) {
            const int* f = flags + slot * world + k;
            for (unsigned int it = 0; ld_acquire_sys(f) != epoch; ++it) {
                __nanosleep(200);
                if ((it & 63u) == 63u && global_timer_ns() - start > wait_ns) {
                    good = false;
                    break;
                }
            }
        }
        s_ok = good ? 1 : 0;
    }
    __syncthreads();
    if (s_ok == 0) {
        if (threadIdx.x == 0) report(status, QSSM_S_TMA_TIMEOUT);
        return;
    }
    const float* base = inbox + (long long)slot * world * 2 * n_chan;
    for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < n_chan;
         c += (long long)gridDim.x * blockDim.x) {
        float run = seed != nullptr ? seed[c] : 0.f;
        if (!reverse) {
            for (int k = 0; k < rank; ++k) {
                const float* pr = base + (long long)k * 2 * n_chan;
                run = fmaf(__ldcg(pr + c), run, __ldcg(pr + n_chan + c));
            }
        } else {
            for (int k = world - 1; k > rank; --k) {
                const float* pr = base + (long long)k * 2 * n_chan;
                run = fmaf(__ldcg(pr + c), run, __ldcg(pr + n_chan + c));
            }
        }
        carry[c] = run;
    }
}

}  // namespace qssm
