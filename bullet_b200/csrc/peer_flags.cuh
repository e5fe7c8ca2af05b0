// Cross-rank fences of the data-parallel exchange, without a collective: counters that the ranks of one
// box write into each other's memory over NVLink (one process per GPU, buffers mapped with CUDA IPC) and
// poll locally.  Shared by the optimiser kernels and by the feature-transformer backward, whose CTAs
// announce finished table row blocks.  New work: the reference trains on one device.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kMaxRanks = 8;

// Every rank owns an array of counters that its peers write with release stores and that it polls:
//   [kFlagReady + r]  rank r's gradients of step n are complete      (value n)
//   [kFlagDone + r]   rank r's exchange kernel of step n has finished (value n)
//   [kFlagTimeout]    a wait of this rank, or of a peer, gave up; the next three ints say which wait of this rank
//   [kFlagBucket + b * kMaxRanks + r]  rank r's gradient of table row block b of step n is complete
// Every wait is bounded (about four seconds).  A wait that gives up raises the timeout word here and,
// with a plain peer store, on every other rank, so that each rank's host sees the failed step with its
// loss; the exchange kernels then return without touching parameters, optimiser state or peer memory,
// and the stream carries on, so nothing ever hangs.
constexpr int kFlagReady = 0, kFlagDone = kMaxRanks, kFlagTimeout = 2 * kMaxRanks, kFlagBucket = 2 * kMaxRanks + 8;
constexpr int kMaxSignalBlocks = 256;  // row blocks whose completion can be signalled one by one
constexpr int kFlagInts = kFlagBucket + kMaxSignalBlocks * kMaxRanks;
constexpr long long kPeerWaitSpins = 20000000;  // default spin_limit

struct PeerFlags {
    int* flags[kMaxRanks];  // every rank's counter array, own included, by rank
    int world, rank;
    long long spin_limit;   // polls (each at least 200 ns apart) before a wait gives up
};

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Called by one thread: waits until every rank has written at least `value` at `base`.  Gives up when
// the budget runs out or when another wait on this GPU has already given up; then tells every rank.
__device__ __forceinline__ bool peer_wait(const PeerFlags& f, int base, int value) {
    int* mine = f.flags[f.rank];
    long long spins = 0;  // one budget for all ranks together
    for (int r = 0; r < f.world; r++) {
        while (ld_acquire_sys(mine + base + r) < value) {
            __nanosleep(200);
            const bool spent = ++spins > f.spin_limit;
            if (spent || ((spins & 63) == 0 && ld_acquire_sys(mine + kFlagTimeout) != 0)) {
                if (spent) {
                    // what was missing, for the host's message: which counter, which value, whose
                    mine[kFlagTimeout + 1] = base;
                    mine[kFlagTimeout + 2] = value;
                    mine[kFlagTimeout + 3] = r;
                    for (int q = 0; q < f.world; q++) *(volatile int*)(f.flags[q] + kFlagTimeout) = 1;  // own word included
                }
                return false;
            }
        }
    }
    return true;
}
// The same for a whole CTA: thread 0 waits, every thread learns the outcome.
__device__ __forceinline__ bool peer_wait_cta(const PeerFlags& f, int base, int value) {
    __shared__ int arrived;
    __syncthreads();  // the previous use of `arrived` has been read by everyone
    if (threadIdx.x == 0) arrived = peer_wait(f, base, value) ? 1 : 0;
    __syncthreads();
    return arrived != 0;
}

// Everything this rank's stream has done so far is complete: tell every rank.  grid = 1, block = 32.
static __global__ void peer_signal_kernel(PeerFlags f, int base, int value) {
    if ((int)threadIdx.x < f.world) {
        __threadfence_system();
        st_release_sys(f.flags[threadIdx.x] + base + f.rank, value);
    }
}
// The stream goes on only after every rank has signalled `value` at `base` (or the wait gave up).
static __global__ void peer_wait_kernel(PeerFlags f, int base, int value) {
    if (threadIdx.x == 0) peer_wait(f, base, value);
}

struct BucketSignal {
    int* done_count;         // [nblocks] CTAs of the backward that have finished, per block; null = no signalling
    const int* done_expect;  // [nblocks] CTAs the running launch has per block
    const PeerFlags* peers;  // in device memory
    int value;
};

// The count itself, by one thread, once all reductions of the CTA into `block` are ordered before it (a fence by
// every thread that issued them, then a barrier): the CTA that completes the count tells every rank.
__device__ __forceinline__ void bucket_count_off(const BucketSignal& s, int block) {
    const int before = atomicAdd(s.done_count + block, 1);
    if (before + 1 == s.done_expect[block]) {
        s.done_count[block] = 0;  // ready for the next launch
        __threadfence_system();
        const PeerFlags& f = *s.peers;
        for (int r = 0; r < f.world; r++) st_release_sys(f.flags[r] + kFlagBucket + block * kMaxRanks + f.rank, s.value);
    }
}

// A whole CTA leaves `block`: every thread's reductions are ordered before the count.
__device__ __forceinline__ void bucket_signal(const BucketSignal& s, int block) {
    if (!s.done_count) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) bucket_count_off(s, block);
}

// Blocks without any work item in this launch: nothing will ever count them, announce them now.
static __global__ void bucket_presignal_kernel(BucketSignal s, int nblocks) {
    const PeerFlags& f = *s.peers;
    for (int b = threadIdx.x; b < nblocks; b += blockDim.x)
        if (s.done_expect[b] == 0) {
            __threadfence_system();
            for (int r = 0; r < f.world; r++) st_release_sys(f.flags[r] + kFlagBucket + b * kMaxRanks + f.rank, s.value);
        }
}

}  // namespace b200
