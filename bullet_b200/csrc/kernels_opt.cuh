// AdamW with fused weight clipping over the whole flat parameter buffer in one launch.
//
// Reference semantics (jw1912/bullet, crates/trainer/src/optimiser/adam.rs:35-52 and
// :117-136): per element, in this order and in fp32,
//     g  = adj * grad_sum            (adj = 1/batch, crates/trainer/src/run.rs:130-131)
//     p *= 1 - decay * rate
//     m  = beta1 * m + (1 - beta1) * g
//     v  = beta2 * v + (1 - beta2) * g * g
//     p -= rate * m / (sqrtf(v) + 1e-8)
//     p  = min(max(p, wmin), wmax)
// There is no bias correction.  The reference launches this once per weight tensor with the
// tensor's own hyper-parameters baked in; here one launch walks every tensor and looks its
// hyper-parameters up in a small segment table.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kMaxSegments = 12;

struct AdamSegment {
    long long begin4, end4;  // range in float4 units within the flat buffer
    float decay, beta1, beta2, wmin, wmax;
};

struct AdamArgs {
    float4* p;
    float4* m;
    float4* v;
    const float4* g;
    long long first4, total4;  // the launch covers float4 indices [first4, first4 + total4)
    int nseg;
    float rate, adj;
    AdamSegment seg[kMaxSegments];
};

__device__ __forceinline__ void adam_op(const AdamSegment& s, float rate, float g, float& p, float& m, float& v) {
    p *= 1.0f - s.decay * rate;
    m = s.beta1 * m + (1.0f - s.beta1) * g;
    v = s.beta2 * v + (1.0f - s.beta2) * g * g;
    const float val = m / (sqrtf(v) + 0.00000001f);
    p -= rate * val;
    p = fminf(fmaxf(p, s.wmin), s.wmax);
}

__global__ void __launch_bounds__(256) adamw_flat_kernel(const __grid_constant__ AdamArgs a) {
    for (long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x; j < a.total4;
         j += (long long)gridDim.x * blockDim.x) {
        const long long i = a.first4 + j;
        int si = -1;
#pragma unroll 1
        for (int k = 0; k < a.nseg; k++)
            if (i >= a.seg[k].begin4 && i < a.seg[k].end4) si = k;
        if (si < 0) continue;  // alignment padding between tensors
        const AdamSegment& s = a.seg[si];
        float4 p = a.p[i], m = a.m[i], v = a.v[i];
        const float4 g = a.g[i];
        adam_op(s, a.rate, a.adj * g.x, p.x, m.x, v.x);
        adam_op(s, a.rate, a.adj * g.y, p.y, m.y, v.y);
        adam_op(s, a.rate, a.adj * g.z, p.z, m.z, v.z);
        adam_op(s, a.rate, a.adj * g.w, p.w, m.w, v.w);
        a.p[i] = p;
        a.m[i] = m;
        a.v[i] = v;
    }
}

// Data-parallel update over peer memory: reduce-scatter, AdamW and all-gather in one launch.
// Every rank's gradient and parameter buffers are mapped into this process (CUDA IPC over
// NVLink).  A thread owns float4 index i of THIS rank's share of the flat buffer: it loads
// G_r[i] from every rank r with plain peer loads, sums them in rank order (one owner per
// element, so all replicas end up bit-identical), runs AdamW on the local p, m, v, and
// stores the new p into every rank's parameter buffer with plain peer stores.  The leading
// padding of the buffer carries the summed loss in float 0: its owner writes the reduced
// value into every rank's parameter buffer, which does not use those floats.
// With store_peers = 0 the new weights stay local: every rank then runs the SAME range and ends
// up with the same values (used for the small tensors, which every rank needs at once).
// The launch sits between two cross-rank fences: every rank's gradients complete before, every
// rank's launch complete after.  Either the caller provides them (any tiny collective), or
// wait_ready makes the kernel itself wait, bounded, for the peers' counters (see PeerFlags).
constexpr int kMaxRanks = 8;

// Cross-rank fences of the exchange, without a collective: every rank owns an array of counters
// that its peers write with release stores over NVLink and that it polls locally.
//   [kFlagReady + r]  rank r's gradients of step n are complete      (value n)
//   [kFlagDone + r]   rank r's exchange kernel of step n has finished (value n)
//   [kFlagTimeout]    a wait of this rank gave up
// Every wait is bounded (about four seconds); when it gives up it raises the timeout word, which the
// host reports with the step's loss, and the kernel carries on so that the stream never hangs.
constexpr int kFlagReady = 0, kFlagDone = kMaxRanks, kFlagTimeout = 2 * kMaxRanks, kFlagInts = 2 * kMaxRanks + 8;
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

// Called by one thread: waits until every rank has written at least `value` at `base`.
__device__ __forceinline__ bool peer_wait(const PeerFlags& f, int base, int value) {
    int* mine = f.flags[f.rank];
    long long spins = 0;  // one budget for all ranks together
    for (int r = 0; r < f.world; r++) {
        while (ld_acquire_sys(mine + base + r) < value) {
            __nanosleep(200);
            if (++spins > f.spin_limit) {
                atomicOr(mine + kFlagTimeout, 1);
                return false;
            }
        }
    }
    return true;
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

struct ExchangeArgs {
    AdamArgs adam;               // local p, m, v; first4 / total4 = this rank's share; g unused
    const float4* g[kMaxRanks];  // gradient buffer of every rank, own included, by rank
    float4* p_out[kMaxRanks];    // parameter buffer of every rank
    int world;
    int store_peers;             // 1: new weights go to every rank; 0: to this rank only (every rank runs the same range)
    long long head4;             // float4s of leading padding (the loss lives in the first)
    PeerFlags flags;
    int wait_ready;              // > 0: every CTA first waits until all ranks signalled this value at kFlagReady
};

// 128 threads and at most 64 registers: one such CTA still fits on an SM beside a 1024-thread
// feature-transformer CTA, so the exchange can run under those kernels instead of in their place.
// WORLD > 0 fixes the number of ranks at compile time; a thread then takes 8 / WORLD float4s per
// round, so that about eight 16-byte loads per thread are in flight over NVLink whatever the
// number of ranks (remote latency is microseconds).  WORLD = 0: any number of ranks up to 8.
template <int WORLD>
__global__ void __launch_bounds__(128, 8) adamw_exchange_kernel(const __grid_constant__ ExchangeArgs x) {
    constexpr int W = WORLD > 0 ? WORLD : kMaxRanks;  // loads held per element
    constexpr int U = WORLD > 0 ? kMaxRanks / WORLD : 1;  // elements per thread and round
    const AdamArgs& a = x.adam;
    if (x.wait_ready > 0) {
        if (threadIdx.x == 0) peer_wait(x.flags, kFlagReady, x.wait_ready);
        __syncthreads();
    }
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long j0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; j0 < a.total4; j0 += stride * U) {
        float4 gr[U][W];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const long long j = j0 + u * stride;
#pragma unroll
            for (int r = 0; r < W; r++)
                if (j < a.total4 && r < x.world) gr[u][r] = x.g[r][a.first4 + j];  // all loads in flight before the first add
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const long long j = j0 + u * stride;
            if (j >= a.total4) break;
            const long long i = a.first4 + j;
            float4 g = gr[u][0];
#pragma unroll
            for (int r = 1; r < W; r++)
                if (r < x.world) g.x += gr[u][r].x, g.y += gr[u][r].y, g.z += gr[u][r].z, g.w += gr[u][r].w;
            int si = -1;
#pragma unroll 1
            for (int k = 0; k < a.nseg; k++)
                if (i >= a.seg[k].begin4 && i < a.seg[k].end4) si = k;
            float4 p;
            if (si < 0) {
                if (i >= x.head4) continue;  // alignment padding between tensors
                p = g;                       // the summed loss (and zeros)
            } else {
                const AdamSegment& s = a.seg[si];
                p = a.p[i];
                float4 m = a.m[i], v = a.v[i];
                adam_op(s, a.rate, a.adj * g.x, p.x, m.x, v.x);
                adam_op(s, a.rate, a.adj * g.y, p.y, m.y, v.y);
                adam_op(s, a.rate, a.adj * g.z, p.z, m.z, v.z);
                adam_op(s, a.rate, a.adj * g.w, p.w, m.w, v.w);
                a.m[i] = m;
                a.v[i] = v;
            }
            if (x.store_peers) {
#pragma unroll
                for (int r = 0; r < W; r++)
                    if (r < x.world) x.p_out[r][i] = p;
            } else {
                a.p[i] = p;
            }
        }
    }
}

}  // namespace b200
