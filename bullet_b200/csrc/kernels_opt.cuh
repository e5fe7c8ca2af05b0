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

#include "peer_flags.cuh"

namespace b200 {

constexpr int kMaxSegments = 12;

struct AdamSegment {
    long long begin4, end4;  // range in float4 units within the flat buffer
    float decay, beta1, beta2, wmin, wmax;
    // RAdam (crates/trainer/src/optimiser/radam.rs:35-52,295-314): the host computes, per step, a factor on
    // the learning rate and whether the second moment divides the update yet.  AdamW: 1 and yes.
    float rate_scale = 1.0f;
    int use_denom = 1;
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

__device__ __forceinline__ void adam_op(const AdamSegment& s, float base_rate, float g, float& p, float& m, float& v) {
    const float rate = base_rate * s.rate_scale;  // radam.rs: rate_ptr[0] * step_size_ptr[0]; AdamW: times one
    p *= 1.0f - s.decay * rate;
    m = s.beta1 * m + (1.0f - s.beta1) * g;
    v = s.beta2 * v + (1.0f - s.beta2) * g * g;
    float val = m;
    if (s.use_denom) val /= sqrtf(v) + 0.00000001f;
    p -= rate * val;
    p = fminf(fmaxf(p, s.wmin), s.wmax);
}

// Ranger's lookahead (crates/trainer/src/optimiser/ranger.rs:23-43), every k-th step, on the tensors that use
// it: w = alpha * w + (1 - alpha) * slow, and slow takes the same value.  `one_minus[k]` is 1 - alpha of
// segment k as the host evaluates it; segments with alpha < 0 are left alone.
struct LookaheadArgs {
    float4* p;
    float4* slow;
    long long total4;
    int nseg;
    long long begin4[kMaxSegments], end4[kMaxSegments];
    float alpha[kMaxSegments], one_minus[kMaxSegments];
};
static __global__ void __launch_bounds__(256) lookahead_kernel(const __grid_constant__ LookaheadArgs a) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < a.total4; i += (long long)gridDim.x * blockDim.x) {
        int si = -1;
#pragma unroll 1
        for (int k = 0; k < a.nseg; k++)
            if (i >= a.begin4[k] && i < a.end4[k] && a.alpha[k] >= 0.f) si = k;
        if (si < 0) continue;
        const float4 w = a.p[i], s = a.slow[i];
        const float al = a.alpha[si], om = a.one_minus[si];
        const float4 n = make_float4(__fadd_rn(__fmul_rn(al, w.x), __fmul_rn(om, s.x)), __fadd_rn(__fmul_rn(al, w.y), __fmul_rn(om, s.y)),
                                     __fadd_rn(__fmul_rn(al, w.z), __fmul_rn(om, s.z)), __fadd_rn(__fmul_rn(al, w.w), __fmul_rn(om, s.w)));
        a.p[i] = n;
        a.slow[i] = n;
    }
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
    // a fence that gave up means some rank's gradients may be incomplete: leave everything as it is
    if (x.wait_ready > 0 && !peer_wait_cta(x.flags, kFlagReady, x.wait_ready)) return;
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

// ---------------------------------------------------------------------------------------------
// The same exchange with every operand moved by bulk asynchronous copies (cp.async.bulk, the TMA engine
// without a tensor map) instead of per-thread loads and stores: no registers and no load slots are held
// while a tile is under way, everything a tile needs is requested several tiles ahead, and the stores leave
// asynchronously as well.  Measured, it is as fast as the per-thread kernel and no faster (alone on eight
// GPUs 0.293 against 0.300 ms, on two 0.184 against 0.189 ms): the exchange is bound by the links, which per
// direction carry this rank's own transfers plus its peers' (pulled gradients in and pushed weights out, the
// replies to the peers' pulls out and their pushed weights in), at 87 % of the rate of a peer copy.  Off by
// default (option "exchange_bulk").
// One CTA per SM; the rank's share is cut into tiles of kBulkTile float4s, one per thread.  Per tile and
// stage thread 0 arms the stage's mbarrier with the byte count and issues one bulk load per rank (that
// rank's gradients of the tile, peer memory -> this CTA's shared memory) and three for the local p, m and v;
// kBulkStages tiles are in flight.  When the barrier flips every thread sums its float4 over the ranks in
// rank order, runs AdamW, and puts the new p, m, v into the stage's three output lines; after a proxy fence
// and a barrier thread 0 sends p to every rank's parameter buffer and m, v home, one bulk store each.
// No multicast, no tensor maps, no cluster: plain bulk copies of linear memory.
// Every wait is bounded: an mbarrier that does not flip within the budget raises the timeout word on every
// rank (detail code -2), the CTA waits for its stores and leaves.
template <int WORLD, int kBulkTile, int kBulkStages>
__host__ __device__ constexpr size_t exchange_bulk_smem() {
    return (size_t)kBulkStages * ((WORLD > 0 ? WORLD : kMaxRanks) + 6) * kBulkTile * sizeof(float4) + kBulkStages * 8;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int WORLD, int kBulkTile, int kBulkStages>
__global__ void __launch_bounds__(kBulkTile, 1) adamw_exchange_bulk_kernel(const __grid_constant__ ExchangeArgs x) {
    constexpr int W = WORLD > 0 ? WORLD : kMaxRanks;
    constexpr int kIn = W + 3, kOut = 3;  // lines per stage: gradients by rank, p, m, v; new p, m, v
    extern __shared__ __align__(128) unsigned char bulk_smem[];
    float4* in = reinterpret_cast<float4*>(bulk_smem);                  // [stage][kIn][kBulkTile]
    float4* out = in + (size_t)kBulkStages * kIn * kBulkTile;           // [stage][kOut][kBulkTile]
    uint64_t* bar = reinterpret_cast<uint64_t*>(out + (size_t)kBulkStages * kOut * kBulkTile);
    __shared__ int gave_up;
    const AdamArgs& a = x.adam;
    if (x.wait_ready > 0 && !peer_wait_cta(x.flags, kFlagReady, x.wait_ready)) return;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kBulkStages; s++) mbar_init(bar + s, 1);
        gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const long long tiles = (a.total4 + kBulkTile - 1) / kBulkTile;
    auto fetch = [&](long long tile, int stage) {  // thread 0
        const long long j0 = tile * kBulkTile, i0 = a.first4 + j0;
        const uint32_t bytes = (uint32_t)min((long long)kBulkTile, a.total4 - j0) * 16u;
        float4* dst = in + (size_t)stage * kIn * kBulkTile;
        mbar_expect_tx(bar + stage, bytes * (uint32_t)(x.world + 3));
        for (int r = 0; r < x.world; r++) bulk_load(dst + (size_t)r * kBulkTile, x.g[r] + i0, bytes, bar + stage);
        bulk_load(dst + (size_t)W * kBulkTile, a.p + i0, bytes, bar + stage);
        bulk_load(dst + (size_t)(W + 1) * kBulkTile, a.m + i0, bytes, bar + stage);
        bulk_load(dst + (size_t)(W + 2) * kBulkTile, a.v + i0, bytes, bar + stage);
    };
    if (threadIdx.x == 0)
        for (int s = 0; s < kBulkStages; s++) {
            const long long tile = blockIdx.x + (long long)s * gridDim.x;
            if (tile < tiles) fetch(tile, s);
        }
    long long k = 0;
    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x, k++) {
        const int stage = (int)(k % kBulkStages);
        const uint32_t parity = (uint32_t)((k / kBulkStages) & 1);
        const long long j = tile * kBulkTile + threadIdx.x, i = a.first4 + j;
        const bool live = j < a.total4;
        int si = -1;
        if (live) {
#pragma unroll 1
            for (int q = 0; q < a.nseg; q++)
                if (i >= a.seg[q].begin4 && i < a.seg[q].end4) si = q;
        }
        // the stores that last read this stage's output lines (tile k - kBulkStages) have left shared memory
        if (threadIdx.x == 0) bulk_wait_read<kBulkStages - 1>();
        {   // wait for this tile's operands, bounded
            long long spins = 0;
            while (!mbar_try_wait(bar + stage, parity)) {
                if (++spins > x.flags.spin_limit) {
                    gave_up = 1;
                    break;
                }
                if ((spins & 1023) == 0 && *(volatile int*)&gave_up) break;
            }
        }
        __syncthreads();
        if (*(volatile int*)&gave_up) {
            if (threadIdx.x == 0) {
                int* mine = x.flags.flags[x.flags.rank];
                mine[kFlagTimeout + 1] = -2;
                mine[kFlagTimeout + 2] = (int)tile;
                mine[kFlagTimeout + 3] = x.flags.rank;
                for (int q = 0; q < x.flags.world; q++) *(volatile int*)(x.flags.flags[q] + kFlagTimeout) = 1;
                bulk_wait_all();
            }
            return;
        }
        float4* dst = out + (size_t)stage * kOut * kBulkTile + threadIdx.x;
        if (live) {
            const float4* src = in + (size_t)stage * kIn * kBulkTile + threadIdx.x;
            float4 g = src[0];
#pragma unroll
            for (int r = 1; r < W; r++)
                if (r < x.world) {
                    const float4 t = src[(size_t)r * kBulkTile];
                    g.x += t.x, g.y += t.y, g.z += t.z, g.w += t.w;
                }
            float4 p = src[(size_t)W * kBulkTile], m = src[(size_t)(W + 1) * kBulkTile], v = src[(size_t)(W + 2) * kBulkTile];
            if (si >= 0) {
                const AdamSegment& s = a.seg[si];
                adam_op(s, a.rate, a.adj * g.x, p.x, m.x, v.x);
                adam_op(s, a.rate, a.adj * g.y, p.y, m.y, v.y);
                adam_op(s, a.rate, a.adj * g.z, p.z, m.z, v.z);
                adam_op(s, a.rate, a.adj * g.w, p.w, m.w, v.w);
            } else if (i < x.head4) {
                p = g;  // the summed loss (and zeros)
            }           // else: alignment padding between tensors keeps what it holds
            dst[0] = p;
            dst[kBulkTile] = m;
            dst[2 * kBulkTile] = v;
        }
        fence_proxy_async();  // the output lines must be visible to the bulk stores
        __syncthreads();      // ... and every thread has read this stage's operands
        if (threadIdx.x == 0) {
            const long long j0 = tile * kBulkTile, i0 = a.first4 + j0;
            const uint32_t bytes = (uint32_t)min((long long)kBulkTile, a.total4 - j0) * 16u;
            const float4* line = out + (size_t)stage * kOut * kBulkTile;
            for (int r = 0; r < x.world; r++) bulk_store(x.p_out[r] + i0, line, bytes);
            bulk_store(a.m + i0, line + kBulkTile, bytes);
            bulk_store(a.v + i0, line + 2 * kBulkTile, bytes);
            bulk_commit();
            const long long next = tile + (long long)kBulkStages * gridDim.x;
            if (next < tiles) fetch(next, stage);
        }
    }
    if (threadIdx.x == 0) bulk_wait_all();  // shared memory must outlive the stores
}

// ---------------------------------------------------------------------------------------------
// The same exchange, run UNDER the feature-transformer backward instead of after it.
//
// The backward's work items are ordered by table row block (king bucket), so the gradient of block b
// is complete long before the kernel ends; the last CTA of every block says so to every rank
// (bucket_signal, called at the end of the backward kernel; empty blocks are announced up front by
// bucket_presignal_kernel).  This kernel is launched before the backward on a stream of higher
// priority, as a few CTAs that each fill an SM (the dynamic shared memory they ask for is only there
// to keep other CTAs off that SM, so the backward simply runs on the SMs that are left).  It walks the
// blocks in order: wait until all ranks have announced block b, sum this rank's 1/world share of the
// block's gradient over all ranks with peer loads (rank order: one owner per element, so the replicas
// stay bit-identical), AdamW, peer stores of the new weights to every rank.  Only the last block's
// share, the factoriser and the small tensors are left when the backward ends.
//
// Factoriser (l0f, as large as one block): its gradient is the sum of the table gradient over the
// blocks.  The owner of share r of every block also owns share r of l0f and keeps the running sum of
// the already reduced block gradients in `facc`, in block order; no separate pass over the table
// gradient is needed.  The small tensors (bias, dense layers, the loss in float 0) are reduced and
// updated by every rank for itself after the all-complete fence (kFlagReady), without peer stores.
//
// Every wait is bounded; a wait that gives up makes the CTA return at once (see peer_wait).
struct OverlapArgs {
    ExchangeArgs x;      // local p, m, v and the segment table; every rank's g and p; flags
    int step;            // the value the ranks announce this step
    int nblocks;
    long long l0w4;      // first float4 of l0w in the flat buffers
    long long block4;    // float4s per row block
    int l0w_seg;         // index of l0w in the segment table
    int l0f_seg;         // index of l0f there when it is summed through facc, else -1
    long long l0f4;      // first float4 of l0f
    float4* facc;        // [block4 / world] running block sum of this rank's share, or null
};

constexpr int kOverlapThreads = 512;      // up to 128 registers each: sixteen 16-byte peer loads in flight per thread
constexpr int kOverlapSmem = 120 * 1024;  // more than half an SM: one such CTA per SM, and no room beside it for a backward CTA

template <int WORLD>
__device__ __forceinline__ float4 reduce_ranks(const ExchangeArgs& x, long long i) {
    constexpr int W = WORLD > 0 ? WORLD : kMaxRanks;
    float4 gr[W];
#pragma unroll
    for (int r = 0; r < W; r++)
        if (r < x.world) gr[r] = x.g[r][i];  // all loads in flight before the first add
    float4 g = gr[0];
#pragma unroll
    for (int r = 1; r < W; r++)
        if (r < x.world) g.x += gr[r].x, g.y += gr[r].y, g.z += gr[r].z, g.w += gr[r].w;
    return g;
}

__device__ __forceinline__ void adam4(const AdamSegment& s, float rate, float adj, const float4& g, float4& p, float4& m, float4& v) {
    adam_op(s, rate, adj * g.x, p.x, m.x, v.x);
    adam_op(s, rate, adj * g.y, p.y, m.y, v.y);
    adam_op(s, rate, adj * g.z, p.z, m.z, v.z);
    adam_op(s, rate, adj * g.w, p.w, m.w, v.w);
}

template <int WORLD>
__global__ void __launch_bounds__(kOverlapThreads, 1) adamw_exchange_overlap_kernel(const __grid_constant__ OverlapArgs o) {
    constexpr int W = WORLD > 0 ? WORLD : kMaxRanks;
    // Elements per thread and round.  Every load of a round (the gradient from each rank, p, m, v and the
    // running factoriser sum) is issued before the first use: U * (W + 4) = 24 independent 16-byte loads
    // per thread hide both the NVLink and the HBM latency.
    constexpr int U = 24 / (W + 4);
    const ExchangeArgs& x = o.x;
    const AdamArgs& a = x.adam;
    const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x, stride = (long long)gridDim.x * blockDim.x;
    const long long share4 = o.block4 / x.world;
    const AdamSegment& seg_w = a.seg[o.l0w_seg];
    for (int b = 0; b < o.nblocks; b++) {
        if (!peer_wait_cta(x.flags, kFlagBucket + b * kMaxRanks, o.step)) return;
        const long long first4 = o.l0w4 + b * o.block4 + x.flags.rank * share4;
        const bool have_f = o.facc != nullptr && b > 0;
        for (long long j0 = tid; j0 < share4; j0 += stride * U) {
            float4 gr[U][W], p[U], m[U], v[U], f[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const long long j = j0 + u * stride;
                if (j < share4) {
#pragma unroll
                    for (int r = 0; r < W; r++)
                        if (r < x.world) gr[u][r] = x.g[r][first4 + j];
                    p[u] = a.p[first4 + j];
                    m[u] = a.m[first4 + j];
                    v[u] = a.v[first4 + j];
                    f[u] = have_f ? o.facc[j] : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const long long j = j0 + u * stride;
                if (j >= share4) break;
                const long long i = first4 + j;
                float4 g = gr[u][0];
#pragma unroll
                for (int r = 1; r < W; r++)
                    if (r < x.world) g.x += gr[u][r].x, g.y += gr[u][r].y, g.z += gr[u][r].z, g.w += gr[u][r].w;
                if (o.facc) {  // blocks are added in order, by the same thread every time
                    f[u].x += g.x, f[u].y += g.y, f[u].z += g.z, f[u].w += g.w;
                    o.facc[j] = f[u];
                }
                adam4(seg_w, a.rate, a.adj, g, p[u], m[u], v[u]);
                a.m[i] = m[u];
                a.v[i] = v[u];
#pragma unroll
                for (int r = 0; r < W; r++)
                    if (r < x.world) x.p_out[r][i] = p[u];
            }
        }
    }
    // everything else needs every rank's whole backward
    if (!peer_wait_cta(x.flags, kFlagReady, o.step)) return;
    if (o.facc) {
        const AdamSegment& seg_f = a.seg[o.l0f_seg];
        const long long first4 = o.l0f4 + x.flags.rank * share4;
        for (long long j = tid; j < share4; j += stride) {
            const long long i = first4 + j;
            float4 p = a.p[i], m = a.m[i], v = a.v[i];
            adam4(seg_f, a.rate, a.adj, o.facc[j], p, m, v);
            a.m[i] = m;
            a.v[i] = v;
#pragma unroll
            for (int r = 0; r < W; r++)
                if (r < x.world) x.p_out[r][i] = p;
        }
    }
    for (long long i = tid; i < o.l0w4; i += stride) {
        int si = -1;
#pragma unroll 1
        for (int k = 0; k < a.nseg; k++)
            if (i >= a.seg[k].begin4 && i < a.seg[k].end4) si = k;
        if (si < 0 && i >= x.head4) continue;  // alignment padding between tensors
        if (si >= 0 && si == o.l0f_seg) continue;
        const float4 g = reduce_ranks<WORLD>(x, i);
        if (si < 0) {
            a.p[i] = g;  // the summed loss (and zeros) in the unused head of the parameter buffer
            continue;
        }
        float4 p = a.p[i], m = a.m[i], v = a.v[i];
        adam4(a.seg[si], a.rate, a.adj, g, p, m, v);
        a.p[i] = p;
        a.m[i] = m;
        a.v[i] = v;
    }
}

}  // namespace b200
