// Feature-transformer kernels: the sparse affine layer on both perspectives with the
// bias, activation, pairwise product and stm|nstm concat fused in, and its backward.
//
// Reference semantics (jw1912/bullet): SparseMatmul::evaluate
// (crates/compiler/src/tensor/operation/linear/sparse.rs:86-119) sums table rows in
// slot order starting from 0 and skips invalid slots; the bias is added afterwards
// (crates/compiler/src/model/builder.rs:145-147); activations and their
// derivatives-from-output follow crates/compiler/src/tensor/operation/autograd/dfo.rs:47-119;
// the backward adds the incoming gradient to one table row per valid slot
// (sparse.rs:151-187).  Both forward kernels add rows in slot order, so their
// pre-activations are bit-identical to the interpreter's fp32 result.
//
// Two families:
//   *_gather : one warp per (position, perspective, 128-column chunk); rows come
//              straight from the table (L2/HBM), gradients go out as 128-bit
//              global reductions.  Works for any index set.
//   *_tiled  : for inputs whose active features of one perspective all lie in one
//              aligned block of R table rows (king buckets).  A forward CTA stages one
//              R x 64-column tile of the table in shared memory and serves every
//              (position, perspective) of that block from it; a backward CTA keeps the
//              matching tile of the table gradient in registers and feeds it from
//              per-row position lists built in shared memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "peer_flags.cuh"

namespace b200 {

constexpr uint32_t kNoFeature = 0xFFFFu;
constexpr int kStatusOutsideBlock = 1;  // a feature fell outside its position's declared row block

struct FtArgs {
    const float* table;   // [n_inputs][H] effective weights: l0w, or l0w + tiled l0f already merged
    const float* factor;  // tiled forward only: [factor_rows][H] l0f to be added to `table` (= l0w) on the fly, or null
    int factor_rows;
    const float* bias;    // [H]
    const uint16_t* idx_stm;
    const uint16_t* idx_nstm;  // [n][nnz] each, 0xFFFF = empty slot
    int n, nnz, H, n_inputs, act;
    float* x;         // dense-stack input: [n][2H], or [n][H] with pairwise
    float* u;         // pairwise only: crelu outputs [n][2][H]
    const float* dx;  // backward: gradient at x
    float* g_table;   // backward: [n_inputs][H] gradient of the table
    float* g_bias;    // backward: [H]
};

struct TileArgs {
    int block_rows;          // R
    int nslabs;              // H/64 column slabs
    // A launch covers the row blocks [first_block, last_block) with gridDim.x CTAs.  The work of those
    // blocks is laid out in one line (block by block; inside a block column slab by column slab; inside a
    // slab pair by pair, for the backward chunk by chunk) and CTA k takes the k-th of gridDim.x near-equal
    // contiguous pieces of that line: every SM gets the same amount of work whatever the blocks hold, and
    // a tile is loaded about once per (block, slab) and SM that touches it.
    int first_block, last_block;
    const int* pair_order;   // [2n] pair ids (position*2 + perspective) grouped by block, or null = identity
    const int* block_begin;  // [nblocks+1] offsets into pair_order
    const int* chunk_begin;  // backward: [nblocks+1] first chunk of every block
    int* status;
    // written by ft_prepare_kernel, read by the tiled kernels: for the i-th pair in visiting
    // order its active rows (local to the pair's block) in slot order; the tail of the last
    // 16-byte group is filled with the index of the all-zero row (= block_rows) and never walked
    uint16_t* lists;  // [2n][list_len]
    int* list_count;  // [2n] number of active rows
    int list_len;     // nnz rounded up to a multiple of 8 (16-byte groups)
    // backward only: the visiting order cut into chunks of at most ft_bwd_chunk pairs that never
    // straddle a block, and per chunk the row-major lists built by ft_csr_kernel
    const int4* chunks;            // [nchunks] (block, first index into pair_order, pairs, 0)
    uint16_t* csr_ent;             // [nchunks][ent_cap] pairs of the chunk grouped by row, every list starting on 16 bytes
    int* csr_start;                // [nchunks][start_cap] per row (start / 8) << 16 | length; [R] = entries in all
    int ent_cap, start_cap;
    int once;                      // table rows and activations through loads that claim no L1 line
    int grab;                      // rows a warp of the backward takes from the row counter at a time
    int chunk_len;  // CP: most pairs per chunk
    // backward only, data-parallel runs: the last CTA of every row block tells all ranks that the block's
    // gradient is complete (done_count null: nobody is told)
    BucketSignal sig;
};

__device__ __forceinline__ float crelu_f(float v) { return fminf(fmaxf(v, 0.f), 1.f); }

// activation of the FT output: 1 = crelu, 2 = screlu
__device__ __forceinline__ float ft_act_fwd(int act, float v) {
    const float c = crelu_f(v);
    return act == 2 ? c * c : c;
}
// d(activation)/d(input) as a function of the activation OUTPUT y (dfo.rs:70-88)
__device__ __forceinline__ float ft_act_bwd(int act, float y) {
    const float c = (y > 0.f && (1.f - y) > 0.f) ? 1.f : 0.f;
    if (act != 2) return c;
    const float half = c * sqrtf(y);
    return half + half;
}

__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

__device__ __forceinline__ void load_slots(const uint16_t* list, int nnz, int lane, uint32_t& s0, uint32_t& s1) {
    s0 = lane < nnz ? list[lane] : kNoFeature;
    s1 = lane + 32 < nnz ? list[lane + 32] : kNoFeature;
}

// ---------------------------------------------------------------- gather forward
// grid = (ceil(2n / pairs_per_block), chunks); block = 256 threads (8 warps).
template <bool PAIRWISE>
__global__ void __launch_bounds__(256) ft_forward_gather_kernel(FtArgs a, int pairs_per_block) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int unit = PAIRWISE ? a.H / 2 : a.H;
    const int col = blockIdx.y * 128 + lane * 4;
    const bool active = col < unit;
    const int pair_end = min(2 * a.n, (int)(blockIdx.x + 1) * pairs_per_block);
    float4 bias_lo = make_float4(0, 0, 0, 0), bias_hi = bias_lo;
    if (active) {
        bias_lo = *reinterpret_cast<const float4*>(a.bias + col);
        if (PAIRWISE) bias_hi = *reinterpret_cast<const float4*>(a.bias + unit + col);
    }
    for (int pair = blockIdx.x * pairs_per_block + warp; pair < pair_end; pair += 8) {
        const int b = pair >> 1, p = pair & 1;
        const uint16_t* list = (p ? a.idx_nstm : a.idx_stm) + (size_t)b * a.nnz;
        uint32_t slot[2];
        load_slots(list, a.nnz, lane, slot[0], slot[1]);
        float4 lo = make_float4(0, 0, 0, 0), hi = lo;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            unsigned m = __ballot_sync(0xffffffffu, slot[half] < (uint32_t)a.n_inputs);
            while (m) {  // up to four independent row loads in flight, added in slot order
                int s[4];
                int cnt = 0;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    s[k] = m ? __ffs(m) - 1 : 0;
                    if (m) cnt++;
                    m &= m - 1;
                }
                float4 vlo[4], vhi[4];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const uint32_t f = __shfl_sync(0xffffffffu, slot[half], s[k]);
                    if (k < cnt && active) {
                        const float* row = a.table + (size_t)f * a.H;
                        vlo[k] = __ldg(reinterpret_cast<const float4*>(row + col));
                        if (PAIRWISE) vhi[k] = __ldg(reinterpret_cast<const float4*>(row + unit + col));
                    }
                }
#pragma unroll
                for (int k = 0; k < 4; k++)
                    if (k < cnt && active) {
                        lo = add4(lo, vlo[k]);
                        if (PAIRWISE) hi = add4(hi, vhi[k]);
                    }
            }
        }
        if (!active) continue;
        lo = add4(lo, bias_lo);
        if (PAIRWISE) {
            hi = add4(hi, bias_hi);
            const float4 ul = make_float4(crelu_f(lo.x), crelu_f(lo.y), crelu_f(lo.z), crelu_f(lo.w));
            const float4 uh = make_float4(crelu_f(hi.x), crelu_f(hi.y), crelu_f(hi.z), crelu_f(hi.w));
            float* up = a.u + (size_t)pair * a.H;
            *reinterpret_cast<float4*>(up + col) = ul;
            *reinterpret_cast<float4*>(up + unit + col) = uh;
            *reinterpret_cast<float4*>(a.x + (size_t)b * a.H + (size_t)p * unit + col) =
                make_float4(ul.x * uh.x, ul.y * uh.y, ul.z * uh.z, ul.w * uh.w);
        } else {
            *reinterpret_cast<float4*>(a.x + (size_t)b * 2 * a.H + (size_t)p * a.H + col) = make_float4(
                ft_act_fwd(a.act, lo.x), ft_act_fwd(a.act, lo.y), ft_act_fwd(a.act, lo.z), ft_act_fwd(a.act, lo.w));
        }
    }
}

// --------------------------------------------------------------- gather backward
// Same decomposition.  The table gradient must be zero on entry; gradients are
// added with 128-bit global reductions, the bias gradient once per lane per block.
template <bool PAIRWISE>
__global__ void __launch_bounds__(256) ft_backward_gather_kernel(FtArgs a, int pairs_per_block) {
    __shared__ float4 red[2][8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int unit = PAIRWISE ? a.H / 2 : a.H;
    const int col = blockIdx.y * 128 + lane * 4;
    const bool active = col < unit;
    const int pair_end = min(2 * a.n, (int)(blockIdx.x + 1) * pairs_per_block);
    float4 bsum_lo = make_float4(0, 0, 0, 0), bsum_hi = bsum_lo;
    for (int pair = blockIdx.x * pairs_per_block + warp; pair < pair_end; pair += 8) {
        const int b = pair >> 1, p = pair & 1;
        float4 glo = make_float4(0, 0, 0, 0), ghi = glo;
        if (active) {
            if (PAIRWISE) {
                const float* up = a.u + (size_t)pair * a.H;
                const float4 ul = *reinterpret_cast<const float4*>(up + col);
                const float4 uh = *reinterpret_cast<const float4*>(up + unit + col);
                const float4 d = *reinterpret_cast<const float4*>(a.dx + (size_t)b * a.H + (size_t)p * unit + col);
                glo = make_float4((d.x * uh.x) * ft_act_bwd(1, ul.x), (d.y * uh.y) * ft_act_bwd(1, ul.y),
                                  (d.z * uh.z) * ft_act_bwd(1, ul.z), (d.w * uh.w) * ft_act_bwd(1, ul.w));
                ghi = make_float4((d.x * ul.x) * ft_act_bwd(1, uh.x), (d.y * ul.y) * ft_act_bwd(1, uh.y),
                                  (d.z * ul.z) * ft_act_bwd(1, uh.z), (d.w * ul.w) * ft_act_bwd(1, uh.w));
            } else {
                const size_t at = (size_t)b * 2 * a.H + (size_t)p * a.H + col;
                const float4 y = *reinterpret_cast<const float4*>(a.x + at);
                const float4 d = *reinterpret_cast<const float4*>(a.dx + at);
                glo = make_float4(d.x * ft_act_bwd(a.act, y.x), d.y * ft_act_bwd(a.act, y.y),
                                  d.z * ft_act_bwd(a.act, y.z), d.w * ft_act_bwd(a.act, y.w));
            }
        }
        const bool lo_nz = glo.x != 0.f || glo.y != 0.f || glo.z != 0.f || glo.w != 0.f;
        const bool hi_nz = PAIRWISE && (ghi.x != 0.f || ghi.y != 0.f || ghi.z != 0.f || ghi.w != 0.f);
        if (!__any_sync(0xffffffffu, lo_nz || hi_nz)) continue;  // the reference skips zero gradients too
        bsum_lo = add4(bsum_lo, glo);
        bsum_hi = add4(bsum_hi, ghi);
        const uint16_t* list = (p ? a.idx_nstm : a.idx_stm) + (size_t)b * a.nnz;
        uint32_t slot[2];
        load_slots(list, a.nnz, lane, slot[0], slot[1]);
#pragma unroll
        for (int half = 0; half < 2; half++) {
            unsigned m = __ballot_sync(0xffffffffu, slot[half] < (uint32_t)a.n_inputs);
            while (m) {
                const int s = __ffs(m) - 1;
                m &= m - 1;
                const uint32_t f = __shfl_sync(0xffffffffu, slot[half], s);
                float* row = a.g_table + (size_t)f * a.H;
                if (lo_nz) atomicAdd(reinterpret_cast<float4*>(row + col), glo);
                if (hi_nz) atomicAdd(reinterpret_cast<float4*>(row + unit + col), ghi);
            }
        }
    }
    red[0][warp][lane] = bsum_lo;
    red[1][warp][lane] = bsum_hi;
    __syncthreads();
    if (warp == 0 && active) {
        float4 s_lo = red[0][0][lane], s_hi = red[1][0][lane];
        for (int w = 1; w < 8; w++) {
            s_lo = add4(s_lo, red[0][w][lane]);
            s_hi = add4(s_hi, red[1][w][lane]);
        }
        atomicAdd(reinterpret_cast<float4*>(a.g_bias + col), s_lo);
        if (PAIRWISE) atomicAdd(reinterpret_cast<float4*>(a.g_bias + unit + col), s_hi);
    }
}

// ------------------------------------------------------------------ tiled kernels
// A tile row holds 64 floats of one table row as 32 (A, B) pairs; lane l owns pair l and
// moves it with one 64-bit shared-memory access and one packed f32x2 add.  Without pairwise
// the pair is two neighbouring columns (64s + 2l, 64s + 2l + 1); with pairwise it is the
// low-half column 32s + l and its partner H/2 + 32s + l, i.e. both factors of one product.
constexpr int kTileCols = 64;
constexpr int kTileRowBytes = kTileCols * 4;

typedef unsigned long long f32x2;  // two packed floats: low word = A, high word = B

__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {  // two IEEE fp32 adds in one instruction
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f32x2 pack2(float a, float b) {
    return (f32x2)__float_as_uint(a) | ((f32x2)__float_as_uint(b) << 32);
}
__device__ __forceinline__ float lo2(f32x2 v) { return __uint_as_float((unsigned)v); }
__device__ __forceinline__ float hi2(f32x2 v) { return __uint_as_float((unsigned)(v >> 32)); }

template <bool PAIRWISE>
__device__ __forceinline__ int tile_col_a(int slab, int lane, int H) { return PAIRWISE ? slab * 32 + lane : slab * 64 + 2 * lane; }
template <bool PAIRWISE>
__device__ __forceinline__ int tile_col_b(int slab, int lane, int H) {
    return PAIRWISE ? H / 2 + slab * 32 + lane : slab * 64 + 2 * lane + 1;
}

// Loads of data that is read once per kernel and must not claim L1 lines: with 196-228 KB of the SM's 256 KB
// configured as shared memory only 28-60 KB of L1 are left, less than these kernels keep in flight.
__device__ __forceinline__ float4 ld_once4(const float4* p) {
    float4 v;
    asm("ld.global.nc.L1::no_allocate.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ float2 ld_once2(const float2* p) {
    float2 v;
    asm("ld.global.nc.L1::no_allocate.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_once(const float* p) {
    float v;
    asm("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

__device__ __forceinline__ const uint16_t* pair_list(const FtArgs& a, int pair) {
    return ((pair & 1) ? a.idx_nstm : a.idx_stm) + (size_t)(pair >> 1) * a.nnz;
}

// Per batch, once: turns every (position, perspective) pair's slots into the list the tiled
// kernels walk — rows local to the pair's block, compacted in slot order, the last 16-byte
// group filled up with the index of the all-zero row.  A valid feature outside the block raises
// the status bit and is dropped.  One warp per pair, in visiting order.  grid = ceil(2n / 8), block = 256.
static __global__ void __launch_bounds__(256) ft_prepare_kernel(FtArgs a, TileArgs t) {
    const int lane = threadIdx.x & 31;
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= 2 * a.n) return;
    const int pair = t.pair_order ? t.pair_order[i] : i;
    uint32_t slot0, slot1;
    load_slots(pair_list(a, pair), a.nnz, lane, slot0, slot1);
    const bool v0 = slot0 < (uint32_t)a.n_inputs, v1 = slot1 < (uint32_t)a.n_inputs;
    // the block of a pair is the block of its first valid feature (as the grouping defines it)
    const unsigned mv0 = __ballot_sync(0xffffffffu, v0), mv1 = __ballot_sync(0xffffffffu, v1);
    int block = 0;
    if (mv0)
        block = (int)__shfl_sync(0xffffffffu, slot0, __ffs(mv0) - 1) / t.block_rows;
    else if (mv1)
        block = (int)__shfl_sync(0xffffffffu, slot1, __ffs(mv1) - 1) / t.block_rows;
    const int row0 = (int)slot0 - block * t.block_rows, row1 = (int)slot1 - block * t.block_rows;
    const bool in0 = v0 && (unsigned)row0 < (unsigned)t.block_rows, in1 = v1 && (unsigned)row1 < (unsigned)t.block_rows;
    if ((v0 && !in0) || (v1 && !in1)) atomicOr(t.status, kStatusOutsideBlock);
    const unsigned m0 = __ballot_sync(0xffffffffu, in0), m1 = __ballot_sync(0xffffffffu, in1);
    const unsigned lt = (1u << lane) - 1u;
    const int cnt0 = __popc(m0), cnt = cnt0 + __popc(m1), cnt8 = (cnt + 7) & ~7;
    uint16_t* list = t.lists + (size_t)i * t.list_len;
    if (in0) list[__popc(m0 & lt)] = (uint16_t)row0;
    if (in1) list[cnt0 + __popc(m1 & lt)] = (uint16_t)row1;
    if (lane < cnt8 - cnt) list[cnt + lane] = (uint16_t)t.block_rows;
    if (lane == 0) t.list_count[i] = cnt;
}

// One 256-byte line of shared memory (a tile row, or a staged gradient line), this lane's 8 bytes of it.
__device__ __forceinline__ f32x2 line_at(const unsigned char* mine, uint32_t index) {
    return *reinterpret_cast<const f32x2*>(mine + index * kTileRowBytes);
}

// Forward.  One CTA of 1024 threads per SM; dynamic shared memory = (R+1) tile rows, the extra row all
// zero, then per warp one prepared list (and 16 bytes that a read-ahead may touch).  A CTA walks its piece of
// the work line segment by segment; a segment is a run of pairs of one (block, slab), whose tile the CTA loads
// first.  Each warp serves one (position, perspective) at a time.  The pair's prepared list reaches the warp
// one pair ahead: every lane loads one 32-bit word of it (two row indices) into a register while the pair
// before is still being walked, and stores it into the warp's list buffer afterwards, so the walk itself
// reads no global memory and the buffer costs one shared-memory wavefront per pair (a cp.async of the same 64
// bytes by four lanes cost seven).  The walk takes four row indices per (warp-uniform) 8-byte shared-memory
// load, and every lane adds its column pair with one 64-bit shared-memory load and one packed add per row, in
// slot order — the same order and arithmetic as the interpreter (adding the zero row changes nothing).
constexpr int kFwdThreads = 1024;
__host__ __device__ inline size_t ft_fwd_smem(int R, int list_len) {
    return (size_t)(R + 1) * kTileRowBytes + (size_t)(kFwdThreads / 32) * list_len * 2 + 16;
}

template <bool PAIRWISE>
__global__ void __launch_bounds__(kFwdThreads, 1) ft_forward_tiled_kernel(FtArgs a, TileArgs t) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int NW = kFwdThreads / 32;
    const int R = t.block_rows;
    float* tile = reinterpret_cast<float*>(smem_raw);
    // this CTA's piece [v, v_end) of the line of nslabs x (pairs of the launch's blocks) positions
    const int pair0 = t.block_begin[t.first_block];
    const long long line = (long long)t.nslabs * (t.block_begin[t.last_block] - pair0);
    long long v = line * blockIdx.x / gridDim.x;
    const long long v_end = line * (blockIdx.x + 1) / gridDim.x;
    int block = t.first_block;
    if (threadIdx.x < kTileCols) tile[R * kTileCols + threadIdx.x] = 0.f;  // the zero row
    const unsigned char* mine = smem_raw + lane * 8;
    // outputs of pair p start at p * (row length): x is [n][2 persp][H or H/2], u is [n][2][H]
    const int x_row = PAIRWISE ? a.H / 2 : a.H;
    while (v < v_end) {
        // the segment v lies in: block, slab, first pair
        long long base = (long long)t.nslabs * (t.block_begin[block] - pair0);
        int in_block = t.block_begin[block + 1] - t.block_begin[block];
        while (v >= base + (long long)t.nslabs * in_block) {
            base += (long long)t.nslabs * in_block;
            block++;
            in_block = t.block_begin[block + 1] - t.block_begin[block];
        }
        const int slab = (int)((v - base) / in_block), first = (int)((v - base) % in_block);
        const int last = (int)min((long long)in_block, first + (v_end - v));
        v += last - first;
        __syncthreads();  // every warp has left the previous tile
        {   // fill the tile: 8 work items per row, each 8 floats of the row
            // with a factoriser the table row is l0w[row] + l0f[row mod factor_rows], one fp32 add per
            // element exactly as the reference forms `l0w + l0f.repeat(n)` (model/builder.rs:421-424)
            const float* src = a.table + (size_t)block * R * a.H;
            for (int i = threadIdx.x; i < R * 8; i += kFwdThreads) {
                const int row = i >> 3, q = i & 7;
                float4* dst = reinterpret_cast<float4*>(tile + row * kTileCols + q * 8);
                const float* frow = a.factor ? a.factor + (size_t)((block * R + row) % a.factor_rows) * a.H : nullptr;
                if (PAIRWISE) {
                    const int c_lo = slab * 32 + q * 4, c_hi = a.H / 2 + c_lo;
                    const float4* plo = reinterpret_cast<const float4*>(src + (size_t)row * a.H + c_lo);
                    const float4* phi = reinterpret_cast<const float4*>(src + (size_t)row * a.H + c_hi);
                    float4 lo = t.once ? ld_once4(plo) : __ldg(plo);
                    float4 hi = t.once ? ld_once4(phi) : __ldg(phi);
                    if (frow) {
                        lo = add4(lo, __ldg(reinterpret_cast<const float4*>(frow + c_lo)));  // (these gain from L1)
                        hi = add4(hi, __ldg(reinterpret_cast<const float4*>(frow + c_hi)));
                    }
                    // (the work items of a row lie 32 bytes apart: the upper four of a row store their second half
                    // first, so that the eight 16-byte stores of a quarter warp fall into eight different bank groups)
                    const int h = q >> 2;
                    const float4 first = make_float4(lo.x, hi.x, lo.y, hi.y), second = make_float4(lo.z, hi.z, lo.w, hi.w);
                    dst[h] = h ? second : first;
                    dst[h ^ 1] = h ? first : second;
                } else {
                    const int c0 = slab * 64 + q * 8;
                    const float4* g = reinterpret_cast<const float4*>(src + (size_t)row * a.H + c0);
                    float4 v0 = t.once ? ld_once4(g) : __ldg(g), v1 = t.once ? ld_once4(g + 1) : __ldg(g + 1);
                    if (frow) {
                        v0 = add4(v0, __ldg(reinterpret_cast<const float4*>(frow + c0)));
                        v1 = add4(v1, __ldg(reinterpret_cast<const float4*>(frow + c0 + 4)));
                    }
                    const int h = q >> 2;
                    dst[h] = h ? v1 : v0;
                    dst[h ^ 1] = h ? v0 : v1;
                }
            }
        }
        const int col_a = tile_col_a<PAIRWISE>(slab, lane, a.H), col_b = tile_col_b<PAIRWISE>(slab, lane, a.H);
        const f32x2 bias = pack2(a.bias[col_a], a.bias[col_b]);
        float* x_out = a.x + col_a;  // with pairwise col_a is also the product's column within the perspective
        __syncthreads();
        // pair id, list length and the list itself are fetched one pair ahead into registers: every lane holds one
        // 32-bit word (two row indices) of the next pair's list and puts it into the warp's list buffer when the walk
        // of the current pair is over, so the walk reads its indices from shared memory and never waits for global memory
        const int seg_end = t.block_begin[block] + last;
        const int list_words = t.list_len / 2;
        uint32_t* ring = reinterpret_cast<uint32_t*>(smem_raw + (size_t)(R + 1) * kTileRowBytes) + warp * list_words;
        const uint32_t* lists_w = reinterpret_cast<const uint32_t*>(t.lists);
        int i = t.block_begin[block] + first + warp;
        int pair = 0, cnt = 0;
        uint32_t word = 0;
        if (i < seg_end) {
            pair = t.pair_order ? t.pair_order[i] : i;
            cnt = t.list_count[i];
            if (lane < list_words) word = __ldg(lists_w + (size_t)i * list_words + lane);
        }
        for (; i < seg_end; i += NW) {
            int pair_next = 0, cnt_next = 0;
            __syncwarp();  // every lane has finished with the list of the pair before
            if (lane < list_words) ring[lane] = word;
            if (i + NW < seg_end) {
                pair_next = t.pair_order ? t.pair_order[i + NW] : i + NW;
                cnt_next = t.list_count[i + NW];
                if (lane < list_words) word = __ldg(lists_w + (size_t)(i + NW) * list_words + lane);
            }
            __syncwarp();
            f32x2 acc = 0;  // (+0.0f, +0.0f)
            const uint2* list = reinterpret_cast<const uint2*>(ring);
            uint2 g = list[0];
            for (int k = 0; k < cnt; k += 4) {
                const uint2 g_ahead = list[(k >> 2) + 1];  // (past the last group: the next warp's buffer or the spare 16 bytes, unused)
                const f32x2 v0 = line_at(mine, g.x & 0xffffu), v1 = line_at(mine, g.x >> 16);
                const f32x2 v2 = line_at(mine, g.y & 0xffffu), v3 = line_at(mine, g.y >> 16);
                acc = add2(add2(add2(add2(acc, v0), v1), v2), v3);
                g = g_ahead;
            }
            acc = add2(acc, bias);
            if (PAIRWISE) {
                const float ua = crelu_f(lo2(acc)), ub = crelu_f(hi2(acc));
                float* up = a.u + (size_t)pair * a.H;
                up[col_a] = ua;
                up[col_b] = ub;
                x_out[(size_t)pair * x_row] = ua * ub;
            } else {
                *reinterpret_cast<float2*>(x_out + (size_t)pair * x_row) =
                    make_float2(ft_act_fwd(a.act, lo2(acc)), ft_act_fwd(a.act, hi2(acc)));
            }
            pair = pair_next;
            cnt = cnt_next;
        }
    }
}

// Backward.  Positions are visited in chunks of at most CP pairs of one row block.
//   ft_csr_kernel (one CTA per chunk, once per batch) turns the chunk's prepared lists around:
//     for every table row of the block, the list of the chunk's pairs that hold it (a count
//     pass, a scan and a fill pass in shared memory), every list starting on a 16-byte
//     boundary and stored with its exact length.  All column slabs share the result.
//   ft_backward_tiled_kernel (same grid as the forward) then, per chunk, copies that list
//     structure into shared memory, stages the chunk's pre-activation gradients (from dx and
//     the kept activations) as one 64-float line per pair, and every warp walks the lists of
//     the rows it owns (row = warp, warp + 32, ...), sums the staged lines in registers and
//     adds the row's total to the table gradient with one global reduction per lane.
// Accumulation needs no atomics, and the table gradient sees one reduction per (row, chunk)
// instead of one per (row, position).  The table gradient must be zero on entry.
constexpr int kCsrThreads = 512;

// Two shapes of the backward: "wide" = one CTA of 1024 threads per SM working on chunks of 512
// pairs, otherwise two CTAs of 512 threads on chunks of 256, so that one CTA's global loads
// overlap the other's shared-memory work.  Chunks halve when nnz > 32.
__host__ __device__ inline int ft_bwd_chunk(int nnz, bool wide) { return (wide ? 512 : 256) / (nnz <= 32 ? 1 : 2); }
// The wide shape takes 640-pair chunks where they fit (768-row blocks with 32 slots: 223 KB): a fifth fewer
// list copies, barriers and per-row reductions for the same walk; measured 2 % faster at 131072 positions.
__host__ __device__ inline int ft_bwd_chunk_large(int nnz) { return 640 / (nnz <= 32 ? 1 : 2); }
// entries per chunk: every slot of every pair plus up to seven padding entries per row (lists start on 16 bytes)
__host__ __device__ inline int ft_bwd_ent_cap(int R, int nnz, int cp) { return (cp * nnz + 8 * R + 7) & ~7; }
__host__ __device__ inline int ft_bwd_start_cap(int R) { return (R + 1 + 3) & ~3; }
__host__ __device__ inline size_t ft_bwd_smem(int R, int nnz, int cp, int nslabs) {
    return (size_t)(cp + 1) * kTileRowBytes + (size_t)ft_bwd_ent_cap(R, nnz, cp) * 2 + (size_t)ft_bwd_start_cap(R) * 4 + (size_t)cp * 4 +
           (size_t)nslabs * kTileRowBytes;  // staged lines, row lists, their starts, pair ids, bias-gradient sums per slab
}
__host__ __device__ inline size_t ft_csr_smem(int R, int nnz, int cp) {
    return (size_t)ft_bwd_ent_cap(R, nnz, cp) * 2 + (size_t)(2 * (R + 2) + 32 + cp) * 4;
}

// grid = number of chunks, block = kCsrThreads.
static __global__ void __launch_bounds__(kCsrThreads) ft_csr_kernel(FtArgs a, TileArgs t) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int NW = kCsrThreads / 32;
    const int4 chunk = t.chunks[blockIdx.x];
    const int R = t.block_rows, CP = t.chunk_len, L = t.list_len, c0 = chunk.y, cn = chunk.z;
    uint16_t* ent = reinterpret_cast<uint16_t*>(smem_raw);
    int* start = reinterpret_cast<int*>(ent + t.ent_cap);  // [R + 1]
    int* cursor = start + R + 2;                                         // [R]
    int* warp_tot = cursor + R + 2;                                      // [32]
    int* count_s = warp_tot + 32;                                        // [CP] prepared list lengths
    const int zero_row = R;
    for (int r = threadIdx.x; r < R; r += kCsrThreads) cursor[r] = 0;
    for (int k = threadIdx.x; k < cn; k += kCsrThreads) count_s[k] = t.list_count[c0 + k];
    __syncthreads();
    // count how often each row occurs in the chunk: a warp per pair, a lane per list entry,
    // four pairs in flight
    const uint16_t* lists = t.lists + (size_t)c0 * L;
    for (int pl0 = warp; pl0 < cn; pl0 += 4 * NW)
        for (int k0 = 0; k0 < L; k0 += 32) {
            int o[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int pl = pl0 + k * NW;
                o[k] = zero_row;
                if (pl < cn && k0 + lane < count_s[pl]) o[k] = __ldg(lists + (size_t)pl * L + k0 + lane);
            }
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (o[k] != zero_row) atomicAdd(&cursor[o[k]], 1);
        }
    __syncthreads();
    // exclusive scan of the row counts, each rounded up to a multiple of eight entries (16 bytes)
    {
        int carry = 0;
        for (int base = 0; base < R; base += kCsrThreads) {
            const int r = base + threadIdx.x;
            const int v = r < R ? (cursor[r] + 7) & ~7 : 0;
            int incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += n;
            }
            if (lane == 31) warp_tot[warp] = incl;
            __syncthreads();
            int before = carry, all = 0;
            for (int k = 0; k < NW; k++) {
                if (k < warp) before += warp_tot[k];
                all += warp_tot[k];
            }
            if (r < R) {
                start[r] = before + incl - v;
                cursor[r] = before + incl - v;
            }
            carry += all;
            __syncthreads();
        }
        if (threadIdx.x == 0) start[R] = carry;
    }
    __syncthreads();
    // fill: entry = index of the pair within the chunk, grouped by row
    for (int pl0 = warp; pl0 < cn; pl0 += 4 * NW)
        for (int k0 = 0; k0 < L; k0 += 32) {
            int o[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int pl = pl0 + k * NW;
                o[k] = zero_row;
                if (pl < cn && k0 + lane < count_s[pl]) o[k] = __ldg(lists + (size_t)pl * L + k0 + lane);
            }
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (o[k] != zero_row) ent[atomicAdd(&cursor[o[k]], 1)] = (uint16_t)(pl0 + k * NW);
        }
    __syncthreads();
    // the unused tail of every list's last 16-byte group points at the all-zero line (index CP)
    for (int r = threadIdx.x; r < R; r += kCsrThreads)
        for (int e = cursor[r]; e < start[r + 1]; e++) ent[e] = (uint16_t)CP;
    __syncthreads();
    // publish: the entries in 16-byte pieces, and per row its start (in 16-byte units) and exact length
    const int total = start[R];
    uint4* ent_out = reinterpret_cast<uint4*>(t.csr_ent + (size_t)blockIdx.x * t.ent_cap);
    for (int i = threadIdx.x; i < total / 8; i += kCsrThreads) ent_out[i] = reinterpret_cast<const uint4*>(ent)[i];
    int* start_out = t.csr_start + (size_t)blockIdx.x * t.start_cap;
    for (int r = threadIdx.x; r < R; r += kCsrThreads) start_out[r] = ((start[r] >> 3) << 16) | (cursor[r] - start[r]);
    if (threadIdx.x == 0) start_out[R] = total;
}

// The backward's work line: block b contributes, per column slab, its pairs plus a fixed amount per chunk
// (the one reduction per row costs about as much as this many pairs).  A unit is one (block, chunk, slab);
// units are numbered block by block, chunk by chunk, and slab by slab INSIDE a chunk: a CTA that takes
// consecutive units keeps the chunk's row lists (which do not depend on the slab) in shared memory for all
// slabs, and reads neighbouring 128- or 256-byte pieces of the same activation rows from one unit to the next.
constexpr int kChunkFixed = 96;
__host__ __device__ inline long long ft_bwd_block_weight(int pairs, int chunks) { return pairs + (long long)kChunkFixed * chunks; }
__host__ __device__ inline long long ft_bwd_line(const int* block_begin, const int* chunk_begin, int first_block, int last_block, int nslabs) {
    long long line = 0;
    for (int b = first_block; b < last_block; b++)
        line += nslabs * ft_bwd_block_weight(block_begin[b + 1] - block_begin[b], chunk_begin[b + 1] - chunk_begin[b]);
    return line;
}
// the unit that holds position `at` of the line (the number of units if `at` is the line's end)
__host__ __device__ inline int ft_bwd_unit_at(long long at, const int* block_begin, const int* chunk_begin, int first_block, int last_block,
                                              int nslabs) {
    long long base = 0;
    int units = 0;
    for (int b = first_block; b < last_block; b++) {
        const int nch = chunk_begin[b + 1] - chunk_begin[b];
        const long long wb = ft_bwd_block_weight(block_begin[b + 1] - block_begin[b], nch);
        if (nch > 0 && at < base + nslabs * wb) {
            const long long j = (at - base) * nch / wb;  // a block's chunks are of equal size, so its units weigh the same
            return units + (int)(j < (long long)nslabs * nch - 1 ? j : (long long)nslabs * nch - 1);
        }
        base += nslabs * wb;
        units += nslabs * nch;
    }
    return units;
}

// grid = one CTA of 1024 threads per SM (or two of 512); CTA k takes the units between the k-th and
// the (k+1)-th of gridDim.x equal cuts of the work line.  With SIGNAL (data-parallel runs whose exchange
// takes finished row blocks while this kernel is still running) the blocks must finish one after the
// other, not all at the end: CTA k then takes the units k, k + gridDim.x, ... of the block-ordered
// numbering, so that all CTAs move through the blocks together, and announces a block it has left after
// the staging phase of its next unit, when that block's reductions have had time to land (the fence
// that must precede the announcement then finds little to wait for).
template <bool PAIRWISE, int THREADS, bool SIGNAL>
__global__ void __launch_bounds__(THREADS, 2048 / (2 * THREADS)) ft_backward_tiled_kernel(FtArgs a, TileArgs t) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kBwdThreads = THREADS;
    constexpr int NW = kBwdThreads / 32;
    const int R = t.block_rows, CP = t.chunk_len;
    f32x2* g_s = reinterpret_cast<f32x2*>(smem_raw);                                          // [CP + 1][32] (A, B) pairs
    uint16_t* ent = reinterpret_cast<uint16_t*>(smem_raw + (size_t)(CP + 1) * kTileRowBytes);  // lists of the chunk
    int* start = reinterpret_cast<int*>(ent + t.ent_cap);                                     // [R + 1]
    int* pairs_s = start + t.start_cap;                                                       // [CP] pair ids of the chunk
    float* bias_s = reinterpret_cast<float*>(pairs_s + CP);                                   // [nslabs][64] bias-gradient sums
    __shared__ int next_rows;  // the walk's row counter
    if (threadIdx.x < 32) g_s[CP * 32 + threadIdx.x] = 0;  // the all-zero line that list padding points at
    for (int i = threadIdx.x; i < t.nslabs * kTileCols; i += kBwdThreads) bias_s[i] = 0.f;

    const long long line = ft_bwd_line(t.block_begin, t.chunk_begin, t.first_block, t.last_block, t.nslabs);
    const int u_begin = ft_bwd_unit_at(line * blockIdx.x / gridDim.x, t.block_begin, t.chunk_begin, t.first_block, t.last_block, t.nslabs);
    const int u_end = ft_bwd_unit_at(line * (blockIdx.x + 1) / gridDim.x, t.block_begin, t.chunk_begin, t.first_block, t.last_block, t.nslabs);

    // Bias gradient: a warp adds the sums of the pairs it staged to the slab's line of bias_s (shared-memory
    // atomics); the CTA adds the lines to global memory once, at the end.
    int col_a = 0, col_b = 0, slab = -1, block = -1, ch_loaded = -1;
    int scan_block = t.first_block, scan_base = 0;  // units before scan_block
    int all_units = 0, left_block = -1;             // SIGNAL: a block this CTA has left and not yet announced
    if (SIGNAL) all_units = t.nslabs * (t.chunk_begin[t.last_block] - t.chunk_begin[t.first_block]);
    for (int u = SIGNAL ? (int)blockIdx.x : u_begin; u < (SIGNAL ? all_units : u_end); u += SIGNAL ? (int)gridDim.x : 1) {
        int nch = t.chunk_begin[scan_block + 1] - t.chunk_begin[scan_block];
        while (u >= scan_base + t.nslabs * nch) {
            scan_base += t.nslabs * nch;
            scan_block++;
            nch = t.chunk_begin[scan_block + 1] - t.chunk_begin[scan_block];
        }
        const int local = u - scan_base, new_slab = local % t.nslabs, ch = t.chunk_begin[scan_block] + local / t.nslabs;
        if (new_slab != slab || scan_block != block) {
            if (SIGNAL && block >= 0 && scan_block != block) {
                if (left_block >= 0) bucket_signal(t.sig, left_block);  // (only if a whole block went by within one unit)
                left_block = block;
            }
            slab = new_slab;
            block = scan_block;
            col_a = tile_col_a<PAIRWISE>(slab, lane, a.H);
            col_b = tile_col_b<PAIRWISE>(slab, lane, a.H);
        }
        const int4 chunk = t.chunks[ch];
        const int c0 = chunk.y, cn = chunk.z;
        // the chunk's row lists, unless the unit before left them here: asynchronous copy into shared memory,
        // overlapped with the staging below
        if (ch != ch_loaded) {
            const int* start_in = t.csr_start + (size_t)ch * t.start_cap;
            for (int i = threadIdx.x; i < t.start_cap / 4; i += kBwdThreads) cp_async16(start + 4 * i, start_in + 4 * i);
            const int total = __ldg(start_in + R);
            const uint16_t* ent_in = t.csr_ent + (size_t)ch * t.ent_cap;
            for (int i = threadIdx.x; i < (total + 7) / 8; i += kBwdThreads) cp_async16(ent + 8 * i, ent_in + 8 * i);
            for (int k = threadIdx.x; k < cn; k += kBwdThreads) pairs_s[k] = t.pair_order ? t.pair_order[c0 + k] : c0 + k;
            ch_loaded = ch;
            __syncthreads();  // the pair ids (and, on the first unit, the zeroed lines) are in place
        }
        float bsum_a = 0.f, bsum_b = 0.f;
        // stage this chunk's gradients at the feature-transformer pre-activation
        for (int pl0 = warp; pl0 < cn; pl0 += 4 * NW) {
            float q0[4], q1[4], q2[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int pl = pl0 + k * NW;
                q0[k] = q1[k] = q2[k] = 0.f;
                if (pl < cn) {
                    const int pair = pairs_s[pl];
                    if (PAIRWISE) {
                        const float* pa = a.u + (size_t)pair * a.H + col_a;
                        const float* pb = a.u + (size_t)pair * a.H + col_b;
                        const float* pd = a.dx + (size_t)pair * (a.H / 2) + col_a;
                        q0[k] = t.once ? ld_once(pa) : *pa;
                        q1[k] = t.once ? ld_once(pb) : *pb;
                        q2[k] = t.once ? ld_once(pd) : *pd;
                    } else {
                        const size_t at = (size_t)pair * a.H + col_a;
                        const float2* pd = reinterpret_cast<const float2*>(a.dx + at);
                        const float2* py = reinterpret_cast<const float2*>(a.x + at);
                        const float2 d = t.once ? ld_once2(pd) : *pd;
                        const float2 y = t.once ? ld_once2(py) : *py;
                        q0[k] = d.x * ft_act_bwd(a.act, y.x);
                        q1[k] = d.y * ft_act_bwd(a.act, y.y);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int pl = pl0 + k * NW;
                if (pl < cn) {
                    float ga = q0[k], gb = q1[k];
                    if (PAIRWISE) {
                        ga = (q2[k] * q1[k]) * ft_act_bwd(1, q0[k]);
                        gb = (q2[k] * q0[k]) * ft_act_bwd(1, q1[k]);
                    }
                    if (PAIRWISE) {  // the line holds the 32 low-half columns, then the 32 high-half ones: a lane of the
                                     // walk then owns two neighbouring columns of the table and reduces them at once
                        float* gf = reinterpret_cast<float*>(g_s) + pl * kTileCols;
                        gf[lane] = ga;
                        gf[32 + lane] = gb;
                    } else {
                        g_s[pl * 32 + lane] = pack2(ga, gb);
                    }
                    bsum_a += ga;
                    bsum_b += gb;
                }
            }
        }
        if (threadIdx.x == 0) next_rows = 0;
        if (bsum_a != 0.f) atomicAdd(bias_s + slab * kTileCols + lane, bsum_a);
        if (bsum_b != 0.f) atomicAdd(bias_s + slab * kTileCols + 32 + lane, bsum_b);
        cp_async_wait_all();
        __syncthreads();
        if (SIGNAL && left_block >= 0) {
            bucket_signal(t.sig, left_block);
            left_block = -1;
        }
        // The next unit of a CTA that walks consecutive units is the same chunk's next slab: ask L2 for the lines
        // its staging will read (the neighbours of the ones just staged) now, so that they arrive during the walk.
        if (!SIGNAL && t.once && new_slab + 1 < t.nslabs && u + 1 < u_end && (int)threadIdx.x < cn) {
            const int pair = pairs_s[threadIdx.x];
            if (PAIRWISE) {
                const float* pu = a.u + (size_t)pair * a.H + (slab + 1) * 32;
                prefetch_l2(pu);
                prefetch_l2(pu + a.H / 2);
                prefetch_l2(a.dx + (size_t)pair * (a.H / 2) + (slab + 1) * 32);
            } else {
                const size_t at = (size_t)pair * a.H + (slab + 1) * 64;
                prefetch_l2(a.dx + at);
                prefetch_l2(a.dx + at + 32);
                prefetch_l2(a.x + at);
                prefetch_l2(a.x + at + 32);
            }
        }
        // accumulate: each warp walks the lists of the rows it owns, four entries per 8-byte load
        const unsigned char* gl = smem_raw + lane * 8;
        // the two table columns this lane sums (see the staging above for the pairwise layout of a line)
        const int col_w = !PAIRWISE ? col_a : lane < 16 ? slab * 32 + 2 * lane : a.H / 2 + slab * 32 + 2 * (lane - 16);
        // rows are handed out a few at a time to whichever warp is free: list lengths differ a lot from row to row
        for (;;) {
            int row2 = 0;
            if (lane == 0) row2 = atomicAdd(&next_rows, t.grab);
            row2 = __shfl_sync(0xffffffffu, row2, 0);
            if (row2 >= R) break;
            for (int row = row2; row < min(R, row2 + t.grab); row++) {
            const unsigned sl = (unsigned)start[row];
            const int len = (int)(sl & 0xffffu);
            const uint2* lp = reinterpret_cast<const uint2*>(ent + (sl >> 16) * 8);
            f32x2 acc = 0;
            uint2 g = lp[0];  // (reads beyond a list's end stay inside the entry array, which has room to spare, and are never used)
            for (int k = 0; k < len; k += 4) {
                const uint2 g_ahead = lp[(k >> 2) + 1];  // the next four entries, before the current four lines are added
                const f32x2 v0 = line_at(gl, g.x & 0xffffu), v1 = line_at(gl, g.x >> 16);
                const f32x2 v2 = line_at(gl, g.y & 0xffffu), v3 = line_at(gl, g.y >> 16);
                acc = add2(add2(add2(add2(acc, v0), v1), v2), v3);
                g = g_ahead;
            }
            float* dst = a.g_table + (size_t)(block * R + row) * a.H + col_w;
            const float ga = lo2(acc), gb = hi2(acc);
            if (ga != 0.f || gb != 0.f) atomicAdd(reinterpret_cast<float2*>(dst), make_float2(ga, gb));
            }
        }
        __syncthreads();
    }
    // entry [slab][j] holds, for j < 32, lane j's first column of that slab, for j >= 32 lane (j - 32)'s second
    for (int i = threadIdx.x; i < t.nslabs * kTileCols; i += kBwdThreads) {
        const float v = bias_s[i];
        const int sl = i / kTileCols, j = i % kTileCols;
        if (v != 0.f) atomicAdd(a.g_bias + (j < 32 ? tile_col_a<PAIRWISE>(sl, j, a.H) : tile_col_b<PAIRWISE>(sl, j - 32, a.H)), v);
    }
    if (SIGNAL && left_block >= 0) bucket_signal(t.sig, left_block);
    if (SIGNAL && block >= 0) bucket_signal(t.sig, block);
}

// ------------------------------------------------------- factoriser helper kernels
// table[i] = l0w[i] + l0f[i mod block]   (model/builder.rs:421-424 `repeat`, then `+`)
static __global__ void factoriser_merge_kernel(const float4* __restrict__ l0w, const float4* __restrict__ l0f,
                                        float4* __restrict__ table, size_t n4, size_t block4) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x)
        table[i] = add4(l0w[i], l0f[i % block4]);
}
// g_l0f[i] = sum over the tiled copies of g_l0w, first copy first (reduce.rs:96-120)
// `g_l0w` points at the first of `copies` consecutive copies; with `accumulate` the sum is added
// to what g_l0f already holds (the copies are then visited in several launches).
static __global__ void factoriser_grad_kernel(const float4* __restrict__ g_l0w, float4* __restrict__ g_l0f, size_t block4,
                                       int copies, int accumulate) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < block4; i += (size_t)gridDim.x * blockDim.x) {
        float4 acc = g_l0w[i];
        for (int k = 1; k < copies; k++) acc = add4(acc, g_l0w[(size_t)k * block4 + i]);
        g_l0f[i] = accumulate ? add4(g_l0f[i], acc) : acc;
    }
}

}  // namespace b200
