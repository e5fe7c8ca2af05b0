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
//              aligned block of R table rows (king buckets).  A CTA stages one
//              R x 32-column tile in shared memory and serves every (position,
//              perspective) of that block from it; the backward accumulates the
//              gradient tile in shared memory and writes it out once.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr uint32_t kNoFeature = 0xFFFFu;
constexpr int kStatusOutsideBlock = 1;  // a feature fell outside its position's declared row block

struct FtArgs {
    const float* table;  // [n_inputs][H] effective weights (l0w, or l0w + tiled l0f)
    const float* bias;   // [H]
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
    int nslabs, nchunks;     // H/32 column slabs; position chunks per (block, slab)
    const int* pair_order;   // [2n] pair ids (position*2 + perspective) grouped by block, or null = identity
    const int* block_begin;  // [nblocks+1] offsets into pair_order
    int* status;
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
// A tile row holds 32 floats of one table row: columns [32s, 32s+32), or with
// pairwise the 16 low-half columns [16s, 16s+16) followed by their 16 partners
// [H/2 + 16s, H/2 + 16s + 16).  Lane l owns tile column l throughout.
template <bool PAIRWISE>
__device__ __forceinline__ int tile_quad_col(int q, int slab, int H) {  // first column of 16-byte quad q of a tile row
    if (PAIRWISE) return q < 4 ? slab * 16 + q * 4 : H / 2 + slab * 16 + (q - 4) * 4;
    return slab * 32 + q * 4;
}
template <bool PAIRWISE>
__device__ __forceinline__ int tile_lane_col(int lane, int slab, int H) {
    if (PAIRWISE) return lane < 16 ? slab * 16 + lane : H / 2 + slab * 16 + (lane - 16);
    return slab * 32 + lane;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

struct TileWork {
    int block, slab, begin, end;  // pair_order range [begin, end) served by this CTA
};
__device__ __forceinline__ TileWork tile_work(const TileArgs& t) {
    TileWork w;
    const int chunk = blockIdx.x % t.nchunks;
    const int rest = blockIdx.x / t.nchunks;
    w.slab = rest % t.nslabs;
    w.block = rest / t.nslabs;
    const int b0 = t.block_begin[w.block], cnt = t.block_begin[w.block + 1] - b0;
    w.begin = b0 + (int)(((long long)cnt * chunk) / t.nchunks);
    w.end = b0 + (int)(((long long)cnt * (chunk + 1)) / t.nchunks);
    return w;
}

// Loads one position's slots and turns them into tile offsets (row * 32).  Returns
// the masks of usable slots; a valid feature outside the block raises the status
// bit and is dropped rather than read out of bounds.
__device__ __forceinline__ void tile_slots(const FtArgs& a, const TileArgs& t, int block, int pair, int lane,
                                           int (&off)[2], unsigned (&mask)[2]) {
    const int b = pair >> 1, p = pair & 1;
    const uint16_t* list = (p ? a.idx_nstm : a.idx_stm) + (size_t)b * a.nnz;
    uint32_t slot[2];
    load_slots(list, a.nnz, lane, slot[0], slot[1]);
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const bool valid = slot[h] < (uint32_t)a.n_inputs;
        const int local = (int)slot[h] - block * t.block_rows;
        const bool inside = valid && (unsigned)local < (unsigned)t.block_rows;
        if (valid && !inside) atomicOr(t.status, kStatusOutsideBlock);
        off[h] = inside ? local * 32 : 0;
        mask[h] = __ballot_sync(0xffffffffu, inside);
    }
}

// grid = nblocks * nslabs * nchunks CTAs of 512 threads; dynamic smem = R*32 floats.
template <bool PAIRWISE>
__global__ void __launch_bounds__(512, 2) ft_forward_tiled_kernel(FtArgs a, TileArgs t) {
    extern __shared__ __align__(16) float tile[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const TileWork w = tile_work(t);
    const int R = t.block_rows;
    for (int i = threadIdx.x; i < R * 8; i += blockDim.x) {
        const int row = i >> 3, q = i & 7;
        cp_async16(&tile[row * 32 + q * 4],
                   a.table + (size_t)(w.block * R + row) * a.H + tile_quad_col<PAIRWISE>(q, w.slab, a.H));
    }
    const int col = tile_lane_col<PAIRWISE>(lane, w.slab, a.H);
    const float bias = a.bias[col];
    cp_async_wait_all();
    __syncthreads();
    const float* mine = tile + lane;
    for (int i = w.begin + warp; i < w.end; i += nwarps) {
        const int pair = t.pair_order ? t.pair_order[i] : i;
        int off[2];
        unsigned mask[2];
        tile_slots(a, t, w.block, pair, lane, off, mask);
        float acc = 0.f;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            unsigned m = mask[h];
            if (m == 0) continue;
            const int cnt = __popc(m);
            if (m == (cnt == 32 ? 0xffffffffu : (1u << cnt) - 1u)) {  // usual case: a prefix of the slots
                for (int k = 0; k < cnt; k += 4) {
                    const int o0 = __shfl_sync(0xffffffffu, off[h], k);
                    const int o1 = __shfl_sync(0xffffffffu, off[h], (k + 1) & 31);
                    const int o2 = __shfl_sync(0xffffffffu, off[h], (k + 2) & 31);
                    const int o3 = __shfl_sync(0xffffffffu, off[h], (k + 3) & 31);
                    const float v0 = mine[o0], v1 = mine[o1], v2 = mine[o2], v3 = mine[o3];
                    acc += v0;
                    if (k + 1 < cnt) acc += v1;
                    if (k + 2 < cnt) acc += v2;
                    if (k + 3 < cnt) acc += v3;
                }
            } else {
                while (m) {
                    const int s = __ffs(m) - 1;
                    m &= m - 1;
                    acc += mine[__shfl_sync(0xffffffffu, off[h], s)];
                }
            }
        }
        const float v = acc + bias;
        const int b = pair >> 1, p = pair & 1;
        if (PAIRWISE) {
            const float uval = crelu_f(v);
            a.u[(size_t)pair * a.H + col] = uval;
            const float other = __shfl_xor_sync(0xffffffffu, uval, 16);
            if (lane < 16) a.x[(size_t)b * a.H + (size_t)p * (a.H / 2) + w.slab * 16 + lane] = uval * other;
        } else {
            a.x[(size_t)b * 2 * a.H + (size_t)p * a.H + col] = ft_act_fwd(a.act, v);
        }
    }
}

// Same grid.  With nchunks == 1 each CTA owns its tile of the table gradient and
// stores it (no zeroing needed); otherwise tiles are added into a zeroed table.
template <bool PAIRWISE>
__global__ void __launch_bounds__(512, 2) ft_backward_tiled_kernel(FtArgs a, TileArgs t) {
    extern __shared__ __align__(16) float tile[];
    __shared__ float bias_red[16][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const TileWork w = tile_work(t);
    const int R = t.block_rows;
    for (int i = threadIdx.x; i < R * 8; i += blockDim.x) reinterpret_cast<float4*>(tile)[i] = make_float4(0, 0, 0, 0);
    __syncthreads();
    const int col = tile_lane_col<PAIRWISE>(lane, w.slab, a.H);
    float* mine = tile + lane;
    float bsum = 0.f;
    for (int i = w.begin + warp; i < w.end; i += nwarps) {
        const int pair = t.pair_order ? t.pair_order[i] : i;
        const int b = pair >> 1, p = pair & 1;
        float g;
        if (PAIRWISE) {
            const float uval = a.u[(size_t)pair * a.H + col];
            const float other = __shfl_xor_sync(0xffffffffu, uval, 16);
            const float d = a.dx[(size_t)b * a.H + (size_t)p * (a.H / 2) + w.slab * 16 + (lane & 15)];
            g = (d * other) * ft_act_bwd(1, uval);
        } else {
            const size_t at = (size_t)b * 2 * a.H + (size_t)p * a.H + col;
            g = a.dx[at] * ft_act_bwd(a.act, a.x[at]);
        }
        if (!__any_sync(0xffffffffu, g != 0.f)) continue;  // the reference skips zero gradients too
        bsum += g;
        int off[2];
        unsigned mask[2];
        tile_slots(a, t, w.block, pair, lane, off, mask);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            unsigned m = mask[h];
            while (m) {
                const int s = __ffs(m) - 1;
                m &= m - 1;
                const int o = __shfl_sync(0xffffffffu, off[h], s);
                if (g != 0.f) atomicAdd(mine + o, g);
            }
        }
    }
    bias_red[warp][lane] = bsum;
    __syncthreads();
    if (warp == 0) {
        float s = 0.f;
        for (int k = 0; k < nwarps; k++) s += bias_red[k][lane];
        if (s != 0.f) atomicAdd(a.g_bias + col, s);
    }
    for (int i = threadIdx.x; i < R * 8; i += blockDim.x) {
        const int row = i >> 3, q = i & 7;
        const float4 v = reinterpret_cast<const float4*>(tile)[i];
        float4* dst = reinterpret_cast<float4*>(a.g_table + (size_t)(w.block * R + row) * a.H +
                                                tile_quad_col<PAIRWISE>(q, w.slab, a.H));
        if (t.nchunks == 1)
            *dst = v;
        else if (v.x != 0.f || v.y != 0.f || v.z != 0.f || v.w != 0.f)
            atomicAdd(dst, v);
    }
}

// ------------------------------------------------------- factoriser helper kernels
// table[i] = l0w[i] + l0f[i mod block]   (model/builder.rs:421-424 `repeat`, then `+`)
__global__ void factoriser_merge_kernel(const float4* __restrict__ l0w, const float4* __restrict__ l0f,
                                        float4* __restrict__ table, size_t n4, size_t block4) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x)
        table[i] = add4(l0w[i], l0f[i % block4]);
}
// g_l0f[i] = sum over the tiled copies of g_l0w, first copy first (reduce.rs:96-120)
__global__ void factoriser_grad_kernel(const float4* __restrict__ g_l0w, float4* __restrict__ g_l0f, size_t block4,
                                       int copies) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < block4; i += (size_t)gridDim.x * blockDim.x) {
        float4 acc = g_l0w[i];
        for (int k = 1; k < copies; k++) acc = add4(acc, g_l0w[(size_t)k * block4 + i]);
        g_l0f[i] = acc;
    }
}

}  // namespace b200
