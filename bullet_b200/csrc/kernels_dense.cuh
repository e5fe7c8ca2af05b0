// Output-bucketed dense layers, sigmoid-MSE loss and their backward.
//
// Reference semantics (jw1912/bullet): every dense layer is `W.matmul(x) + b`
// (crates/compiler/src/model/builder.rs:145-147, Matmul::evaluate in
// crates/compiler/src/tensor/operation/linear/matmul.rs:62-93) computed for ALL output
// buckets and then narrowed by `select` (crates/compiler/src/tensor/operation/index/select.rs:12-26);
// its backward pads the selected gradient with zeros (select.rs:93-110).  Here only the
// selected bucket's rows are ever computed, which gives the same numbers: the rows of the
// other buckets contribute exactly zero to every gradient.
// Weights are column-major: element (bucket k, row r, column c) of layer i sits at
// W[c * (O*M_i) + k*M_i + r].
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels_ft.cuh"

namespace b200 {

constexpr int kDenseTile = 32;    // positions of one output bucket handled by one CTA (8 warps)
constexpr int kDenseWarpPos = 4;  // of which each warp takes four
constexpr int kDenseChunk = 128;  // first-layer columns staged in shared memory per round

struct DenseArgs {
    const float* x;        // [n][K1] dense-stack input
    const int* buckets;    // [n] output bucket per position
    const float* targets;  // [n]
    const int* order;      // [n] position ids grouped by output bucket
    const int2* tiles;     // [ntiles] (begin, count <= kDenseTile) ranges of `order`, one bucket each
    int n, ntiles, K1, O, n_dense;
    int M[3], act[3];
    const float* W[3];
    const float* B[3];
    const float* W1g;  // first-layer weights regrouped as [bucket][column][row]
    float* a1;         // [n][M1] activated layer-1 output (kept for the weight gradients)
    float* a2;         // [n][M2]
    float* dz[3];      // gradient at each layer's selected pre-activation: [n][M_i]
    float* out;        // [n] network output
    float* loss;       // scalar, accumulated
    int want_grad;
    // the register-tiled forward also forms the weight and bias gradients of the layers after the
    // first (it holds everything they need in shared memory): gradient tensors of layers 2 and 3
    int fuse_small;
    float* gW[3];
    float* gB[3];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float act_fwd(int act, float v) { return act == 0 ? v : ft_act_fwd(act, v); }
__device__ __forceinline__ float act_bwd(int act, float y) { return act == 0 ? 1.f : ft_act_bwd(act, y); }

// l1w is stored column-major over ALL buckets' rows, so the M1 rows of one bucket for
// consecutive columns lie O*M1 floats apart.  The kernels below read the regrouped copy
// W1g[bucket][column][row], in which one bucket's weights for a run of columns are contiguous.
__global__ void dense_regroup_kernel(const float* __restrict__ W1, float* __restrict__ W1g, int K1, int O, int M1) {
    const int total = K1 * O * M1;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int r = i % M1, c = (i / M1) % K1, k = i / (M1 * K1);
        W1g[i] = W1[(size_t)c * (O * M1) + k * M1 + r];
    }
}

// Shared-memory stride of one column's M1 weights: padded so that the 128-bit reads of
// eight neighbouring lanes (neighbouring columns) fall into different banks.
template <int M1>
__host__ __device__ constexpr int dense_col_stride() { return M1 % 8 == 0 ? M1 + 4 : M1; }

__device__ __forceinline__ void dense_cp_async16(void* smem, const void* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void dense_cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void dense_cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Stages columns [chunk*128, chunk*128+128) of bucket k's first-layer weights; columns past
// K1 are zero-filled.  All 256 threads take part.
template <int M1>
__device__ __forceinline__ void dense_stage_chunk(const DenseArgs& a, int k, int chunk, float* buf, bool commit = true) {
    constexpr int MP = dense_col_stride<M1>();
    const int c_begin = chunk * kDenseChunk;
    const float* src = a.W1g + ((size_t)k * a.K1 + c_begin) * M1;
    if (M1 % 4 == 0) {
        constexpr int Q = M1 >= 4 ? M1 / 4 : 1;  // 16-byte pieces per column
        for (int i = threadIdx.x; i < kDenseChunk * Q; i += blockDim.x) {
            const int c = i / Q, q = i % Q;
            float* dst = buf + c * MP + q * 4;
            if (c_begin + c < a.K1)
                dense_cp_async16(dst, src + (size_t)c * M1 + q * 4);
            else
                *reinterpret_cast<float4*>(dst) = make_float4(0, 0, 0, 0);
        }
    } else {
        for (int i = threadIdx.x; i < kDenseChunk * M1; i += blockDim.x)
            buf[i] = c_begin + i / M1 < a.K1 ? __ldg(src + i) : 0.f;
    }
    if (commit) dense_cp_commit();
}

template <int M1>
__device__ __forceinline__ void dense_read_weights(const float* buf, int c, float (&w)[M1]) {
    constexpr int MP = dense_col_stride<M1>();
    if (M1 % 4 == 0) {
#pragma unroll
        for (int r = 0; r < M1; r += 4) {
            const float4 wv = *reinterpret_cast<const float4*>(buf + c * MP + r);
            w[r] = wv.x, w[r + 1] = wv.y, w[r + 2] = wv.z, w[r + 3] = wv.w;
        }
    } else {
#pragma unroll
        for (int r = 0; r < M1; r++) w[r] = buf[c * MP + r];
    }
}

// One CTA per tile of up to 32 positions of the same output bucket, four per warp.  The
// bucket's first-layer weights AND the tile's rows of x stream through shared memory in
// 128-column chunks, three chunks in flight (cp.async), so no global latency sits between
// the chunks; lane l takes columns l, l+32, l+64, l+96 of a chunk.  After the K1-long dot
// products the tiny remaining layers, the loss and the backward pass down to the first
// layer's pre-activation gradient follow per position.  grid = ntiles, block = 256, dynamic
// shared memory = dense_fwd_smem<M1>().
constexpr int kDenseStages = 3;
template <int M1>
__host__ __device__ constexpr size_t dense_fwd_smem() {
    return (size_t)kDenseStages * (kDenseChunk * dense_col_stride<M1>() + kDenseTile * kDenseChunk) * sizeof(float);
}

template <int M1>
__global__ void __launch_bounds__(256, (M1 > 16 ? 1 : 2)) dense_forward_kernel(DenseArgs a) {
    constexpr int P = kDenseWarpPos, MP = dense_col_stride<M1>();
    constexpr int kStageFloats = kDenseChunk * MP + kDenseTile * kDenseChunk;
    extern __shared__ __align__(16) float dense_smem[];
    __shared__ float loss_part[8];
    __shared__ int s_pos[kDenseTile];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int2 t = a.tiles[blockIdx.x];
    if (threadIdx.x < kDenseTile) s_pos[threadIdx.x] = a.order[t.x + min((int)threadIdx.x, t.y - 1)];
    __syncthreads();
    const int k = a.buckets[s_pos[0]];
    const int npos = max(0, min(P, t.y - warp * P));
    int pos[P];
#pragma unroll
    for (int j = 0; j < P; j++) pos[j] = s_pos[min(warp * P + j, t.y - 1)];
    float acc[P][M1];
#pragma unroll
    for (int j = 0; j < P; j++)
#pragma unroll
        for (int r = 0; r < M1; r++) acc[j][r] = 0.f;
    const int nchunks = (a.K1 + kDenseChunk - 1) / kDenseChunk;
    // one cp.async group per chunk: the bucket's weights and the tile's x for 128 columns
    auto stage = [&](int ch) {
        if (ch < nchunks) {
            float* wb = dense_smem + (ch % kDenseStages) * kStageFloats;
            float* xb = wb + kDenseChunk * MP;
            dense_stage_chunk<M1>(a, k, ch, wb, false);
            for (int i = threadIdx.x; i < kDenseTile * (kDenseChunk / 4); i += blockDim.x) {
                const int p = i / (kDenseChunk / 4), q = i % (kDenseChunk / 4);
                const int c = ch * kDenseChunk + q * 4;  // K1 is a multiple of four: a quad is inside or outside
                float* dst = xb + p * kDenseChunk + q * 4;
                if (c < a.K1)
                    dense_cp_async16(dst, a.x + (size_t)s_pos[p] * a.K1 + c);
                else
                    *reinterpret_cast<float4*>(dst) = make_float4(0, 0, 0, 0);
            }
        }
        dense_cp_commit();  // an empty group past the end keeps the group count in step with `ch`
    };
    stage(0);
    stage(1);
    for (int ch = 0; ch < nchunks; ch++) {
        stage(ch + 2);
        dense_cp_wait<kDenseStages - 1>();  // chunk ch has landed
        __syncthreads();
        if (npos) {
            const float* wb = dense_smem + (ch % kDenseStages) * kStageFloats;
            const float* xb = wb + kDenseChunk * MP + (warp * P) * kDenseChunk;
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                float w[M1];
                dense_read_weights<M1>(wb, jj * 32 + lane, w);
#pragma unroll
                for (int j = 0; j < P; j++) {
                    const float xv = xb[j * kDenseChunk + jj * 32 + lane];
#pragma unroll
                    for (int r = 0; r < M1; r++) acc[j][r] += w[r] * xv;
                }
            }
        }
        __syncthreads();  // the stage read here is refilled by the next iteration
    }
    float my_loss = 0.f;
#pragma unroll
    for (int j = 0; j < P; j++) {
        if (j >= npos) break;  // warp-uniform
        const int b = pos[j];
        float a1v[M1];
#pragma unroll
        for (int r = 0; r < M1; r++) a1v[r] = act_fwd(a.act[0], warp_sum(acc[j][r]) + a.B[0][k * M1 + r]);

        float o;        // network output
        float a2v = 0;  // lane r2 holds a2[r2] when there are three layers
        if (a.n_dense == 1) {
            o = a1v[0];
        } else {
            const int M2 = a.M[1], OM2 = a.O * M2;
            float z2 = 0.f;
            if (lane < M2) {
#pragma unroll
                for (int c = 0; c < M1; c++) z2 += a.W[1][c * OM2 + k * M2 + lane] * a1v[c];
                z2 += a.B[1][k * M2 + lane];
            }
            if (a.n_dense == 2) {
                o = __shfl_sync(0xffffffffu, z2, 0);
            } else {
                a2v = lane < M2 ? act_fwd(a.act[1], z2) : 0.f;
                const float term = lane < M2 ? a.W[2][lane * a.O + k] * a2v : 0.f;
                o = warp_sum(term) + a.B[2][k];
            }
        }
        if (lane == 0) a.out[b] = o;
        if (!a.want_grad) continue;

        const float s = 1.f / (1.f + expf(-o));
        const float diff = s - a.targets[b];
        my_loss += diff * diff;
        const float dout = (diff + diff) * (s * (1.f - s));
        float dz1[M1];
        if (a.n_dense == 1) {
            dz1[0] = dout;  // M1 == 1, no activation on the last layer
        } else if (a.n_dense == 2) {
            if (lane == 0) a.dz[1][b] = dout;
#pragma unroll
            for (int c = 0; c < M1; c++) dz1[c] = (a.W[1][c * a.O + k] * dout) * act_bwd(a.act[0], a1v[c]);
        } else {
            const int M2 = a.M[1], OM2 = a.O * M2;
            if (lane == 0) a.dz[2][b] = dout;
            float dz2 = 0.f;
            if (lane < M2) {
                dz2 = (a.W[2][lane * a.O + k] * dout) * act_bwd(a.act[1], a2v);
                a.dz[1][(size_t)b * M2 + lane] = dz2;
                a.a2[(size_t)b * M2 + lane] = a2v;
            }
#pragma unroll
            for (int c = 0; c < M1; c++) {
                const float term = lane < M2 ? a.W[1][c * OM2 + k * M2 + lane] * dz2 : 0.f;
                dz1[c] = warp_sum(term) * act_bwd(a.act[0], a1v[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < M1; c++)
            if (lane == (c & 31)) {
                a.dz[0][(size_t)b * M1 + c] = dz1[c];
                if (a.n_dense > 1) a.a1[(size_t)b * M1 + c] = a1v[c];
            }
    }
    if (a.want_grad) {
        if (lane == 0) loss_part[warp] = my_loss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float s = 0.f;
            for (int w = 0; w < 8; w++) s += loss_part[w];
            atomicAdd(a.loss, s);
        }
    }
}

// Register-tiled forward for M1 a multiple of four and two or three dense layers.  Same
// tiles, staging pipeline and results as dense_forward_kernel, different work split: the M1 x 32
// block of first-layer outputs of a tile is cut into (four rows) x (M1/4 positions) pieces, one
// per lane, and the eight warps split each 128-column chunk into 16-column slices.  A lane
// then reads, per four columns, four 16-byte weight pieces (M1/4 distinct addresses in the
// warp: a broadcast) and M1/4 16-byte pieces of x (32/(M1/4) distinct addresses, rows padded
// by four floats so they fall into different banks): one shared-memory wavefront per load
// instead of four, and no shuffles.  The warps' partial sums meet in shared memory; the small
// layers, the loss and the way back to the first layer's pre-activation gradient run from
// shared memory with one warp per position.
// grid = ntiles, block = 256, dynamic shared memory = dense_fwd_tile_smem<M1>().
constexpr int kDenseXStride = kDenseChunk + 4;
template <int M1>
__host__ __device__ constexpr size_t dense_fwd_tile_smem() {
    return (size_t)kDenseStages * (kDenseChunk * M1 + kDenseTile * kDenseXStride) * sizeof(float);
}

template <int M1>
__global__ void __launch_bounds__(256, 2) dense_forward_tile_kernel(DenseArgs a) {
    static_assert(M1 % 4 == 0 && M1 <= 32, "four-row pieces");
    constexpr int RG = M1 / 4;           // row groups = positions per lane
    constexpr int PG = 32 / RG;          // position groups in a warp
    constexpr int XS = kDenseXStride;
    constexpr int kStageFloats = kDenseChunk * M1 + kDenseTile * XS;
    static_assert(8 * kDenseTile * M1 <= kDenseStages * kStageFloats, "partial sums reuse the stage buffers");
    extern __shared__ __align__(16) float dense_smem[];
    __shared__ float s_w2[M1][33], s_b2[32], s_w3[32], s_a1[kDenseTile][M1], loss_part[8];
    __shared__ float s_dz2[kDenseTile][33], s_a2[kDenseTile][33], s_dout[kDenseTile];  // kept per position for the small gradients
    __shared__ int s_pos[kDenseTile];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rg = lane % RG, pg = lane / RG;
    const int2 t = a.tiles[blockIdx.x];
    if (threadIdx.x < kDenseTile) s_pos[threadIdx.x] = a.order[t.x + min((int)threadIdx.x, t.y - 1)];
    __syncthreads();
    const int k = a.buckets[s_pos[0]];
    const int M2 = a.M[1], OM2 = a.O * M2;
    // the bucket's small-layer weights: needed only after the long loop
    for (int i = threadIdx.x; i < M1 * M2; i += blockDim.x) s_w2[i / M2][i % M2] = a.W[1][(i / M2) * OM2 + k * M2 + i % M2];
    if (threadIdx.x < 32) {
        const bool on = (int)threadIdx.x < M2;
        s_b2[threadIdx.x] = on ? a.B[1][k * M2 + threadIdx.x] : 0.f;
        s_w3[threadIdx.x] = on && a.n_dense == 3 ? a.W[2][threadIdx.x * a.O + k] : 0.f;
    }

    float acc[RG][4];
#pragma unroll
    for (int i = 0; i < RG; i++)
#pragma unroll
        for (int r = 0; r < 4; r++) acc[i][r] = 0.f;
    const int nchunks = (a.K1 + kDenseChunk - 1) / kDenseChunk;
    auto stage = [&](int ch) {
        if (ch < nchunks) {
            float* wb = dense_smem + (ch % kDenseStages) * kStageFloats;
            float* xb = wb + kDenseChunk * M1;
            const int c_begin = ch * kDenseChunk;
            const float* src = a.W1g + ((size_t)k * a.K1 + c_begin) * M1;  // 128 columns x M1 rows, contiguous
            const int wq = min(kDenseChunk, a.K1 - c_begin) * RG;          // 16-byte pieces inside K1
            for (int i = threadIdx.x; i < kDenseChunk * RG; i += blockDim.x) {
                if (i < wq)
                    dense_cp_async16(wb + i * 4, src + i * 4);
                else
                    *reinterpret_cast<float4*>(wb + i * 4) = make_float4(0, 0, 0, 0);
            }
            for (int i = threadIdx.x; i < kDenseTile * (kDenseChunk / 4); i += blockDim.x) {
                const int p = i / (kDenseChunk / 4), q = i % (kDenseChunk / 4);
                const int c = c_begin + q * 4;  // K1 is a multiple of four: a quad is inside or outside
                float* dst = xb + p * XS + q * 4;
                if (c < a.K1)
                    dense_cp_async16(dst, a.x + (size_t)s_pos[p] * a.K1 + c);
                else
                    *reinterpret_cast<float4*>(dst) = make_float4(0, 0, 0, 0);
            }
        }
        dense_cp_commit();
    };
    stage(0);
    stage(1);
    for (int ch = 0; ch < nchunks; ch++) {
        stage(ch + 2);
        dense_cp_wait<kDenseStages - 1>();
        __syncthreads();
        const float* wb = dense_smem + (ch % kDenseStages) * kStageFloats;
        const float* xb = wb + kDenseChunk * M1;
#pragma unroll
        for (int kq = 0; kq < 4; kq++) {
            const int c0 = warp * 16 + kq * 4;
            float4 xv[RG];
#pragma unroll
            for (int i = 0; i < RG; i++) xv[i] = *reinterpret_cast<const float4*>(xb + (i * PG + pg) * XS + c0);
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                const float4 wv = *reinterpret_cast<const float4*>(wb + (c0 + kk) * M1 + rg * 4);
#pragma unroll
                for (int i = 0; i < RG; i++) {
                    const float xs = kk == 0 ? xv[i].x : kk == 1 ? xv[i].y : kk == 2 ? xv[i].z : xv[i].w;
                    acc[i][0] += wv.x * xs;
                    acc[i][1] += wv.y * xs;
                    acc[i][2] += wv.z * xs;
                    acc[i][3] += wv.w * xs;
                }
            }
        }
        __syncthreads();
    }
    // partial sums of the eight column slices -> shared memory -> first-layer activations
    float* red = dense_smem;  // [8][32][M1]; every real cp.async group has been waited for
#pragma unroll
    for (int i = 0; i < RG; i++)
        *reinterpret_cast<float4*>(red + ((warp * kDenseTile) + i * PG + pg) * M1 + rg * 4) =
            make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    __syncthreads();
    for (int o = threadIdx.x; o < kDenseTile * M1; o += blockDim.x) {
        float z = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) z += red[w * kDenseTile * M1 + o];
        const int p = o / M1, r = o % M1;
        const float v = act_fwd(a.act[0], z + a.B[0][k * M1 + r]);
        s_a1[p][r] = v;
        if (a.want_grad && p < t.y) a.a1[(size_t)s_pos[p] * M1 + r] = v;
    }
    __syncthreads();

    float my_loss = 0.f;
    for (int p = warp; p < t.y; p += 8) {  // warp-uniform
        const int b = s_pos[p];
        float z2 = 0.f;
        if (lane < M2) {
#pragma unroll
            for (int c = 0; c < M1; c++) z2 += s_w2[c][lane] * s_a1[p][c];
            z2 += s_b2[lane];
        }
        float o, a2v = 0.f;
        if (a.n_dense == 2) {
            o = __shfl_sync(0xffffffffu, z2, 0);
        } else {
            a2v = lane < M2 ? act_fwd(a.act[1], z2) : 0.f;
            o = warp_sum(s_w3[lane] * a2v) + a.B[2][k];
        }
        if (lane == 0) a.out[b] = o;
        if (!a.want_grad) continue;

        const float s = 1.f / (1.f + expf(-o));
        const float diff = s - a.targets[b];
        my_loss += diff * diff;
        const float dout = (diff + diff) * (s * (1.f - s));
        float dz2;  // gradient at the second layer's pre-activation, lane = row
        if (a.n_dense == 2) {
            dz2 = lane == 0 ? dout : 0.f;
            if (lane == 0 && !a.fuse_small) a.dz[1][b] = dout;
        } else {
            dz2 = lane < M2 ? (s_w3[lane] * dout) * act_bwd(a.act[1], a2v) : 0.f;
            if (!a.fuse_small) {
                if (lane == 0) a.dz[2][b] = dout;
                if (lane < M2) {
                    a.dz[1][(size_t)b * M2 + lane] = dz2;
                    a.a2[(size_t)b * M2 + lane] = a2v;
                }
            }
        }
        s_dz2[p][lane] = dz2;
        s_a2[p][lane] = a2v;
        if (lane == 0) s_dout[p] = dout;
        __syncwarp();
        // dz1[c] = (sum_r2 W2[c][r2] * dz2[r2]) * act'(a1[c]); 32/M1 lanes share one c
        const int c = lane % M1;
        float sum = 0.f;
        for (int r2 = lane / M1; r2 < M2; r2 += 32 / M1) sum += s_w2[c][r2] * s_dz2[p][r2];
#pragma unroll
        for (int o2 = M1; o2 < 32; o2 <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o2);
        if (lane < M1) a.dz[0][(size_t)b * M1 + c] = sum * act_bwd(a.act[0], s_a1[p][c]);
        __syncwarp();
    }
    if (a.want_grad) {
        if (lane == 0) loss_part[warp] = my_loss;
        __syncthreads();
        if (threadIdx.x == 0) {
            float s = 0.f;
            for (int w = 0; w < 8; w++) s += loss_part[w];
            atomicAdd(a.loss, s);
        }
        if (a.fuse_small) {
            // Weight and bias gradients of the narrow layers for this tile's bucket: a thread owns
            // entries (row r, column c) of the M x (K+1) block (column K is the bias), sums over the
            // tile's positions from shared memory and adds the result with one atomic per entry
            // (Matmul::backward on the zero-padded gradient, bias = sum over the batch).
            for (int o = threadIdx.x; o < M2 * (M1 + 1); o += blockDim.x) {  // layer 2: X = a1, dY = dz2
                const int r = o % M2, c = o / M2;
                float sum = 0.f;
                for (int p = 0; p < t.y; p++) sum += s_dz2[p][r] * (c < M1 ? s_a1[p][c] : 1.f);
                if (sum != 0.f) atomicAdd(c < M1 ? a.gW[1] + (size_t)c * OM2 + k * M2 + r : a.gB[1] + k * M2 + r, sum);
            }
            if (a.n_dense == 3)
                for (int o = threadIdx.x; o < M2 + 1; o += blockDim.x) {  // layer 3: X = a2, dY = dout (one row)
                    float sum = 0.f;
                    for (int p = 0; p < t.y; p++) sum += s_dout[p] * (o < M2 ? s_a2[p][o] : 1.f);
                    if (sum != 0.f) atomicAdd(o < M2 ? a.gW[2] + (size_t)o * a.O + k : a.gB[2] + k, sum);
                }
        }
    }
}

// dx[b][c] = sum_r W1[c][k_b][r] * dz1[b][r]   (Matmul::backward, matmul.rs:99-126, on the
// selected rows).  Same tiling and weight staging as the forward; grid = ntiles, block = 256.
template <int M1>
__global__ void __launch_bounds__(256, (M1 > 16 ? 1 : 2)) dense_dx_kernel(DenseArgs a, float* dx) {
    constexpr int P = kDenseWarpPos, MP = dense_col_stride<M1>();
    __shared__ __align__(16) float wbuf[2][kDenseChunk * MP];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int2 t = a.tiles[blockIdx.x];
    const int k = a.buckets[a.order[t.x]];
    const int npos = max(0, min(P, t.y - warp * P));
    int pos[P];
#pragma unroll
    for (int j = 0; j < P; j++) pos[j] = a.order[npos ? t.x + warp * P + min(j, npos - 1) : t.x];
    float g[P][M1];
#pragma unroll
    for (int j = 0; j < P; j++)
#pragma unroll
        for (int r = 0; r < M1; r++) g[j][r] = a.dz[0][(size_t)pos[j] * M1 + r];
    const int nchunks = (a.K1 + kDenseChunk - 1) / kDenseChunk;
    dense_stage_chunk<M1>(a, k, 0, wbuf[0]);
    for (int ch = 0; ch < nchunks; ch++) {
        if (ch + 1 < nchunks) {
            dense_stage_chunk<M1>(a, k, ch + 1, wbuf[(ch + 1) & 1]);
            dense_cp_wait<1>();
        } else {
            dense_cp_wait<0>();
        }
        __syncthreads();
        if (npos) {
            const float* buf = wbuf[ch & 1];
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                const int c = ch * kDenseChunk + jj * 32 + lane;
                float w[M1];
                dense_read_weights<M1>(buf, jj * 32 + lane, w);
#pragma unroll
                for (int j = 0; j < P; j++) {
                    float s = 0.f;
#pragma unroll
                    for (int r = 0; r < M1; r++) s += w[r] * g[j][r];
                    if (j < npos && c < a.K1) dx[(size_t)pos[j] * a.K1 + c] = s;
                }
            }
        }
        __syncthreads();
    }
}

// Weight and bias gradient of one dense layer: gW[c][k][r] += sum_b [k_b == k] dY[b][r] * X[b][c],
// gB[k][r] += sum_b [k_b == k] dY[b][r]  (Matmul::backward on the zero-padded gradient,
// reduce over the batch for the bias: model/builder.rs:263-267).
// Positions are visited in bucket-sorted order (`order`), so a thread keeps M running sums
// for the current bucket and flushes them with atomics only when the bucket changes.
// A thread owns four neighbouring columns (16 bytes of x per position, prefetched eight positions
// ahead through shared memory); the thread after the last column owns the bias.  grid = (ceil((K/4 + 1) / 128), chunks), block = 128.
struct WgradArgs {
    const float* X;      // [n][K]
    const float* dY;     // [n][M]
    const int* order;    // [n] position ids sorted by bucket, or null = identity
    const int* buckets;  // [n] by position id
    int n, K, O, chunk_len;
    float* gW;
    float* gB;
};

template <int M>
__global__ void __launch_bounds__(128) dense_wgrad_kernel(WgradArgs a) {
    constexpr int S = 64;  // positions staged per round
    __shared__ int s_pos[S], s_bucket[S];
    __shared__ __align__(16) float s_dy[S][M];
    const int c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);  // this thread's four columns c .. c+3
    const bool is_col = c < a.K, is_bias = c == a.K;             // K is a multiple of four
    const int OM = a.O * M;
    const int begin = blockIdx.y * a.chunk_len, end = min(a.n, begin + a.chunk_len);
    float acc[4][M];
#pragma unroll
    for (int q = 0; q < 4; q++)
#pragma unroll
        for (int r = 0; r < M; r++) acc[q][r] = 0.f;
    int cur = -1;
    auto flush = [&]() {  // one column's M rows are contiguous: 128-bit reductions when M allows
        if (cur >= 0 && (is_col || is_bias)) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
                float* dst = is_col ? a.gW + (size_t)(c + q) * OM + cur * M : a.gB + cur * M;
                if (is_col || q == 0) {
                    if (M % 4 == 0) {
#pragma unroll
                        for (int r = 0; r < M; r += 4)
                            atomicAdd(reinterpret_cast<float4*>(dst + r), make_float4(acc[q][r], acc[q][r + 1], acc[q][r + 2], acc[q][r + 3]));
                    } else {
#pragma unroll
                        for (int r = 0; r < M; r++)
                            if (acc[q][r] != 0.f) atomicAdd(dst + r, acc[q][r]);
                    }
                }
#pragma unroll
                for (int r = 0; r < M; r++) acc[q][r] = 0.f;
            }
        }
    };
    // x reaches the thread through a private ring of D shared-memory slots filled by cp.async:
    // D positions' loads stay in flight at no register cost, so HBM latency hides behind the FMAs
    constexpr int D = 8;
    __shared__ float4 s_x[D][128];
    float4* my_slot = &s_x[0][threadIdx.x];
    for (int base = begin; base < end; base += S) {
        const int cnt = min(S, end - base);
        __syncthreads();
        for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
            const int pos = a.order ? a.order[base + i] : base + i;
            s_pos[i] = pos;
            s_bucket[i] = a.buckets[pos];
        }
        __syncthreads();
        for (int i = threadIdx.x; i < cnt * M; i += blockDim.x) s_dy[i / M][i % M] = a.dY[(size_t)s_pos[i / M] * M + i % M];
#pragma unroll
        for (int u = 0; u < D; u++) {
            if (u < cnt && is_col) dense_cp_async16(my_slot + u * 128, a.X + (size_t)s_pos[u] * a.K + c);
            dense_cp_commit();
        }
        __syncthreads();
        for (int j = 0; j < cnt; j++) {
            dense_cp_wait<D - 1>();  // position j's 16 bytes have landed
            const float4 xv = is_col ? my_slot[(j & (D - 1)) * 128] : make_float4(is_bias ? 1.f : 0.f, 0.f, 0.f, 0.f);  // the bias "column" sees x = 1
            const int k = s_bucket[j];
            if (k != cur) {
                flush();
                cur = k;
            }
            const float xs[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int r = 0; r < M; r++) {
                const float dy = s_dy[j][r];
#pragma unroll
                for (int q = 0; q < 4; q++) acc[q][r] += dy * xs[q];
            }
            // refill the slot just read (after its value has been used) with position j + D
            if (j + D < cnt && is_col) dense_cp_async16(my_slot + (j & (D - 1)) * 128, a.X + (size_t)s_pos[j + D] * a.K + c);
            dense_cp_commit();
        }
    }
    flush();
}

// Weight and bias gradients of the narrow layers after the first, all in one launch: one CTA
// per tile of up to 32 positions of one output bucket (the tiles of the forward).  For layer
// l >= 1 with input X = the activated output of layer l-1 (K values per position) and dY = the
// gradient at its selected pre-activation (M values): a thread owns entries (row r, column c)
// of the bucket's M x (K+1) block (column K is the bias), sums dY[p][r] * X[p][c] over the
// tile's positions from shared memory and adds the result with one atomic per entry.
// grid = ntiles, block = 256.
struct SmallGradArgs {
    const int* order;
    const int2* tiles;
    const int* buckets;
    int O, n_layers;     // layers handled here: dense layers 1 .. n_dense-1
    int K[2], M[2];
    const float* X[2];   // [n][K]
    const float* dY[2];  // [n][M]
    float* gW[2];
    float* gB[2];
};

static __global__ void __launch_bounds__(256) dense_small_grads_kernel(SmallGradArgs a) {
    __shared__ float s_x[32][33], s_dy[32][33];
    __shared__ int s_pos[32];
    const int2 t = a.tiles[blockIdx.x];
    if (threadIdx.x < t.y) s_pos[threadIdx.x] = a.order[t.x + threadIdx.x];
    __syncthreads();
    const int k = a.buckets[s_pos[0]];
    for (int l = 0; l < a.n_layers; l++) {
        const int K = a.K[l], M = a.M[l], OM = a.O * M;
        __syncthreads();
        for (int i = threadIdx.x; i < t.y * (K + 1); i += blockDim.x) {
            const int p = i / (K + 1), c = i % (K + 1);
            s_x[p][c] = c < K ? a.X[l][(size_t)s_pos[p] * K + c] : 1.f;
        }
        for (int i = threadIdx.x; i < t.y * M; i += blockDim.x) {
            const int p = i / M, r = i % M;
            s_dy[p][r] = a.dY[l][(size_t)s_pos[p] * M + r];
        }
        __syncthreads();
        for (int o = threadIdx.x; o < M * (K + 1); o += blockDim.x) {
            const int r = o % M, c = o / M;
            float sum = 0.f;
            for (int p = 0; p < t.y; p++) sum += s_dy[p][r] * s_x[p][c];
            if (sum != 0.f) atomicAdd(c < K ? a.gW[l] + (size_t)c * OM + k * M + r : a.gB[l] + k * M + r, sum);
        }
    }
}

}  // namespace b200
