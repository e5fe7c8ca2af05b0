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

struct DenseArgs {
    const float* x;        // [n][K1] dense-stack input
    const int* buckets;    // [n] output bucket per position
    const float* targets;  // [n]
    int n, K1, O, n_dense;
    int M[3], act[3];
    const float* W[3];
    const float* B[3];
    float* a1;     // [n][M1] activated layer-1 output (kept for the weight gradients)
    float* a2;     // [n][M2]
    float* dz[3];  // gradient at each layer's selected pre-activation: [n][M_i]
    float* out;    // [n] network output
    float* loss;   // scalar, accumulated
    int want_grad;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float act_fwd(int act, float v) { return act == 0 ? v : ft_act_fwd(act, v); }
__device__ __forceinline__ float act_bwd(int act, float y) { return act == 0 ? 1.f : ft_act_bwd(act, y); }

// One warp per position: first layer as a K1-long dot product per selected row, the tiny
// remaining layers, the loss, and the backward pass down to the first layer's
// pre-activation gradient.  grid = ceil(n/8), block = 256.
template <int M1>
__global__ void __launch_bounds__(256) dense_forward_kernel(DenseArgs a) {
    __shared__ float loss_part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = blockIdx.x * 8 + warp;
    float my_loss = 0.f;
    if (b < a.n) {
        const int k = a.buckets[b];
        const int OM1 = a.O * M1;
        float acc[M1];
#pragma unroll
        for (int r = 0; r < M1; r++) acc[r] = 0.f;
        const float* xb = a.x + (size_t)b * a.K1;
        const float* w1 = a.W[0] + k * M1;
        for (int c0 = lane * 4; c0 < a.K1; c0 += 128) {
            const float4 xv = *reinterpret_cast<const float4*>(xb + c0);
            const float xs[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float* wc = w1 + (size_t)(c0 + j) * OM1;
                if (M1 % 4 == 0) {
#pragma unroll
                    for (int r = 0; r < M1; r += 4) {
                        const float4 wv = __ldg(reinterpret_cast<const float4*>(wc + r));
                        acc[r] += wv.x * xs[j];
                        acc[r + 1] += wv.y * xs[j];
                        acc[r + 2] += wv.z * xs[j];
                        acc[r + 3] += wv.w * xs[j];
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < M1; r++) acc[r] += __ldg(wc + r) * xs[j];
                }
            }
        }
        float a1v[M1];
#pragma unroll
        for (int r = 0; r < M1; r++) a1v[r] = act_fwd(a.act[0], warp_sum(acc[r]) + a.B[0][k * M1 + r]);

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

        if (a.want_grad) {
            const float s = 1.f / (1.f + expf(-o));
            const float diff = s - a.targets[b];
            my_loss = diff * diff;
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

// dx[b][c] = sum_r W1[c][k_b][r] * dz1[b][r]   (Matmul::backward, matmul.rs:99-126, on the
// selected rows).  One warp per position; grid = ceil(n/8), block = 256.
template <int M1>
__global__ void __launch_bounds__(256) dense_dx_kernel(DenseArgs a, float* dx) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int b = blockIdx.x * 8 + warp;
    if (b >= a.n) return;
    const int k = a.buckets[b];
    const int OM1 = a.O * M1;
    float g[M1];
#pragma unroll
    for (int r = 0; r < M1; r++) g[r] = a.dz[0][(size_t)b * M1 + r];
    const float* w1 = a.W[0] + k * M1;
    float* out = dx + (size_t)b * a.K1;
    for (int c0 = lane * 4; c0 < a.K1; c0 += 128) {
        float res[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float* wc = w1 + (size_t)(c0 + j) * OM1;
            float s = 0.f;
            if (M1 % 4 == 0) {
#pragma unroll
                for (int r = 0; r < M1; r += 4) {
                    const float4 wv = __ldg(reinterpret_cast<const float4*>(wc + r));
                    s += wv.x * g[r];
                    s += wv.y * g[r + 1];
                    s += wv.z * g[r + 2];
                    s += wv.w * g[r + 3];
                }
            } else {
#pragma unroll
                for (int r = 0; r < M1; r++) s += __ldg(wc + r) * g[r];
            }
            res[j] = s;
        }
        *reinterpret_cast<float4*>(out + c0) = make_float4(res[0], res[1], res[2], res[3]);
    }
}

// Weight and bias gradient of one dense layer: gW[c][k][r] += sum_b [k_b == k] dY[b][r] * X[b][c],
// gB[k][r] += sum_b [k_b == k] dY[b][r]  (Matmul::backward on the zero-padded gradient,
// reduce over the batch for the bias: model/builder.rs:263-267).
// Positions are visited in bucket-sorted order (`order`), so a thread keeps M running sums
// for the current bucket and flushes them with atomics only when the bucket changes.
// Thread c < K owns column c; thread c == K owns the bias.  grid = (ceil((K+1)/T), chunks).
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
__global__ void __launch_bounds__(256) dense_wgrad_kernel(WgradArgs a) {
    constexpr int S = 64;  // positions staged per round
    __shared__ int s_pos[S], s_bucket[S];
    __shared__ float s_dy[S][M];
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const bool is_col = c < a.K, is_bias = c == a.K;
    const int OM = a.O * M;
    const int begin = blockIdx.y * a.chunk_len, end = min(a.n, begin + a.chunk_len);
    float acc[M];
#pragma unroll
    for (int r = 0; r < M; r++) acc[r] = 0.f;
    int cur = -1;
    auto flush = [&]() {
        if (cur >= 0 && (is_col || is_bias)) {
            float* dst = is_col ? a.gW + (size_t)c * OM + cur * M : a.gB + cur * M;
#pragma unroll
            for (int r = 0; r < M; r++) {
                if (acc[r] != 0.f) atomicAdd(dst + r, acc[r]);
                acc[r] = 0.f;
            }
        }
    };
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
        __syncthreads();
        for (int j0 = 0; j0 < cnt; j0 += 4) {
            float xv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int j = j0 + u;
                xv[u] = j < cnt ? (is_col ? a.X[(size_t)s_pos[j] * a.K + c] : 1.f) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int j = j0 + u;
                if (j < cnt) {
                    const int k = s_bucket[j];
                    if (k != cur) {
                        flush();
                        cur = k;
                    }
#pragma unroll
                    for (int r = 0; r < M; r++) acc[r] += s_dy[j][r] * xv[u];
                }
            }
        }
    }
    flush();
}

}  // namespace b200
