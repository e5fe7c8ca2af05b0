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

}  // namespace b200
