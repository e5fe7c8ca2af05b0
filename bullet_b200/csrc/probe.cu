// Bandwidth probes that give the roofline denominators this library quotes for kernels whose working set
// stays in L2: repeated 16-byte loads of a buffer small enough to stay resident (the gather forward's
// row reads) and repeated 16-byte vector reductions into such a buffer (the gather backward's
// red.global.add.v4.f32; also with 4 and 8 bytes per lane, as the tiled backward issues them).  With a buffer
// far larger than L2 the same loads measure HBM.
// No counterpart in the reference; the numbers are reported by bench.py beside the kernels' achieved rates.
#include <cuda_runtime.h>

#include <stdint.h>

#include "../../include/bullet_b200.h"
#include "common.h"

#define CK(call)                                                                                          \
    do {                                                                                                  \
        cudaError_t e_ = (call);                                                                          \
        if (e_ != cudaSuccess)                                                                            \
            return b200::fail(B200_ERR_CUDA, "%s failed: %s (%d) at %s:%d", #call, cudaGetErrorString(e_), \
                              (int)e_, __FILE__, __LINE__);                                               \
    } while (0)

namespace {

// every thread sums `reps` passes over the buffer, 16 bytes per load, four loads in flight
__global__ void __launch_bounds__(512) probe_read_kernel(const float4* __restrict__ buf, size_t n4, int reps, float* sink) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < reps; r++) {
        size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
        for (; i + 3 * stride < n4; i += 4 * stride) {
            const float4 a = __ldcg(buf + i), b = __ldcg(buf + i + stride), c = __ldcg(buf + i + 2 * stride), d = __ldcg(buf + i + 3 * stride);
            acc.x += a.x + b.x + c.x + d.x;
            acc.y += a.y + b.y + c.y + d.y;
            acc.z += a.z + b.z + c.z + d.z;
            acc.w += a.w + b.w + c.w + d.w;
        }
        for (; i < n4; i += stride) {
            const float4 a = __ldcg(buf + i);
            acc.x += a.x, acc.y += a.y, acc.z += a.z, acc.w += a.w;
        }
    }
    if (acc.x + acc.y + acc.z + acc.w == 12345.678f) *sink = acc.x;  // keeps the loads alive
}

__global__ void __launch_bounds__(512) probe_atomic_kernel(float4* buf, size_t n4, int reps) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
    for (int r = 0; r < reps; r++)
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) atomicAdd(buf + i, one);
}

// the same with one float (kind 2) or two floats (kind 3) per lane: a warp's reduction still covers one
// contiguous 128- or 256-byte run, as the tiled backward's per-row reductions do
__global__ void __launch_bounds__(512) probe_atomic1_kernel(float* buf, size_t n, int reps) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (int r = 0; r < reps; r++)
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) atomicAdd(buf + i, 1.f);
}
__global__ void __launch_bounds__(512) probe_atomic2_kernel(float2* buf, size_t n2, int reps) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const float2 one = make_float2(1.f, 1.f);
    for (int r = 0; r < reps; r++)
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n2; i += stride) atomicAdd(buf + i, one);
}

}  // namespace

extern "C" int b200_probe_bandwidth(int device, int kind, int64_t bytes, int reps, double* gb_per_s) {
    if (!gb_per_s || bytes < 4096 || bytes % 16 || reps < 1 || kind < 0 || kind > 3)
        return b200::fail(B200_ERR_ARG, "probe_bandwidth: kind 0 (loads), 1, 2 or 3 (reductions of 16, 4 or 8 bytes per lane), bytes a multiple of 16, reps >= 1");
    CK(cudaSetDevice(device));
    int sms = 0;
    CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    float4* buf = nullptr;
    float* sink = nullptr;
    CK(cudaMalloc(&buf, (size_t)bytes));
    CK(cudaMalloc(&sink, sizeof(float)));
    CK(cudaMemset(buf, 0, (size_t)bytes));
    cudaEvent_t t0, t1;
    CK(cudaEventCreate(&t0));
    CK(cudaEventCreate(&t1));
    const size_t n4 = (size_t)bytes / 16;
    const int grid = sms * 4;
    float best = 1e30f;
    for (int round = 0; round < 4; round++) {  // the first round warms the cache; the best of the rest counts
        CK(cudaEventRecord(t0));
        if (kind == 0)
            probe_read_kernel<<<grid, 512>>>(buf, n4, reps, sink);
        else if (kind == 1)
            probe_atomic_kernel<<<grid, 512>>>(buf, n4, reps);
        else if (kind == 2)
            probe_atomic1_kernel<<<grid, 512>>>(reinterpret_cast<float*>(buf), n4 * 4, reps);
        else
            probe_atomic2_kernel<<<grid, 512>>>(reinterpret_cast<float2*>(buf), n4 * 2, reps);
        CK(cudaEventRecord(t1));
        CK(cudaEventSynchronize(t1));
        CK(cudaGetLastError());
        float ms = 0.f;
        CK(cudaEventElapsedTime(&ms, t0, t1));
        if (round > 0 && ms < best) best = ms;
    }
    *gb_per_s = (double)bytes * reps / (best * 1e-3) / 1e9;
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    cudaFree(buf);
    cudaFree(sink);
    return 0;
}
