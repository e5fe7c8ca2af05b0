// Operator-level entry points: the feature-transformer forward on caller-owned device memory.
//
// b200_op_ft_forward computes, for both perspectives of n positions, what the reference's
// graph computes with SparseMatmul::evaluate (crates/compiler/src/tensor/operation/linear/sparse.rs:86-119)
// followed by the bias add (crates/compiler/src/model/builder.rs:145-147), the activation
// (crates/compiler/src/tensor/operation/autograd/dfo.rs:47-88), the optional pairwise product
// (model/builder.rs:390-393) and the stm|nstm concat (model/builder.rs:375-388) — the same
// kernel b200_step runs, but without a b200_net: table, bias, packed index lists and outputs are
// device pointers of the caller.
//
// The tiled kernel visits (position, perspective) pairs grouped by the table row block their
// features live in.  A b200_net gets that grouping from the host packer; here it is built on
// the device into scratch memory: a block id per pair, a histogram, its scan and the grouped
// pair order.  b200_op_ft_forward takes that scratch from cudaMalloc for the duration of the
// call; b200_op_ft_forward_noalloc keeps it in a fixed array that is part of the library image.
#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <mutex>

#include "../../include/bullet_b200.h"
#include "common.h"
#include "kernels_ft.cuh"

#define CK(call)                                                                                          \
    do {                                                                                                  \
        cudaError_t e_ = (call);                                                                          \
        if (e_ != cudaSuccess)                                                                            \
            return b200::fail(B200_ERR_CUDA, "%s failed: %s (%d) at %s:%d", #call, cudaGetErrorString(e_), \
                              (int)e_, __FILE__, __LINE__);                                               \
    } while (0)

namespace {

constexpr int kMaxBlocks = 1024;  // table row blocks the grouping supports

// Scratch layout, in ints: [0] status word, [1 .. 1+kMaxBlocks] histogram then running
// cursors, [.. +kMaxBlocks+1] block_begin, one work item (int4) per block, then per pair:
// block id [2n], pair order [2n], prepared list length [2n], and the prepared row lists
// [2n][nnz rounded up to 4] as u16.
// Every section starts on a 256-byte boundary: the row lists are read with 16-byte loads.
constexpr size_t kSectionAlign = 64;  // ints
constexpr size_t align_ints(size_t v) { return (v + kSectionAlign - 1) / kSectionAlign * kSectionAlign; }
constexpr size_t kItemsAt = align_ints(1 + (kMaxBlocks + 1) + (kMaxBlocks + 1));
constexpr size_t kScratchHeader = kItemsAt + 4 * kMaxBlocks;
int list_len(int nnz) { return (nnz + 7) & ~7; }  // 16-byte groups of u16 row indices
size_t scratch_ints(int n, int nnz) { return kScratchHeader + 3 * align_ints((size_t)2 * n) + (size_t)2 * n * list_len(nnz); }

// Scratch of b200_op_ft_forward_noalloc: room for B200_OP_NOALLOC_MAX_POSITIONS positions of
// up to 32 index slots (about 4.6 MB).  It is a file-scope device array, so every GPU on
// which the library is loaded carries it from load until the process exits, and every call
// on that GPU uses the same bytes.
constexpr size_t kStaticInts =
    kScratchHeader + 3 * align_ints((size_t)2 * B200_OP_NOALLOC_MAX_POSITIONS) + (size_t)2 * B200_OP_NOALLOC_MAX_POSITIONS * 32;
static __device__ __align__(256) int g_op_scratch[kStaticInts];

__global__ void group_count_kernel(const uint16_t* stm, const uint16_t* nstm, int n, int nnz, int n_inputs,
                                   int block_rows, int* counts, int* blk) {
    const int pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= 2 * n) return;
    const uint16_t* list = ((pair & 1) ? nstm : stm) + (size_t)(pair >> 1) * nnz;
    int b = 0;  // a perspective without any valid feature may go anywhere
    for (int k = 0; k < nnz; k++) {
        const unsigned v = list[k];
        if (v < (unsigned)n_inputs) {
            b = (int)v / block_rows;
            break;
        }
    }
    blk[pair] = b;
    atomicAdd(&counts[b], 1);
}

// one CTA: exclusive scan of the histogram -> block_begin, cursors = block_begin
__global__ void group_scan_kernel(int* counts, int* begin, int nblocks) {
    __shared__ int s[kMaxBlocks + 1];
    for (int i = threadIdx.x; i < nblocks; i += blockDim.x) s[i] = counts[i];
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int i = 0; i < nblocks; i++) {
            const int c = s[i];
            s[i] = run;
            run += c;
        }
        s[nblocks] = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i <= nblocks; i += blockDim.x) {
        begin[i] = s[i];
        if (i < nblocks) counts[i] = s[i];
    }
}

__global__ void group_fill_kernel(const int* blk, int n, int* cursors, int* order) {
    const int pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= 2 * n) return;
    order[atomicAdd(&cursors[blk[pair]], 1)] = pair;
}

int check_op(const b200_ft_op* op, const char* who) {
    if (!op) return b200::fail(B200_ERR_ARG, "%s: null operator description", who);
    if (!op->table || !op->bias || !op->idx_stm || !op->idx_nstm || !op->x || (op->pairwise && !op->u))
        return b200::fail(B200_ERR_ARG, "%s: null device pointer", who);
    if (op->n < 1) return b200::fail(B200_ERR_ARG, "%s: n must be positive", who);
    if (op->n > INT32_MAX / 4) return b200::fail(B200_ERR_ARG, "%s: at most %d positions per call", who, INT32_MAX / 4);
    if (op->nnz < 1 || op->nnz > 64 || op->n_inputs < 1 || op->n_inputs > 65534)
        return b200::fail(B200_ERR_UNSUPPORTED, "%s: nnz must be in [1, 64] and n_inputs in [1, 65534]", who);
    if (op->ft_act != B200_ACT_CRELU && op->ft_act != B200_ACT_SCRELU)
        return b200::fail(B200_ERR_UNSUPPORTED, "%s: activation must be CReLU or SCReLU", who);
    if (op->pairwise && op->ft_act != B200_ACT_CRELU) return b200::fail(B200_ERR_UNSUPPORTED, "%s: pairwise needs CReLU", who);
    const int R = op->ft_block_rows;
    if (R < 1 || op->n_inputs % R || op->ft_out < 64 || op->ft_out % b200::kTileCols || op->n_inputs / R > kMaxBlocks ||
        b200::ft_fwd_smem(R, list_len(op->nnz)) > 227 * 1024)
        return b200::fail(B200_ERR_UNSUPPORTED,
                          "%s: needs ft_block_rows > 0 dividing n_inputs (at most about 800 rows, at most %d blocks) "
                          "and ft_out a multiple of 64",
                          who, kMaxBlocks);
    return 0;
}

// Groups the pairs into `scratch` and runs the tiled forward; synchronises the stream and
// reports a feature outside its block.  Allocates nothing.
int run_op(int device, cudaStream_t stream, const b200_ft_op* op, int* scratch) {
    const int n = op->n, R = op->ft_block_rows, nblocks = op->n_inputs / R;
    int* status = scratch;
    int* counts = scratch + 1;
    int* begin = counts + kMaxBlocks + 1;
    int* blk = scratch + kScratchHeader;
    int* order = blk + align_ints((size_t)2 * n);
    int* counts_per_pair = order + align_ints((size_t)2 * n);
    int* lists = counts_per_pair + align_ints((size_t)2 * n);
    // the scratch keeps whatever the previous call left: clear what must start at zero
    CK(cudaMemsetAsync(scratch, 0, (1 + kMaxBlocks + 1) * sizeof(int), stream));
    const int threads = 256, grid = (2 * n + threads - 1) / threads;
    group_count_kernel<<<grid, threads, 0, stream>>>(op->idx_stm, op->idx_nstm, n, op->nnz, op->n_inputs, R, counts, blk);
    group_scan_kernel<<<1, 256, 0, stream>>>(counts, begin, nblocks);
    group_fill_kernel<<<grid, threads, 0, stream>>>(blk, n, counts, order);
    CK(cudaGetLastError());

    b200::FtArgs a{};
    a.table = op->table;
    a.bias = op->bias;
    a.idx_stm = op->idx_stm;
    a.idx_nstm = op->idx_nstm;
    a.n = n;
    a.nnz = op->nnz;
    a.H = op->ft_out;
    a.n_inputs = op->n_inputs;
    a.act = op->ft_act;
    a.x = op->x;
    a.u = op->u;
    b200::TileArgs t{};
    t.block_rows = R;
    t.nslabs = op->ft_out / b200::kTileCols;
    t.first_block = 0;
    t.last_block = nblocks;
    t.pair_order = order;
    t.block_begin = begin;
    t.status = status;
    t.lists = reinterpret_cast<uint16_t*>(lists);
    t.list_count = counts_per_pair;
    t.list_len = list_len(op->nnz);
    t.once = 1;
    b200::ft_prepare_kernel<<<(2 * n + 7) / 8, 256, 0, stream>>>(a, t);
    CK(cudaGetLastError());
    const size_t smem = b200::ft_fwd_smem(R, t.list_len);
    // one CTA per SM, each taking an equal piece of the (block, slab, pair) work line
    int sms = 0;
    CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const int ctas = (int)std::max<long long>(1, std::min<long long>(sms, (long long)2 * n * t.nslabs / 128));
    if (op->pairwise) {
        CK(cudaFuncSetAttribute(b200::ft_forward_tiled_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        b200::ft_forward_tiled_kernel<true><<<ctas, b200::kFwdThreads, smem, stream>>>(a, t);
    } else {
        CK(cudaFuncSetAttribute(b200::ft_forward_tiled_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        b200::ft_forward_tiled_kernel<false><<<ctas, b200::kFwdThreads, smem, stream>>>(a, t);
    }
    CK(cudaGetLastError());
    int host_status = 0;
    CK(cudaMemcpyAsync(&host_status, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    CK(cudaStreamSynchronize(stream));
    if (host_status & b200::kStatusOutsideBlock)
        return b200::fail(B200_ERR_DATA, "a feature index fell outside the row block of its position (ft_block_rows=%d)", R);
    return 0;
}

}  // namespace

extern "C" {

int b200_op_ft_forward(int device, void* stream, const b200_ft_op* op) {
    if (int rc = check_op(op, "op_ft_forward")) return rc;
    CK(cudaSetDevice(device));
    int* scratch = nullptr;
    CK(cudaMalloc(&scratch, scratch_ints(op->n, op->nnz) * sizeof(int)));
    const int rc = run_op(device, static_cast<cudaStream_t>(stream), op, scratch);
    cudaFree(scratch);
    return rc;
}

// Same result as b200_op_ft_forward without touching the allocator.  It is meant for code
// that shares a GPU with a running training loop, or that runs after the process has handed
// out all of its device memory: cudaMalloc and cudaFree synchronise the whole device and
// serialise on a driver lock, so an evaluation thread that allocated per call would stall the
// trainer's streams every time, and a caller with a fixed memory budget has nothing left to
// allocate from.  Here the grouping scratch is the fixed array above and the call makes no
// cudaMalloc, cudaFree or other allocating call.
//
// The first call on each device looks up the array's device address (one
// cudaGetSymbolAddress, with that device current) and keeps it; make that first call before
// starting any stream capture on the thread.  All calls on one device share the array and it
// keeps the previous call's contents: the counters that must start at zero are cleared at
// the start of every call, and two calls whose GPU work overlaps (different streams or
// threads, same device) would overwrite each other's grouping — run them one after the other.
int b200_op_ft_forward_noalloc(int device, void* stream, const b200_ft_op* op) {
    if (int rc = check_op(op, "op_ft_forward_noalloc")) return rc;
    const int most = op->nnz <= 32 ? B200_OP_NOALLOC_MAX_POSITIONS : B200_OP_NOALLOC_MAX_POSITIONS / 2;
    if (op->n > most || scratch_ints(op->n, op->nnz) > kStaticInts)
        return b200::fail(B200_ERR_ARG,
                          "op_ft_forward_noalloc: %d positions do not fit the fixed scratch, which holds at most %d with "
                          "nnz=%d; split the batch or call b200_op_ft_forward",
                          op->n, most, op->nnz);
    constexpr int kMaxDevices = 64;
    if (device < 0 || device >= kMaxDevices)
        return b200::fail(B200_ERR_ARG, "op_ft_forward_noalloc: device %d out of range", device);
    CK(cudaSetDevice(device));
    // In host code `g_op_scratch` is only a handle for the runtime, not an address a kernel
    // could use: ask once per device, with that device current, where the array lives there.
    static std::mutex lock;
    static int* address[kMaxDevices] = {nullptr};
    int* scratch = nullptr;
    {
        std::lock_guard<std::mutex> guard(lock);
        if (!address[device]) {
            void* p = nullptr;
            CK(cudaGetSymbolAddress(&p, g_op_scratch));
            address[device] = static_cast<int*>(p);
        }
        scratch = address[device];
    }
    return run_op(device, static_cast<cudaStream_t>(stream), op, scratch);
}

}  // extern "C"
