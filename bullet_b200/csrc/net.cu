// b200_net: device state, staging slots and the fixed step schedule behind the C ABI.
//
// Replaces, for the NNUE training step only, what the reference assembles at run time from
// generated CUDA text: Function::new/prealloc/execute (crates/gpu/src/function.rs:73-280),
// the per-weight AdamW launches (crates/trainer/src/optimiser/adam.rs:217-291) and the
// batch copies of PreparedBatchHost (crates/trainer/src/run/dataloader.rs:41-61).  All
// device memory is allocated once in b200_net_create; a step only enqueues kernels.
//
// HBM layout
//   P, G, M, V   flat fp32 buffers: a 256-byte head whose first float (in G) is the summed
//                loss, then every tensor in name order (l0b, l0f, l1b, l1w, ...) except l0w,
//                which comes last; each tensor starts on a 256-byte boundary.  A
//                data-parallel host moves gradients and loss with one all-reduce of G, or
//                in parts: runs of l0w row blocks as the backward finishes them, then the
//                head (loss and all other tensors) in one piece.
//   table        l0w + tiled l0f (only with a factoriser; otherwise an alias of l0w in P)
//   x, u, dx     activations kept between forward and backward, position-major
//   slots        per staging slot one pinned host block and one device block holding the
//                packed u16 index lists, buckets, targets and the two visiting orders
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/bullet_b200.h"
#include "common.h"
#include "kernels_dense.cuh"
#include "kernels_ft.cuh"
#include "kernels_opt.cuh"
#include "kernels_prep.cuh"
#include "host_map.h"

#define CK(call)                                                                                          \
    do {                                                                                                  \
        cudaError_t e_ = (call);                                                                          \
        if (e_ != cudaSuccess)                                                                            \
            return b200::fail(B200_ERR_CUDA, "%s failed: %s (%d) at %s:%d", #call, cudaGetErrorString(e_), \
                              (int)e_, __FILE__, __LINE__);                                               \
    } while (0)

// after every kernel launch: surface a launch error, count the launch
#define LAUNCHED(net)            \
    do {                         \
        CK(cudaGetLastError());  \
        (net)->launches++;       \
    } while (0)

namespace {

constexpr int64_t kAlignFloats = 64;       // 256-byte tensor alignment in the flat buffers
constexpr int kMinItemPairs = 128;         // a forward work item serves at least this many pairs per tile load

struct Tensor {
    std::string name;
    int64_t n = 0, off = 0;
    int64_t rows = 0, cols = 0;  // column-major shape, as the reference's Shape(rows, cols)
    b200_adamw_params hp{0.01f, 0.9f, 0.999f, -1.98f, 1.98f};
    // which update rule: AdamW, RAdam, or RAdam under Ranger's lookahead (crates/trainer/src/optimiser/{radam,ranger}.rs)
    int opt_kind = B200_OPT_ADAMW;
    float n_sma_threshold = 5.0f, alpha = 0.5f;
    int lookahead_k = 6;
};

struct Slot {
    char* d_blob = nullptr;
    char* h_blob = nullptr;
    size_t capacity = 0;
    int n = 0;
    int n_dtiles = 0;  // CTA tiles of the dense kernels held in off_dtiles
    int n_chunks = 0, chunk_len = 0;  // chunks of the tiled FT backward held in off_chunks, and their size
    std::vector<int> block_begin;     // [nblocks + 1] host copy: first pair (in visiting order) of every block
    std::vector<int> chunk_begin;     // [nblocks + 1] host copy: first chunk of every block
    int expect_grid = 0;              // grid size the per-block CTA counts in off_bexpect were made for
    // device-side batch preparation (b200_batch_upload_records_gpu): raw records, scratch, totals read-back
    uint4* d_records = nullptr;
    uint16_t* d_pair_block = nullptr;
    int* d_cta_hist = nullptr;
    int* d_totals = nullptr;
    int* h_totals = nullptr;          // pinned: bin totals, bin bases, then the status word
    cudaEvent_t totals_ready = nullptr;
    // derived from the indices alone, so built once per upload on the copy stream (or on first use):
    uint16_t* lists = nullptr;        // prepared per-pair row lists of the tiled kernels
    int* list_count = nullptr;
    uint16_t* csr_ent = nullptr;      // per-chunk row-major lists of the tiled backward
    int* csr_start = nullptr;
    bool prepared = false, csr_built = false;
    size_t off_status = 0;            // one int in the blob, zero on upload: bits raised by ft_prepare_kernel
    size_t off_stm = 0, off_nstm = 0, off_buckets = 0, off_targets = 0, off_order = 0, off_pairs = 0, off_blocks = 0,
           off_dtiles = 0, off_chunks = 0, off_cbegin = 0, off_bexpect = 0, bytes = 0;
    cudaEvent_t ready = nullptr, consumed = nullptr;
    bool has_ready = false, has_consumed = false;
    template <class T>
    T* dev(size_t off) const { return reinterpret_cast<T*>(d_blob + off); }
    template <class T>
    T* host(size_t off) const { return reinterpret_cast<T*>(h_blob + off); }
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct b200_net {
    int device = 0;
    int sm_count = 1;  // cudaDevAttrMultiProcessorCount of `device`: grids are sized in waves of it
    cudaStream_t stream = nullptr, copy_stream = nullptr;
    // clears the gradient buffer beside the feature-transformer forward, which does not touch it
    cudaStream_t zero_stream = nullptr;
    cudaEvent_t zero_fork = nullptr, zero_done = nullptr;
    bool zero_pending = false;
    bool own_stream = false;
    b200_net_desc d{};
    std::vector<Tensor> tensors;
    int64_t n_flat = 0;
    float *P = nullptr, *G = nullptr, *M = nullptr, *V = nullptr, *table = nullptr;
    float *x = nullptr, *u = nullptr, *dx = nullptr, *a1 = nullptr, *a2 = nullptr, *out = nullptr, *w1g = nullptr;
    float* dz[3] = {nullptr, nullptr, nullptr};
    int wgrad_per_sm = 0;          // resident CTAs per SM of the first layer's weight-gradient kernel (looked up once)
    int status_slot = -1;          // slot whose status word the running step reports (-1: the step used no tiled kernel)
    // pinned read-back ring: loss and status word of the last kLossRing updates
    static constexpr int kLossRing = 4;
    int* h_status = nullptr;
    int* d_status = nullptr;       // [kLossRing] the slot's status word, saved before the slot is released to the uploader
    float* h_loss = nullptr;
    cudaEvent_t loss_ev[kLossRing] = {};
    int64_t updates = 0;
    Slot slots[B200_NUM_SLOTS];
    int ft_fwd_mode = B200_FT_AUTO, ft_bwd_mode = B200_FT_AUTO;
    bool bwd_wide = true;  // shape of the tiled backward (see ft_bwd_chunk)
    int exchange_bulk = 0;  // the peer exchange moves gradients and weights with bulk asynchronous copies (measured no faster)
    int bwd_grab = 0;  // rows a warp of the tiled backward takes from the row counter at a time (0: chosen by block size)
    int ft_once = 1;       // bit 0: the tiled kernels read table rows and activations with loads that claim no L1 line
    int wide_chunk = 0;    // the larger chunk of the 1024-thread backward where it fits into shared memory, else the standard one
    // Pairs per chunk for a batch of n positions.  The larger chunk saves list copies, barriers and reductions,
    // but needs enough units to keep every SM's share even: measured faster from about eight units per SM.
    int bwd_chunk(int n) const {
        if (!bwd_wide) return b200::ft_bwd_chunk(d.nnz, false);
        const long long units = (long long)nslabs * ((2LL * n + wide_chunk - 1) / wide_chunk);
        return units >= 8LL * sm_count ? wide_chunk : b200::ft_bwd_chunk(d.nnz, true);
    }
    int bwd_slot = -1, bwd_parts_done = 0, bwd_parts = 0;  // progress of a phased backward
    int fwd_slot = -1, fwd_parts_done = 0, fwd_parts = 0;  // progress of a forward pass run in pieces
    // peers of the fused data-parallel update: every rank's gradient and parameter buffer mapped here
    int xch_rank = -1, xch_world = 0;
    float* peer_g[b200::kMaxRanks] = {};
    float* peer_p[b200::kMaxRanks] = {};
    int* xch_flags = nullptr;  // this rank's fence counters (kernels_opt.cuh: PeerFlags)
    int* peer_flags[b200::kMaxRanks] = {};
    int xch_step = 0;          // fenced exchanges issued so far
    long long xch_spin_limit = b200::kPeerWaitSpins;
    int xch_wait_ready = 0;    // value the next exchange launch waits for at kFlagReady (0: the caller fences)
    bool xch_fenced_used = false;
    int* h_xstatus = nullptr;  // pinned ring beside h_status: per update the fence time-out word and what was missing
    bool loss_in_param = false;  // the last update left the summed loss in P[0] instead of G[0]
    int exchange_ctas = 0;          // CTAs of a side-stream exchange launch (0: one per SM)
    // the exchange that runs under the feature-transformer backward (b200_step_exchange)
    cudaStream_t xch_stream = nullptr;  // highest priority: its few CTAs take their SMs before the backward's many
    cudaEvent_t xch_fork = nullptr, xch_join = nullptr;
    b200::PeerFlags* d_peers = nullptr;  // device copy of the peers' counter arrays, for the backward's CTAs
    int* done_count = nullptr;           // [nblocks] backward CTAs finished per row block
    float* facc = nullptr;               // running block sum of this rank's share of the factoriser gradient
    float* d_win_rate = nullptr;         // device-side preparation: sigmoid(score / scale) for every 16-bit score
    float win_rate_scale = 0.f;          // the scale the table was made for (0: none yet)
    int* d_expanded = nullptr;           // [64] 768 * king bucket per square, and the layout it was made from
    int32_t expanded_layout[32] = {};
    bool expanded_valid = false;
    int overlap_ctas = 20;               // SMs the overlapped exchange occupies
    bool overlap_mode = false;           // batches are cut for a backward that runs beside the exchange
    bool sig_on = false;                 // the running backward announces finished row blocks
    int sig_value = 0;
    bool manual_grad_zero = false;  // the caller zeroes the gradient buffer range by range (b200_grad_zero_range)
    bool tiled_ok = false, table_dirty = true, have_backward = false;
    int nblocks = 1, nslabs = 1;
    int last_n = 0;
    // per-step CUDA events on the compute stream, kept for the last kTimingRing steps
    static constexpr int kTimingRing = 256, kTimingEvents = 8;
    cudaEvent_t tev[kTimingRing][kTimingEvents] = {};
    int64_t steps_begun = 0, steps_done = 0, timing_origin = 0;
    bool step_open = false;
    int64_t opt_step = 0;   // completed optimiser steps (RAdam's step count; reset when the rule changes)
    float* S = nullptr;     // Ranger's slow weights, same layout as P (allocated when a tensor first uses Ranger)
    int64_t launches = 0, h2d_bytes = 0;
    std::vector<void*> allocations;

    int D1() const { return d.pairwise ? d.ft_out : 2 * d.ft_out; }
    int dense_in(int l) const { return l == 0 ? D1() : d.dense_out[l - 1]; }
    Tensor* find(const char* name) {
        for (auto& t : tensors)
            if (t.name == name) return &t;
        return nullptr;
    }
    // AUTO: both passes take the shared-memory kernels whenever the inputs allow it (measured
    // at 16384 positions, H = 2048: backward 0.50 ms against 0.61 ms for global vector reductions)
    bool fwd_tiled() const { return ft_fwd_mode == B200_FT_TILED || (ft_fwd_mode == B200_FT_AUTO && tiled_ok); }
    bool bwd_tiled() const { return ft_bwd_mode == B200_FT_TILED || (ft_bwd_mode == B200_FT_AUTO && tiled_ok); }
    // the register-tiled dense forward (rows per bucket in fours, more layers after the first) also
    // forms the gradients of those later layers
    bool fused_small_grads() const { return d.dense_out[0] % 4 == 0 && d.n_dense >= 2; }
};

namespace {

// The per-tensor table of the update kernels for the step that is being enqueued.  RAdam's step size and
// its "second moment divides yet" flag depend on the step count only and are evaluated here in fp32, as
// RAdam::update does on the host (radam.rs:295-314).
void fill_segments(const b200_net* net, b200::AdamArgs& a) {
    a.nseg = (int)net->tensors.size();
    for (int i = 0; i < a.nseg; i++) {
        const Tensor& t = net->tensors[i];
        b200::AdamSegment seg{t.off / 4, (t.off + t.n + 3) / 4, t.hp.decay, t.hp.beta1, t.hp.beta2, t.hp.min_weight, t.hp.max_weight};
        if (t.opt_kind != B200_OPT_ADAMW) {
            const float step = (float)(net->opt_step + 1);
            const float beta2_t = powf(t.hp.beta2, step);
            const float n_sma_max = 2.0f / (1.0f - t.hp.beta2) - 1.0f;
            const float n_sma = n_sma_max - 2.0f * step * beta2_t / (1.0f - beta2_t);
            const float denom = 1.0f - powf(t.hp.beta1, step);
            if (n_sma > t.n_sma_threshold) {
                const float p1 = (n_sma - 4.0f) / (n_sma_max - 4.0f), p2 = (n_sma - 2.0f) / n_sma, p3 = n_sma_max / (n_sma_max - 2.0f);
                seg.rate_scale = sqrtf((1.0f - beta2_t) * p1 * p2 * p3) / denom;
                seg.use_denom = 1;
            } else {
                seg.rate_scale = 1.0f / denom;
                seg.use_denom = 0;
            }
        }
        a.seg[i] = seg;
    }
}

int set_device(const b200_net* net) {
    CK(cudaSetDevice(net->device));
    return 0;
}

template <class T>
int dev_alloc(b200_net* net, T** p, size_t count) {
    void* raw = nullptr;
    CK(cudaMalloc(&raw, std::max<size_t>(count, 1) * sizeof(T)));
    net->allocations.push_back(raw);
    *p = static_cast<T*>(raw);
    return 0;
}

bool supported_m(int m) { return m == 1 || m == 2 || m == 4 || m == 8 || m == 16 || m == 32; }

int validate(const b200_net_desc& d) {
    if (d.n_inputs < 1 || d.n_inputs > 65534) return b200::fail(B200_ERR_UNSUPPORTED, "n_inputs must be in [1, 65534]");
    if (d.nnz < 1 || d.nnz > 64) return b200::fail(B200_ERR_UNSUPPORTED, "nnz must be in [1, 64]");
    if (d.ft_out < 8 || d.ft_out % 8) return b200::fail(B200_ERR_UNSUPPORTED, "ft_out must be a positive multiple of 8");
    if (d.ft_act != B200_ACT_CRELU && d.ft_act != B200_ACT_SCRELU)
        return b200::fail(B200_ERR_UNSUPPORTED, "ft_act must be CReLU or SCReLU");
    if (d.pairwise && d.ft_act != B200_ACT_CRELU) return b200::fail(B200_ERR_UNSUPPORTED, "pairwise_mul needs CReLU");
    if (d.factoriser_rows < 0 || (d.factoriser_rows && d.n_inputs % d.factoriser_rows))
        return b200::fail(B200_ERR_ARG, "factoriser_rows must tile n_inputs");
    if (d.n_out_buckets < 1 || d.n_out_buckets > 64) return b200::fail(B200_ERR_UNSUPPORTED, "1..64 output buckets");
    if (d.n_dense < 1 || d.n_dense > 3) return b200::fail(B200_ERR_UNSUPPORTED, "one to three dense layers");
    for (int l = 0; l < d.n_dense; l++) {
        if (d.dense_out[l] < 1 || d.dense_out[l] > 32 || (l == 0 && !supported_m(d.dense_out[l])))
            return b200::fail(B200_ERR_UNSUPPORTED, "dense layer %d: rows per bucket must be 1,2,4,8,16 or 32", l + 1);
        if (d.dense_act[l] < 0 || d.dense_act[l] > 2) return b200::fail(B200_ERR_ARG, "dense layer %d: bad activation", l + 1);
    }
    for (int l = 1; l < d.n_dense; l++)
        if (!supported_m(d.dense_out[l])) return b200::fail(B200_ERR_UNSUPPORTED, "dense layer %d: rows per bucket must be a power of two <= 32", l + 1);
    if (d.dense_out[d.n_dense - 1] != 1 || d.dense_act[d.n_dense - 1] != B200_ACT_NONE)
        return b200::fail(B200_ERR_UNSUPPORTED, "the last dense layer must have one row per bucket and no activation");
    if (d.max_batch < 1) return b200::fail(B200_ERR_ARG, "max_batch must be positive");
    if (d.ft_block_rows < 0) return b200::fail(B200_ERR_ARG, "ft_block_rows must not be negative");
    return 0;
}

void slot_layout(const b200_net* net, Slot& s, int n) {
    const b200_net_desc& d = net->d;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off = align_up(off + bytes, 256);
        return at;
    };
    s.off_stm = take((size_t)n * d.nnz * 2);
    s.off_nstm = take((size_t)n * d.nnz * 2);
    s.off_buckets = take((size_t)n * 4);
    s.off_targets = take((size_t)n * 4);
    s.off_order = take((size_t)n * 4);
    s.off_pairs = take((size_t)n * 8);
    s.off_blocks = take((size_t)(net->nblocks + 1) * 4);
    s.off_dtiles = take(((size_t)n / b200::kDenseTile + d.n_out_buckets + 1) * 8);
    s.off_chunks = take(((size_t)2 * n / b200::ft_bwd_chunk(d.nnz, false) + net->nblocks + 1) * 16);
    s.off_cbegin = take((size_t)(net->nblocks + 1) * 4);
    s.off_bexpect = take((size_t)net->nblocks * 4);
    s.off_status = take(4);
    s.bytes = off;
}

template <bool PW>
int launch_ft_forward(b200_net* net, const b200::FtArgs& a, const b200::TileArgs& t, bool tiled, int grid) {
    if (tiled) {
        b200::ft_forward_tiled_kernel<PW><<<grid, b200::kFwdThreads, b200::ft_fwd_smem(t.block_rows, t.list_len), net->stream>>>(a, t);
    } else {
        const int unit = PW ? a.H / 2 : a.H;
        dim3 grid((2 * a.n + 63) / 64, (unit + 127) / 128);
        b200::ft_forward_gather_kernel<PW><<<grid, 256, 0, net->stream>>>(a, 64);
    }
    LAUNCHED(net);
    return 0;
}

template <bool PW>
int launch_ft_backward(b200_net* net, const b200::FtArgs& a, const b200::TileArgs& t, bool tiled, int grid) {
    if (tiled) {
        const size_t smem = b200::ft_bwd_smem(t.block_rows, a.nnz, t.chunk_len, t.nslabs);
        const bool wide = t.chunk_len > b200::ft_bwd_chunk(a.nnz, false);
// data-parallel runs that announce finished row blocks take an instantiation of their own: the
        // fence it ends with makes every CTA wait for its reductions to land (measured: +18 %)
        if (wide && t.sig.done_count)
            b200::ft_backward_tiled_kernel<PW, 1024, true><<<grid, 1024, smem, net->stream>>>(a, t);
        else if (wide)
            b200::ft_backward_tiled_kernel<PW, 1024, false><<<grid, 1024, smem, net->stream>>>(a, t);
        else if (t.sig.done_count)
            b200::ft_backward_tiled_kernel<PW, 512, true><<<grid, 512, smem, net->stream>>>(a, t);
        else
            b200::ft_backward_tiled_kernel<PW, 512, false><<<grid, 512, smem, net->stream>>>(a, t);
    } else {
        const int unit = PW ? a.H / 2 : a.H;
        dim3 grid((2 * a.n + 63) / 64, (unit + 127) / 128);
        b200::ft_backward_gather_kernel<PW><<<grid, 256, 0, net->stream>>>(a, 64);
    }
    LAUNCHED(net);
    return 0;
}

#define DISPATCH_M(m, ...)                                                    \
    switch (m) {                                                              \
        case 1: { constexpr int MM = 1; __VA_ARGS__; } break;                 \
        case 2: { constexpr int MM = 2; __VA_ARGS__; } break;                 \
        case 4: { constexpr int MM = 4; __VA_ARGS__; } break;                 \
        case 8: { constexpr int MM = 8; __VA_ARGS__; } break;                 \
        case 16: { constexpr int MM = 16; __VA_ARGS__; } break;               \
        case 32: { constexpr int MM = 32; __VA_ARGS__; } break;               \
        default: return b200::fail(B200_ERR_UNSUPPORTED, "rows per bucket %d", m); \
    }

// The first dense layer's forward: register-tiled when its rows per bucket come in fours and
// more layers follow, else the dot-product kernel (single-output networks).
template <int MM>
constexpr bool dense_tiled() { return MM % 4 == 0; }

template <int MM>
void launch_dense_forward(b200_net* net, const b200::DenseArgs& da, int ntiles) {
    if constexpr (dense_tiled<MM>()) {
        if (da.n_dense >= 2) {
            b200::dense_forward_tile_kernel<MM><<<ntiles, 256, b200::dense_fwd_tile_smem<MM>(), net->stream>>>(da);
            return;
        }
    }
    b200::dense_forward_kernel<MM><<<ntiles, 256, b200::dense_fwd_smem<MM>(), net->stream>>>(da);
}

template <int MM>
cudaError_t set_dense_forward_smem() {
    if constexpr (dense_tiled<MM>()) {
        cudaError_t e = cudaFuncSetAttribute(b200::dense_forward_tile_kernel<MM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)b200::dense_fwd_tile_smem<MM>());
        if (e != cudaSuccess) return e;
    }
    return cudaFuncSetAttribute(b200::dense_forward_kernel<MM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                (int)b200::dense_fwd_smem<MM>());
}

// Grid of the tiled kernels for the row blocks [first, last): one CTA per SM (two for the 512-thread
// backward), fewer when there is too little work to give every CTA a worthwhile piece.
int ft_forward_grid(const b200_net* net, const Slot& s, int first, int last) {
    const long long line = (long long)net->nslabs * (s.block_begin[last] - s.block_begin[first]);
    return (int)std::max<long long>(1, std::min<long long>(net->sm_count, line / kMinItemPairs));
}
int ft_backward_grid(const b200_net* net, const Slot& s, int first, int last, bool beside_exchange) {
    const long long units = (long long)net->nslabs * (s.chunk_begin[last] - s.chunk_begin[first]);
    const int per_sm = s.chunk_len > b200::ft_bwd_chunk(net->d.nnz, false) ? 1 : 2;
    const int sms = net->sm_count - (beside_exchange ? std::min(net->overlap_ctas, net->sm_count - 1) : 0);
    return (int)std::max<long long>(1, std::min<long long>((long long)sms * per_sm, units));
}

b200::FtArgs ft_args(b200_net* net, const Slot& s) {
    b200::FtArgs a{};
    const b200_net_desc& d = net->d;
    // the tiled forward adds the factoriser while it fills its tile; only the gather forward
    // needs the merged table
    const bool merged = net->d.factoriser_rows && !net->fwd_tiled();
    a.table = merged ? net->table : net->P + net->find("l0w")->off;
    a.factor = (net->d.factoriser_rows && !merged) ? net->P + net->find("l0f")->off : nullptr;
    a.factor_rows = net->d.factoriser_rows;
    a.bias = net->P + net->find("l0b")->off;
    a.idx_stm = s.dev<uint16_t>(s.off_stm);
    a.idx_nstm = s.dev<uint16_t>(s.off_nstm);
    a.n = s.n;
    a.nnz = d.nnz;
    a.H = d.ft_out;
    a.n_inputs = d.n_inputs;
    a.act = d.ft_act;
    a.x = net->x;
    a.u = net->u;
    a.dx = net->dx;
    a.g_table = net->G + net->find("l0w")->off;
    a.g_bias = net->G + net->find("l0b")->off;
    return a;
}

b200::TileArgs tile_args(b200_net* net, const Slot& s, bool backward) {
    b200::TileArgs t{};
    t.block_rows = net->d.ft_block_rows;
    t.nslabs = net->nslabs;
    t.first_block = 0;
    t.last_block = net->nblocks;
    t.chunk_begin = s.dev<int>(s.off_cbegin);
    t.pair_order = net->nblocks > 1 ? s.dev<int>(s.off_pairs) : nullptr;
    t.block_begin = s.dev<int>(s.off_blocks);
    t.status = s.dev<int>(s.off_status);
    t.lists = s.lists;
    t.list_count = s.list_count;
    t.list_len = (net->d.nnz + 7) & ~7;
    t.chunks = s.dev<int4>(s.off_chunks);
    t.csr_ent = s.csr_ent;
    t.csr_start = s.csr_start;
    t.chunk_len = s.chunk_len;
    t.once = net->ft_once;
    // rows per grab: measured best at eight for 768-row blocks (runs of neighbouring rows per warp, and still four
    // grabs per warp and unit to even out the list lengths), two to four for the 147-row ataxx table
    t.grab = net->bwd_grab > 0 ? net->bwd_grab : std::max(2, std::min(8, net->d.ft_block_rows / 96));
    t.ent_cap = b200::ft_bwd_ent_cap(net->d.ft_block_rows, net->d.nnz, s.chunk_len);
    t.start_cap = b200::ft_bwd_start_cap(net->d.ft_block_rows);
    if (backward && net->sig_on) {
        t.sig.done_count = net->done_count;
        t.sig.done_expect = s.dev<int>(s.off_bexpect);
        t.sig.peers = net->d_peers;
        t.sig.value = net->sig_value;
    }
    return t;
}

b200::DenseArgs dense_args(b200_net* net, const Slot& s, bool want_grad) {
    b200::DenseArgs a{};
    const b200_net_desc& d = net->d;
    a.x = net->x;
    a.buckets = s.dev<int>(s.off_buckets);
    a.targets = s.dev<float>(s.off_targets);
    a.n = s.n;
    a.K1 = net->D1();
    a.O = d.n_out_buckets;
    a.n_dense = d.n_dense;
    for (int l = 0; l < d.n_dense; l++) {
        a.M[l] = d.dense_out[l];
        a.act[l] = d.dense_act[l];
        char name[16];
        snprintf(name, sizeof name, "l%dw", l + 1);
        a.W[l] = net->P + net->find(name)->off;
        snprintf(name, sizeof name, "l%db", l + 1);
        a.B[l] = net->P + net->find(name)->off;
        a.dz[l] = net->dz[l];
    }
    a.order = s.dev<int>(s.off_order);
    a.tiles = s.dev<int2>(s.off_dtiles);
    a.ntiles = s.n_dtiles;
    a.W1g = net->w1g;
    a.a1 = net->a1;
    a.a2 = net->a2;
    a.out = net->out;
    a.loss = net->G;
    a.want_grad = want_grad ? 1 : 0;
    a.fuse_small = want_grad && net->fused_small_grads() ? 1 : 0;
    for (int l = 1; l < d.n_dense; l++) {
        char name[16];
        snprintf(name, sizeof name, "l%dw", l + 1);
        a.gW[l] = net->G + net->find(name)->off;
        snprintf(name, sizeof name, "l%db", l + 1);
        a.gB[l] = net->G + net->find(name)->off;
    }
    return a;
}

int refresh_table(b200_net* net) {
    if (!net->table_dirty) return 0;
    if (net->d.factoriser_rows && !net->fwd_tiled()) {
        const Tensor* w = net->find("l0w");
        const Tensor* f = net->find("l0f");
        const size_t n4 = (size_t)w->n / 4, block4 = (size_t)f->n / 4;
        b200::factoriser_merge_kernel<<<net->sm_count * 8, 256, 0, net->stream>>>(
            reinterpret_cast<const float4*>(net->P + w->off), reinterpret_cast<const float4*>(net->P + f->off),
            reinterpret_cast<float4*>(net->table), n4, block4);
        LAUNCHED(net);
    }
    {
        const Tensor* w1 = net->find("l1w");
        b200::dense_regroup_kernel<<<std::min<int>(net->sm_count * 4, (int)((w1->n + 255) / 256)), 256, 0, net->stream>>>(
            net->P + w1->off, net->w1g, net->D1(), net->d.n_out_buckets, net->d.dense_out[0]);
        LAUNCHED(net);
    }
    net->table_dirty = false;
    return 0;
}

int check_slot(b200_net* net, int slot, const char* who) {
    if (!net) return b200::fail(B200_ERR_ARG, "%s: null net", who);
    if (slot < 0 || slot >= B200_NUM_SLOTS) return b200::fail(B200_ERR_ARG, "%s: slot %d out of range", who, slot);
    if (net->slots[slot].n < 1 || !net->slots[slot].has_ready)
        return b200::fail(B200_ERR_STATE, "%s: slot %d holds no batch", who, slot);
    return 0;
}

// The forward pass in three pieces: the per-pair row lists, the feature-transformer items of a
// run of work items, and the dense layers.
int forward_prepare(b200_net* net, Slot& s, bool want_grad) {
    b200::FtArgs fa = ft_args(net, s);
    b200::TileArgs ta = tile_args(net, s, false);
    const bool needed = net->fwd_tiled() || (want_grad && net->bwd_tiled());
    if (needed && !s.prepared) {  // normally built at upload; here only if the kernel choice changed since
        b200::ft_prepare_kernel<<<(2 * s.n + 7) / 8, 256, 0, net->stream>>>(fa, ta);
        LAUNCHED(net);
        s.prepared = true;
    }
    if (want_grad) net->status_slot = needed ? (int)(&s - net->slots) : -1;
    if (want_grad) CK(cudaEventRecord(net->tev[net->steps_begun % b200_net::kTimingRing][0], net->stream));
    return 0;
}

int forward_ft_blocks(b200_net* net, Slot& s, int first_block, int last_block) {
    const bool tiled = net->fwd_tiled();
    b200::FtArgs fa = ft_args(net, s);
    b200::TileArgs ta = tile_args(net, s, false);
    int grid = 0;
    if (tiled) {
        if (s.block_begin[last_block] == s.block_begin[first_block]) return 0;  // no position in these blocks
        ta.first_block = first_block;
        ta.last_block = last_block;
        grid = ft_forward_grid(net, s, first_block, last_block);
    }
    return net->d.pairwise ? launch_ft_forward<true>(net, fa, ta, tiled, grid) : launch_ft_forward<false>(net, fa, ta, tiled, grid);
}

int forward_dense(b200_net* net, Slot& s, bool want_grad) {
    if (want_grad) CK(cudaEventRecord(net->tev[net->steps_begun % b200_net::kTimingRing][1], net->stream));
    if (net->zero_pending) {  // the loss and every gradient from here on land in the cleared buffer
        CK(cudaStreamWaitEvent(net->stream, net->zero_done, 0));
        net->zero_pending = false;
    }
    b200::DenseArgs da = dense_args(net, s, want_grad);
    DISPATCH_M(net->d.dense_out[0], launch_dense_forward<MM>(net, da, s.n_dtiles));
    LAUNCHED(net);
    return 0;
}

int forward_part(b200_net* net, Slot& s, bool want_grad) {
    if (int rc = forward_prepare(net, s, want_grad)) return rc;
    if (int rc = forward_ft_blocks(net, s, 0, net->nblocks)) return rc;
    return forward_dense(net, s, want_grad);
}

int launch_wgrad(b200_net* net, const Slot& s, int layer) {
    const b200_net_desc& d = net->d;
    b200::WgradArgs w{};
    w.X = layer == 0 ? net->x : (layer == 1 ? net->a1 : net->a2);
    w.dY = net->dz[layer];
    w.order = d.n_out_buckets > 1 ? s.dev<int>(s.off_order) : nullptr;
    w.buckets = s.dev<int>(s.off_buckets);
    w.n = s.n;
    w.K = net->dense_in(layer);
    w.O = d.n_out_buckets;
    char name[16];
    snprintf(name, sizeof name, "l%dw", layer + 1);
    w.gW = net->G + net->find(name)->off;
    snprintf(name, sizeof name, "l%db", layer + 1);
    w.gB = net->G + net->find(name)->off;
    const int groups = w.K / 4 + 1;  // four columns per thread, plus the bias
    const int threads = groups >= 128 ? 128 : ((groups + 31) / 32) * 32;
    const int gx = (groups + threads - 1) / threads;
    // The grid should fill the CTA slots the device offers exactly once or twice: a few CTAs
    // left over for another wave would double the kernel's time.
    if (!net->wgrad_per_sm) {
        int per_sm = 0;
        DISPATCH_M(d.dense_out[layer], cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, b200::dense_wgrad_kernel<MM>, threads, 0));
        net->wgrad_per_sm = std::max(1, per_sm);
    }
    const int slots = net->wgrad_per_sm * net->sm_count;
    const int waves = s.n >= 65536 ? 2 : 1;
    int chunks = std::max(1, std::min((s.n + 31) / 32, waves * slots / gx));
    w.chunk_len = (s.n + chunks - 1) / chunks;
    chunks = (s.n + w.chunk_len - 1) / w.chunk_len;
    dim3 grid(gx, chunks);
    DISPATCH_M(d.dense_out[layer], b200::dense_wgrad_kernel<MM><<<grid, threads, 0, net->stream>>>(w));
    LAUNCHED(net);
    return 0;
}

// Weight and bias gradients of every dense layer.  They need the forward pass and the loss
// gradient only, so they run before the feature-transformer backward: once that ends, every
// gradient outside l0w is complete as well.
int launch_dense_grads(b200_net* net, Slot& s) {
    const b200_net_desc& d = net->d;
    if (net->d.n_dense > 1 && !net->fused_small_grads()) {  // the narrow layers' weight and bias gradients, one launch
        b200::SmallGradArgs g{};
        g.order = s.dev<int>(s.off_order);
        g.tiles = s.dev<int2>(s.off_dtiles);
        g.buckets = s.dev<int>(s.off_buckets);
        g.O = d.n_out_buckets;
        g.n_layers = d.n_dense - 1;
        for (int l = 1; l < d.n_dense; l++) {
            char name[16];
            g.K[l - 1] = d.dense_out[l - 1];
            g.M[l - 1] = d.dense_out[l];
            g.X[l - 1] = l == 1 ? net->a1 : net->a2;
            g.dY[l - 1] = net->dz[l];
            snprintf(name, sizeof name, "l%dw", l + 1);
            g.gW[l - 1] = net->G + net->find(name)->off;
            snprintf(name, sizeof name, "l%db", l + 1);
            g.gB[l - 1] = net->G + net->find(name)->off;
        }
        b200::dense_small_grads_kernel<<<s.n_dtiles, 256, 0, net->stream>>>(g);
        LAUNCHED(net);
    }
    return launch_wgrad(net, s, 0);
}

// With lazy module loading (the CUDA default) a kernel's code reaches the GPU at its first launch, and
// that load can wait for running kernels to finish.  The data-parallel exchange has kernels that wait,
// bounded, for other kernels launched after them, so no kernel of this library may be loaded for the
// first time while one of those is spinning: load them all when the network is created.
template <class K>
bool load_kernel(K* kernel) {
    cudaFuncAttributes attr;
    return cudaFuncGetAttributes(&attr, reinterpret_cast<const void*>(kernel)) == cudaSuccess;
}

template <int MM>
bool load_dense_kernels() {
    bool ok = load_kernel(b200::dense_forward_kernel<MM>) && load_kernel(b200::dense_dx_kernel<MM>) && load_kernel(b200::dense_wgrad_kernel<MM>);
    if constexpr (dense_tiled<MM>()) ok = ok && load_kernel(b200::dense_forward_tile_kernel<MM>);
    return ok;
}

int preload_kernels(b200_net* net) {
    bool ok = true;
    DISPATCH_M(net->d.dense_out[0], ok = load_dense_kernels<MM>());
    for (int l = 1; l < net->d.n_dense; l++) DISPATCH_M(net->d.dense_out[l], ok = ok && load_kernel(b200::dense_wgrad_kernel<MM>));
    ok = ok && load_kernel(b200::dense_regroup_kernel) && load_kernel(b200::dense_small_grads_kernel);
    ok = ok && load_kernel(b200::ft_forward_gather_kernel<true>) && load_kernel(b200::ft_forward_gather_kernel<false>);
    ok = ok && load_kernel(b200::ft_backward_gather_kernel<true>) && load_kernel(b200::ft_backward_gather_kernel<false>);
    ok = ok && load_kernel(b200::ft_forward_tiled_kernel<true>) && load_kernel(b200::ft_forward_tiled_kernel<false>);
    ok = ok && load_kernel(b200::ft_backward_tiled_kernel<true, 1024, true>) && load_kernel(b200::ft_backward_tiled_kernel<false, 1024, true>);
    ok = ok && load_kernel(b200::ft_backward_tiled_kernel<true, 512, true>) && load_kernel(b200::ft_backward_tiled_kernel<false, 512, true>);
    ok = ok && load_kernel(b200::ft_backward_tiled_kernel<true, 1024, false>) && load_kernel(b200::ft_backward_tiled_kernel<false, 1024, false>);
    ok = ok && load_kernel(b200::ft_backward_tiled_kernel<true, 512, false>) && load_kernel(b200::ft_backward_tiled_kernel<false, 512, false>);
    ok = ok && load_kernel(b200::ft_prepare_kernel) && load_kernel(b200::ft_csr_kernel);
    ok = ok && load_kernel(b200::factoriser_merge_kernel) && load_kernel(b200::factoriser_grad_kernel);
    ok = ok && load_kernel(b200::adamw_flat_kernel) && load_kernel(b200::lookahead_kernel);
    ok = ok && load_kernel(b200::adamw_exchange_kernel<0>) && load_kernel(b200::adamw_exchange_kernel<2>);
    ok = ok && load_kernel(b200::adamw_exchange_kernel<4>) && load_kernel(b200::adamw_exchange_kernel<8>);
    ok = ok && load_kernel(b200::adamw_exchange_bulk_kernel<2, 256, 6>) && load_kernel(b200::adamw_exchange_bulk_kernel<2, 512, 3>);
    ok = ok && load_kernel(b200::adamw_exchange_bulk_kernel<2, 128, 12>) && load_kernel(b200::adamw_exchange_bulk_kernel<4, 256, 5>);
    ok = ok && load_kernel(b200::adamw_exchange_bulk_kernel<0, 256, 3>) && load_kernel(b200::adamw_exchange_bulk_kernel<0, 512, 1>);
    ok = ok && load_kernel(b200::adamw_exchange_bulk_kernel<0, 128, 6>);
    ok = ok && load_kernel(b200::adamw_exchange_overlap_kernel<0>) && load_kernel(b200::adamw_exchange_overlap_kernel<2>);
    ok = ok && load_kernel(b200::adamw_exchange_overlap_kernel<4>) && load_kernel(b200::adamw_exchange_overlap_kernel<8>);
    ok = ok && load_kernel(b200::prep_featurise_kernel) && load_kernel(b200::prep_scan_kernel) && load_kernel(b200::prep_scatter_kernel);
    ok = ok && load_kernel(b200::peer_signal_kernel) && load_kernel(b200::peer_wait_kernel) && load_kernel(b200::bucket_presignal_kernel);
    if (!ok) return b200::fail(B200_ERR_CUDA, "net_create: loading the kernels failed: %s", cudaGetErrorString(cudaGetLastError()));
    return 0;
}

}  // namespace

extern "C" {

const char* b200_last_error(void) { return b200::error_buffer(); }
int b200_version(void) { return 1; }

int b200_net_create(int device, void* stream, const b200_net_desc* desc, b200_net** out) {
    if (!desc || !out) return b200::fail(B200_ERR_ARG, "net_create: null argument");
    *out = nullptr;
    if (int rc = validate(*desc)) return rc;
    int count = 0;
    CK(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return b200::fail(B200_ERR_CUDA, "net_create: no CUDA device %d (%d visible)", device, count);
    b200_net* net = new b200_net();
    net->device = device;
    net->d = *desc;
    const b200_net_desc& d = net->d;
    auto bail = [&](int rc) {
        b200_net_destroy(net);
        return rc;
    };
    if (int rc = set_device(net)) return bail(rc);
    if (cudaDeviceGetAttribute(&net->sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || net->sm_count < 1)
        return bail(b200::fail(B200_ERR_CUDA, "net_create: cannot read the SM count of device %d", device));
    if (stream) {
        net->stream = static_cast<cudaStream_t>(stream);
    } else {
        if (cudaStreamCreateWithFlags(&net->stream, cudaStreamNonBlocking) != cudaSuccess)
            return bail(b200::fail(B200_ERR_CUDA, "net_create: cannot create a stream"));
        net->own_stream = true;
    }
    if (cudaStreamCreateWithFlags(&net->zero_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&net->zero_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&net->zero_done, cudaEventDisableTiming) != cudaSuccess)
        return bail(b200::fail(B200_ERR_CUDA, "net_create: cannot create the side stream"));
    if (cudaStreamCreateWithFlags(&net->copy_stream, cudaStreamNonBlocking) != cudaSuccess)
        return bail(b200::fail(B200_ERR_CUDA, "net_create: cannot create the copy stream"));
    {
        int least = 0, greatest = 0;
        cudaDeviceGetStreamPriorityRange(&least, &greatest);
        if (cudaStreamCreateWithPriority(&net->xch_stream, cudaStreamNonBlocking, greatest) != cudaSuccess ||
            cudaEventCreateWithFlags(&net->xch_fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&net->xch_join, cudaEventDisableTiming) != cudaSuccess)
            return bail(b200::fail(B200_ERR_CUDA, "net_create: cannot create the exchange stream"));
    }

    // flat layout, tensors in name order
    auto add = [&](const char* name, int64_t rows, int64_t cols) {
        Tensor t;
        t.name = name;
        t.rows = rows;
        t.cols = cols;
        t.n = rows * cols;
        net->tensors.push_back(t);
    };
    add("l0b", d.ft_out, 1);
    if (d.factoriser_rows) add("l0f", d.ft_out, d.factoriser_rows);
    for (int l = 0; l < d.n_dense; l++) {
        char name[16];
        const int64_t rows = (int64_t)d.n_out_buckets * d.dense_out[l];
        snprintf(name, sizeof name, "l%db", l + 1);
        add(name, rows, 1);
        snprintf(name, sizeof name, "l%dw", l + 1);
        add(name, rows, net->dense_in(l));
    }
    add("l0w", d.ft_out, d.n_inputs);  // last, so that everything else is one contiguous head
    int64_t off = kAlignFloats;                  // float 0 of G is the loss
    for (auto& t : net->tensors) {
        t.off = off;
        off += (t.n + kAlignFloats - 1) / kAlignFloats * kAlignFloats;
    }
    net->n_flat = (off + 1023) / 1024 * 1024;  // a multiple of 4 floats x 256: splits evenly over up to 256 ranks

    constexpr size_t kMaxSmem = 227 * 1024;
    net->tiled_ok = d.ft_block_rows > 0 && d.n_inputs % d.ft_block_rows == 0 && d.ft_out % b200::kTileCols == 0 &&
                    b200::ft_fwd_smem(d.ft_block_rows, (d.nnz + 7) & ~7) <= kMaxSmem &&
                    b200::ft_bwd_smem(d.ft_block_rows, d.nnz, b200::ft_bwd_chunk(d.nnz, true), d.ft_out / b200::kTileCols) <= kMaxSmem;
    if (net->tiled_ok) {
        const int larger = b200::ft_bwd_chunk_large(d.nnz);
        net->wide_chunk = b200::ft_bwd_smem(d.ft_block_rows, d.nnz, larger, d.ft_out / b200::kTileCols) <= kMaxSmem ? larger : b200::ft_bwd_chunk(d.nnz, true);
    }
    net->nblocks = net->tiled_ok ? d.n_inputs / d.ft_block_rows : 1;
    net->nslabs = d.ft_out / b200::kTileCols;

    const size_t B = d.max_batch;
    int rc = 0;
    rc = rc ? rc : dev_alloc(net, &net->P, net->n_flat);
    rc = rc ? rc : dev_alloc(net, &net->G, net->n_flat);
    rc = rc ? rc : dev_alloc(net, &net->M, net->n_flat);
    rc = rc ? rc : dev_alloc(net, &net->V, net->n_flat);
    if (d.factoriser_rows) rc = rc ? rc : dev_alloc(net, &net->table, (size_t)d.n_inputs * d.ft_out);
    rc = rc ? rc : dev_alloc(net, &net->x, B * net->D1());
    if (d.pairwise) rc = rc ? rc : dev_alloc(net, &net->u, B * 2 * d.ft_out);
    rc = rc ? rc : dev_alloc(net, &net->dx, B * net->D1());
    rc = rc ? rc : dev_alloc(net, &net->a1, B * d.dense_out[0]);
    rc = rc ? rc : dev_alloc(net, &net->a2, B * 32);
    for (int l = 0; l < 3; l++) rc = rc ? rc : dev_alloc(net, &net->dz[l], B * 32);
    rc = rc ? rc : dev_alloc(net, &net->out, B);
    rc = rc ? rc : dev_alloc(net, &net->d_status, b200_net::kLossRing);
    rc = rc ? rc : dev_alloc(net, &net->w1g, (size_t)d.n_out_buckets * d.dense_out[0] * net->D1());
    // the fence counters get an allocation of their own size class (2 MiB), so that its IPC handle maps exactly it
    rc = rc ? rc : dev_alloc(net, &net->xch_flags, (size_t)(2 << 20) / sizeof(int));
    if (!rc) cudaMemsetAsync(net->xch_flags, 0, (size_t)2 << 20, net->stream);
    rc = rc ? rc : dev_alloc(net, &net->d_peers, 1);
    rc = rc ? rc : dev_alloc(net, &net->done_count, (size_t)net->nblocks);
    if (!rc) cudaMemsetAsync(net->done_count, 0, (size_t)net->nblocks * sizeof(int), net->stream);
    if (net->tiled_ok && d.factoriser_rows == d.ft_block_rows)
        rc = rc ? rc : dev_alloc(net, &net->facc, (size_t)d.ft_block_rows * d.ft_out / 2);
    if (net->tiled_ok) {
        // sized for whichever backward shape needs more: every block may end in a partly filled chunk
        size_t ent_total = 0, max_chunks = 0;
        for (int shape = 0; shape < 3; shape++) {
            const int cp = shape == 2 ? net->wide_chunk : b200::ft_bwd_chunk(d.nnz, shape != 0);
            const size_t chunks = 2 * B / cp + net->nblocks + 1;
            max_chunks = std::max(max_chunks, chunks);
            ent_total = std::max(ent_total, chunks * b200::ft_bwd_ent_cap(d.ft_block_rows, d.nnz, cp));
        }
        for (auto& s : net->slots) {
            rc = rc ? rc : dev_alloc(net, &s.lists, 2 * B * ((d.nnz + 7) & ~7));
            rc = rc ? rc : dev_alloc(net, &s.list_count, 2 * B);
            rc = rc ? rc : dev_alloc(net, &s.csr_ent, ent_total);
            rc = rc ? rc : dev_alloc(net, &s.csr_start, max_chunks * b200::ft_bwd_start_cap(d.ft_block_rows));
        }
    }
    if (rc) return bail(rc);
    if (!d.factoriser_rows) net->table = net->P + net->find("l0w")->off;
    cudaMemsetAsync(net->P, 0, net->n_flat * 4, net->stream);
    cudaMemsetAsync(net->G, 0, net->n_flat * 4, net->stream);
    cudaMemsetAsync(net->M, 0, net->n_flat * 4, net->stream);
    cudaMemsetAsync(net->V, 0, net->n_flat * 4, net->stream);

    for (auto& s : net->slots) {
        slot_layout(net, s, d.max_batch);
        s.capacity = s.bytes;
        void* raw = nullptr;
        if (cudaMalloc(&raw, s.capacity) != cudaSuccess) return bail(b200::fail(B200_ERR_CUDA, "net_create: slot allocation failed"));
        s.d_blob = static_cast<char*>(raw);
        if (cudaHostAlloc(&raw, s.capacity, cudaHostAllocDefault) != cudaSuccess)
            return bail(b200::fail(B200_ERR_CUDA, "net_create: pinned slot allocation failed"));
        s.h_blob = static_cast<char*>(raw);
        cudaEventCreateWithFlags(&s.ready, cudaEventDisableTiming);
        cudaEventCreateWithFlags(&s.consumed, cudaEventDisableTiming);
        s.n = 0;
    }
    void* raw = nullptr;
    if (cudaHostAlloc(&raw, 128, cudaHostAllocDefault) != cudaSuccess) return bail(b200::fail(B200_ERR_CUDA, "net_create: pinned alloc failed"));
    net->h_loss = static_cast<float*>(raw);
    net->h_status = reinterpret_cast<int*>(net->h_loss + 8);
    net->h_xstatus = net->h_status + b200_net::kLossRing;
    memset(net->h_loss, 0, 128);  // 8 floats, 4 status words, 4 x 4 fence words
    for (auto& e : net->loss_ev) cudaEventCreateWithFlags(&e, cudaEventDisableTiming);
    for (auto& ring : net->tev)
        for (auto& e : ring) cudaEventCreate(&e);

    {
        constexpr int MM_unused = 0;
        (void)MM_unused;
        auto set_dense = [&](int m) -> int {
            cudaError_t e = cudaSuccess;
            DISPATCH_M(m, e = set_dense_forward_smem<MM>());
            if (e != cudaSuccess) return b200::fail(B200_ERR_CUDA, "dense forward shared memory: %s", cudaGetErrorString(e));
            return 0;
        };
        if (int rc2 = set_dense(d.dense_out[0])) return bail(rc2);
    }
    if (net->tiled_ok) {
        const int fs = (int)b200::ft_fwd_smem(d.ft_block_rows, (d.nnz + 7) & ~7);
        const int wide = net->wide_chunk, narrow = b200::ft_bwd_chunk(d.nnz, false);
        const int bs = (int)b200::ft_bwd_smem(d.ft_block_rows, d.nnz, wide, net->nslabs), bn = (int)b200::ft_bwd_smem(d.ft_block_rows, d.nnz, narrow, net->nslabs);
        cudaFuncSetAttribute(b200::ft_forward_tiled_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, fs);
        cudaFuncSetAttribute(b200::ft_forward_tiled_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, fs);
        cudaFuncSetAttribute(b200::ft_backward_tiled_kernel<true, 1024, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bs);
        cudaFuncSetAttribute(b200::ft_backward_tiled_kernel<false, 1024, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bs);
        cudaFuncSetAttribute(b200::ft_backward_tiled_kernel<true, 512, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bn);
        cudaFuncSetAttribute(b200::ft_backward_tiled_kernel<false, 512, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bn);
        cudaFuncSetAttribute(b200::ft_backward_tiled_kernel<true, 1024, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bs);
        cudaFuncSetAttribute(b200::ft_backward_tiled_kernel<false, 1024, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bs);
        cudaFuncSetAttribute(b200::ft_backward_tiled_kernel<true, 512, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bn);
        cudaFuncSetAttribute(b200::ft_backward_tiled_kernel<false, 512, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bn);
        cudaFuncSetAttribute(b200::ft_csr_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)b200::ft_csr_smem(d.ft_block_rows, d.nnz, wide));
    }
    cudaFuncSetAttribute(b200::adamw_exchange_overlap_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, b200::kOverlapSmem);
    cudaFuncSetAttribute(b200::adamw_exchange_overlap_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, b200::kOverlapSmem);
    cudaFuncSetAttribute(b200::adamw_exchange_overlap_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, b200::kOverlapSmem);
    cudaFuncSetAttribute(b200::adamw_exchange_overlap_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, b200::kOverlapSmem);
    if (int rc2 = preload_kernels(net)) return bail(rc2);
    CK(cudaStreamSynchronize(net->stream));
    CK(cudaGetLastError());
    *out = net;
    return 0;
}

int b200_net_destroy(b200_net* net) {
    if (!net) return 0;
    cudaSetDevice(net->device);
    if (net->stream) cudaStreamSynchronize(net->stream);
    if (net->copy_stream) cudaStreamSynchronize(net->copy_stream);
    if (net->zero_stream) cudaStreamSynchronize(net->zero_stream);
    if (net->xch_stream) cudaStreamSynchronize(net->xch_stream);
    for (int r = 0; r < net->xch_world; r++)
        if (r != net->xch_rank) {
            if (net->peer_g[r]) cudaIpcCloseMemHandle(net->peer_g[r]);
            if (net->peer_p[r]) cudaIpcCloseMemHandle(net->peer_p[r]);
            if (net->peer_flags[r]) cudaIpcCloseMemHandle(net->peer_flags[r]);
        }
    for (void* p : net->allocations) cudaFree(p);
    for (auto& s : net->slots) {
        if (s.d_blob) cudaFree(s.d_blob);
        if (s.h_blob) cudaFreeHost(s.h_blob);
        if (s.d_records) cudaFree(s.d_records);
        if (s.d_pair_block) cudaFree(s.d_pair_block);
        if (s.d_cta_hist) cudaFree(s.d_cta_hist);
        if (s.d_totals) cudaFree(s.d_totals);
        if (s.h_totals) cudaFreeHost(s.h_totals);
        if (s.totals_ready) cudaEventDestroy(s.totals_ready);
        if (s.ready) cudaEventDestroy(s.ready);
        if (s.consumed) cudaEventDestroy(s.consumed);
    }
    if (net->h_loss) cudaFreeHost(net->h_loss);
    for (auto& e : net->loss_ev)
        if (e) cudaEventDestroy(e);
    for (auto& ring : net->tev)
        for (auto& e : ring)
            if (e) cudaEventDestroy(e);
    if (net->own_stream && net->stream) cudaStreamDestroy(net->stream);
    if (net->copy_stream) cudaStreamDestroy(net->copy_stream);
    if (net->zero_stream) cudaStreamDestroy(net->zero_stream);
    if (net->xch_stream) cudaStreamDestroy(net->xch_stream);
    if (net->xch_fork) cudaEventDestroy(net->xch_fork);
    if (net->xch_join) cudaEventDestroy(net->xch_join);
    if (net->zero_fork) cudaEventDestroy(net->zero_fork);
    if (net->zero_done) cudaEventDestroy(net->zero_done);
    delete net;
    return 0;
}

int b200_net_set_option(b200_net* net, const char* key, int64_t value) {
    if (!net || !key) return b200::fail(B200_ERR_ARG, "set_option: null argument");
    if (!strcmp(key, "ft_mode") || !strcmp(key, "ft_fwd_mode") || !strcmp(key, "ft_bwd_mode")) {
        if (value < B200_FT_AUTO || value > B200_FT_TILED) return b200::fail(B200_ERR_ARG, "ft_mode %lld unknown", (long long)value);
        if (value == B200_FT_TILED && !net->tiled_ok)
            return b200::fail(B200_ERR_UNSUPPORTED,
                              "tiled feature-transformer kernels need ft_block_rows > 0 dividing n_inputs, at most "
                              "about 800 rows per block, and ft_out a multiple of 64");
        if (strcmp(key, "ft_bwd_mode")) net->ft_fwd_mode = (int)value;
        net->table_dirty = true;  // the gather forward reads the merged table, the tiled one does not keep it fresh
        if (strcmp(key, "ft_fwd_mode")) net->ft_bwd_mode = (int)value;
        return 0;
    }
    if (!strcmp(key, "exchange_wait_ms")) {  // how long a fence of the peer exchange polls before it gives up
        net->xch_spin_limit = std::max<int64_t>(1, value) * 5000;
        return 0;
    }
    if (!strcmp(key, "exchange_ctas")) {
        net->exchange_ctas = (int)std::max<int64_t>(0, value);
        return 0;
    }
    if (!strcmp(key, "overlap_ctas")) {  // SMs that b200_step_exchange takes away from the backward for the exchange
        if (value < 1 || value >= net->sm_count) return b200::fail(B200_ERR_ARG, "overlap_ctas must be in [1, %d)", net->sm_count);
        net->overlap_ctas = (int)value;
        return 0;
    }
    if (!strcmp(key, "overlap_mode")) {  // takes effect for batches uploaded afterwards
        net->overlap_mode = value != 0;
        return 0;
    }
    if (!strcmp(key, "exchange_step")) {
        // After a step that reported B200_ERR_STATE the ranks' step counters may differ.  Every rank, with nothing
        // in flight and after a host-side barrier, sets the same value, larger than any count reached so far;
        // the call also clears this rank's timeout word.
        if (value < net->xch_step) return b200::fail(B200_ERR_ARG, "exchange_step must not go back (now %d)", net->xch_step);
        if (int rc = set_device(net)) return rc;
        CK(cudaStreamSynchronize(net->stream));
        CK(cudaStreamSynchronize(net->xch_stream));
        CK(cudaMemset(net->xch_flags + b200::kFlagTimeout, 0, 4 * sizeof(int)));
        CK(cudaMemset(net->done_count, 0, (size_t)net->nblocks * sizeof(int)));
        net->xch_step = (int)value;
        return 0;
    }
    if (!strcmp(key, "manual_grad_zero")) {
        net->manual_grad_zero = value != 0;
        return 0;
    }
    if (!strcmp(key, "exchange_bulk")) {  // 0: the exchange kernel fetches peer gradients with per-thread loads
        net->exchange_bulk = (int)value;
        return 0;
    }
    if (!strcmp(key, "ft_bwd_grab")) {
        if (value < 0 || value > 64) return b200::fail(B200_ERR_ARG, "ft_bwd_grab must be in [0, 64]");
        net->bwd_grab = (int)value;
        return 0;
    }
    if (!strcmp(key, "ft_once")) {
        net->ft_once = (int)value;
        return 0;
    }
    if (!strcmp(key, "ft_bwd_wide")) {  // takes effect for batches uploaded afterwards
        net->bwd_wide = value != 0;
        return 0;
    }
    return b200::fail(B200_ERR_ARG, "set_option: unknown key '%s'", key);
}

int b200_net_tensor_size(b200_net* net, const char* name, int64_t* n) {
    if (!net || !name || !n) return b200::fail(B200_ERR_ARG, "tensor_size: null argument");
    const Tensor* t = net->find(name);
    if (!t) return b200::fail(B200_ERR_ARG, "no tensor named '%s' in this network", name);
    *n = t->n;
    return 0;
}

int b200_net_tensor_offset(b200_net* net, const char* name, int64_t* first_float) {
    if (!net || !name || !first_float) return b200::fail(B200_ERR_ARG, "tensor_offset: null argument");
    const Tensor* t = net->find(name);
    if (!t) return b200::fail(B200_ERR_ARG, "no tensor named '%s' in this network", name);
    *first_float = t->off;
    return 0;
}

int b200_net_tensor_shape(b200_net* net, const char* name, int64_t* rows, int64_t* cols) {
    if (!net || !name || !rows || !cols) return b200::fail(B200_ERR_ARG, "tensor_shape: null argument");
    const Tensor* t = net->find(name);
    if (!t) return b200::fail(B200_ERR_ARG, "no tensor named '%s' in this network", name);
    *rows = t->rows;
    *cols = t->cols;
    return 0;
}

static float* kind_base(b200_net* net, int kind) {
    switch (kind) {
        case B200_KIND_WEIGHT: return net->P;
        case B200_KIND_MOMENTUM: return net->M;
        case B200_KIND_VELOCITY: return net->V;
        case B200_KIND_GRAD: return net->G;
        case B200_KIND_SLOW: return net->S;
        default: return nullptr;
    }
}

int b200_net_set_tensor(b200_net* net, const char* name, int kind, const float* host, int64_t n) {
    if (!net || !name || !host) return b200::fail(B200_ERR_ARG, "set_tensor: null argument");
    const Tensor* t = net->find(name);
    if (!t) return b200::fail(B200_ERR_ARG, "no tensor named '%s' in this network", name);
    if (n != t->n) return b200::fail(B200_ERR_ARG, "tensor '%s' holds %lld values, %lld given", name, (long long)t->n, (long long)n);
    if ((kind < B200_KIND_WEIGHT || kind > B200_KIND_VELOCITY) && kind != B200_KIND_SLOW)
        return b200::fail(B200_ERR_ARG, "set_tensor: kind %d is not writable", kind);
    if (kind == B200_KIND_SLOW && !net->S) return b200::fail(B200_ERR_STATE, "set_tensor: no tensor of this network uses Ranger");
    if (int rc = set_device(net)) return rc;
    CK(cudaStreamSynchronize(net->stream));
    CK(cudaMemcpy(kind_base(net, kind) + t->off, host, n * sizeof(float), cudaMemcpyHostToDevice));
    if (kind == B200_KIND_WEIGHT) net->table_dirty = true;
    return 0;
}

int b200_net_get_tensor(b200_net* net, const char* name, int kind, float* host, int64_t n) {
    if (!net || !name || !host) return b200::fail(B200_ERR_ARG, "get_tensor: null argument");
    const Tensor* t = net->find(name);
    if (!t) return b200::fail(B200_ERR_ARG, "no tensor named '%s' in this network", name);
    if (n != t->n) return b200::fail(B200_ERR_ARG, "tensor '%s' holds %lld values, %lld asked", name, (long long)t->n, (long long)n);
    float* base = kind_base(net, kind);
    if (!base) return b200::fail(B200_ERR_ARG, "get_tensor: unknown kind %d (or no tensor uses Ranger's slow weights)", kind);
    if (int rc = set_device(net)) return rc;
    CK(cudaStreamSynchronize(net->stream));
    CK(cudaMemcpy(host, base + t->off, n * sizeof(float), cudaMemcpyDeviceToHost));
    return 0;
}

int b200_net_set_adamw(b200_net* net, const char* name, const b200_adamw_params* params) {
    if (!net || !params) return b200::fail(B200_ERR_ARG, "set_adamw: null argument");
    if (!(params->min_weight <= params->max_weight)) return b200::fail(B200_ERR_ARG, "set_adamw: min_weight > max_weight");
    if (!name) {
        for (auto& t : net->tensors) t.hp = *params, t.opt_kind = B200_OPT_ADAMW;
        return 0;
    }
    Tensor* t = net->find(name);
    if (!t) return b200::fail(B200_ERR_ARG, "no tensor named '%s' in this network", name);
    t->hp = *params;
    t->opt_kind = B200_OPT_ADAMW;
    return 0;
}

int b200_net_set_optimiser(b200_net* net, const char* name, const b200_optimiser_params* params) {
    if (!net || !params) return b200::fail(B200_ERR_ARG, "set_optimiser: null argument");
    if (params->kind < B200_OPT_ADAMW || params->kind > B200_OPT_RANGER) return b200::fail(B200_ERR_ARG, "set_optimiser: unknown kind %d", params->kind);
    if (!(params->min_weight <= params->max_weight)) return b200::fail(B200_ERR_ARG, "set_optimiser: min_weight > max_weight");
    if (params->kind == B200_OPT_RANGER && (params->k < 1 || !(params->alpha >= 0.f && params->alpha <= 1.f)))
        return b200::fail(B200_ERR_ARG, "set_optimiser: Ranger needs k >= 1 and alpha in [0, 1]");
    Tensor* only = nullptr;
    if (name && !(only = net->find(name))) return b200::fail(B200_ERR_ARG, "no tensor named '%s' in this network", name);
    if (int rc = set_device(net)) return rc;
    if (params->kind == B200_OPT_RANGER && !net->S) {  // slow weights start at zero, as in the reference (ranger.rs:70)
        if (int rc = dev_alloc(net, &net->S, (size_t)net->n_flat)) return rc;
        CK(cudaMemset(net->S, 0, (size_t)net->n_flat * sizeof(float)));
    }
    for (auto& t : net->tensors) {
        if (only && &t != only) continue;
        t.hp = {params->decay, params->beta1, params->beta2, params->min_weight, params->max_weight};
        t.opt_kind = params->kind;
        t.n_sma_threshold = params->n_sma_threshold;
        t.alpha = params->alpha;
        t.lookahead_k = params->k;
    }
    net->opt_step = 0;  // OptimiserState::set_params of the lookahead resets its step (ranger.rs:107-113)
    return 0;
}

// Common start of both uploads: the slot's pinned block is free once its last copy has landed and
// the last step that read the device block has finished.
static int upload_begin(b200_net* net, int slot, int32_t n, const char* who) {
    if (slot < 0 || slot >= B200_NUM_SLOTS) return b200::fail(B200_ERR_ARG, "%s: slot %d out of range", who, slot);
    if (n < 1 || n > net->d.max_batch) return b200::fail(B200_ERR_ARG, "%s: %d positions, capacity is %d", who, n, net->d.max_batch);
    if (int rc = set_device(net)) return rc;
    Slot& s = net->slots[slot];
    if (s.has_ready) CK(cudaEventSynchronize(s.ready));
    if (s.has_consumed) CK(cudaEventSynchronize(s.consumed));
    slot_layout(net, s, n);
    s.n = 0;
    return 0;
}

static int upload_finish(b200_net* net, Slot& s, int32_t n);

int b200_batch_upload(b200_net* net, int slot, const int32_t* stm, const int32_t* nstm, const int32_t* buckets,
                      const float* targets, int32_t n) {
    if (!net || !stm || !nstm || !targets) return b200::fail(B200_ERR_ARG, "batch_upload: null argument");
    const b200_net_desc& d = net->d;
    if (d.n_out_buckets > 1 && !buckets) return b200::fail(B200_ERR_ARG, "batch_upload: this network needs output buckets");
    if (int rc = upload_begin(net, slot, n, "batch_upload")) return rc;
    Slot& s = net->slots[slot];
    const int64_t count = (int64_t)n * d.nnz;
    uint16_t* h_stm = s.host<uint16_t>(s.off_stm);
    uint16_t* h_nstm = s.host<uint16_t>(s.off_nstm);
    const uint32_t limit = (uint32_t)d.n_inputs;
#pragma omp parallel for schedule(static) if (count > 200000)
    for (int64_t i = 0; i < count; i++) {
        const uint32_t a = (uint32_t)stm[i], b = (uint32_t)nstm[i];
        h_stm[i] = a < limit ? (uint16_t)a : (uint16_t)0xFFFFu;
        h_nstm[i] = b < limit ? (uint16_t)b : (uint16_t)0xFFFFu;
    }
    int* h_buckets = s.host<int>(s.off_buckets);
    const int O = d.n_out_buckets;
    if (buckets) {
        for (int i = 0; i < n; i++) {
            if ((unsigned)buckets[i] >= (unsigned)O)
                return b200::fail(B200_ERR_DATA, "batch_upload: position %d has output bucket %d, network has %d", i, buckets[i], O);
            h_buckets[i] = buckets[i];
        }
    } else {
        memset(h_buckets, 0, (size_t)n * 4);
    }
    memcpy(s.host<float>(s.off_targets), targets, (size_t)n * 4);
    return upload_finish(net, s, n);
}

// Records in, batch on the device: the featuriser, the output bucket and the target blend of
// ValueTrainerState::make_mapper (crates/bullet_lib/src/value.rs:77-117) write straight into the
// pinned staging block as packed u16 lists; no int32 arrays in between.
int b200_batch_upload_records(b200_net* net, int slot, const void* records, int32_t n, int32_t game, const int32_t* layout32,
                              float scale, float blend) {
    if (!net || !records) return b200::fail(B200_ERR_ARG, "batch_upload_records: null argument");
    if (game < B200_GAME_CHESS768 || game > B200_GAME_ATAXX147) return b200::fail(B200_ERR_ARG, "batch_upload_records: unknown game %d", game);
    if (game == B200_GAME_CHESS_BUCKETS_MIRRORED && !layout32) return b200::fail(B200_ERR_ARG, "batch_upload_records: the king-bucket layout is missing");
    if (!(blend >= 0.f && blend <= 1.f) || !(scale > 0.f)) return b200::fail(B200_ERR_ARG, "batch_upload_records: bad scale or blend");
    const b200_net_desc& d = net->d;
    const int O = d.n_out_buckets;
    if (O > 1 && game == B200_GAME_ATAXX147) return b200::fail(B200_ERR_UNSUPPORTED, "batch_upload_records: no output buckets for ataxx records");
    if (int rc = upload_begin(net, slot, n, "batch_upload_records")) return rc;
    Slot& s = net->slots[slot];
    uint16_t* h_stm = s.host<uint16_t>(s.off_stm);
    uint16_t* h_nstm = s.host<uint16_t>(s.off_nstm);
    int* h_buckets = s.host<int>(s.off_buckets);
    float* h_targets = s.host<float>(s.off_targets);
    int32_t expanded[64] = {0};
    if (game == B200_GAME_CHESS_BUCKETS_MIRRORED) b200::expand_king_buckets(layout32, expanded);
    const b200::ChessRecord* chess = static_cast<const b200::ChessRecord*>(records);
    const b200::AtaxxRecord* ataxx = static_cast<const b200::AtaxxRecord*>(records);
    const int nnz = d.nnz;
    const uint32_t limit = (uint32_t)d.n_inputs;
    const float rscale = 1.0f / scale;
    int bad = n, bad_bucket = n;
#pragma omp parallel for schedule(static) reduction(min : bad) reduction(min : bad_bucket) if (n >= 4096)
    for (int32_t i = 0; i < n; i++) {
        uint16_t* a = h_stm + (size_t)i * nnz;
        uint16_t* b = h_nstm + (size_t)i * nnz;
        int count;
        if (game == B200_GAME_CHESS768)
            count = b200::map_chess_record<false, uint16_t>(chess[i], expanded, a, b, nnz, (uint16_t)0xFFFFu);
        else if (game == B200_GAME_CHESS_BUCKETS_MIRRORED)
            count = b200::map_chess_record<true, uint16_t>(chess[i], expanded, a, b, nnz, (uint16_t)0xFFFFu);
        else
            count = b200::map_ataxx_record<uint16_t>(ataxx[i], a, b, nnz, (uint16_t)0xFFFFu);
        if (count < 0) {
            bad = i < bad ? i : bad;
            continue;
        }
        for (int k = 0; k < count; k++) {  // as b200_batch_upload: an index the table does not have is an empty slot
            if (a[k] >= limit) a[k] = 0xFFFFu;
            if (b[k] >= limit) b[k] = 0xFFFFu;
        }
        int bucket = 0;
        if (O > 1) {
            bucket = b200::material_bucket(chess[i].occ, O);
            if ((unsigned)bucket >= (unsigned)O) bad_bucket = i < bad_bucket ? i : bad_bucket;
        }
        h_buckets[i] = bucket;
        h_targets[i] = b200::blended_target(chess[i].score, chess[i].result, rscale, blend);  // same offsets in both record types
    }
    if (bad < n) return b200::fail(B200_ERR_DATA, "batch_upload_records: record %d holds more than nnz=%d pieces", bad, nnz);
    if (bad_bucket < n) return b200::fail(B200_ERR_DATA, "batch_upload_records: record %d has no valid output bucket", bad_bucket);
    return upload_finish(net, s, n);
}

// Everything the kernels need beyond the batch itself, from two histograms: how many positions take each
// output bucket and how many (position, perspective) pairs fall into each table row block.  Fills, in the
// slot's pinned block: the dense kernels' tiles, the blocks' first pairs, the backward's chunks, their
// first chunk per block and the per-block CTA counts of a whole-batch backward launch.
static void derive_tables(b200_net* net, Slot& s, const int* bucket_count, const int* block_count) {
    const b200_net_desc& d = net->d;
    const int O = d.n_out_buckets, nb = net->nblocks;
    {   // CTA tiles of the dense kernels: runs of up to kDenseTile positions of one bucket
        int2* h_tiles = s.host<int2>(s.off_dtiles);
        int nt = 0, at = 0;
        for (int k = 0; k < O; k++) {
            const int end = at + bucket_count[k];
            for (; at < end; at += b200::kDenseTile) h_tiles[nt++] = make_int2(at, std::min(b200::kDenseTile, end - at));
            at = end;
        }
        s.n_dtiles = nt;
    }
    int* h_blocks = s.host<int>(s.off_blocks);
    h_blocks[0] = 0;
    for (int b = 0; b < nb; b++) h_blocks[b + 1] = h_blocks[b] + block_count[b];
    s.block_begin.assign(h_blocks, h_blocks + nb + 1);
    if (net->tiled_ok) {
        // chunks of the tiled backward: every block cut into the fewest equal runs of at most ft_bwd_chunk pairs
        int4* h_chunks = s.host<int4>(s.off_chunks);
        int* h_cbegin = s.host<int>(s.off_cbegin);
        const int cp = net->bwd_chunk(h_blocks[nb] / 2);  // (all pairs of the batch = two per position)
        s.chunk_len = cp;
        int nc = 0;
        for (int b = 0; b < nb; b++) {
            h_cbegin[b] = nc;
            const int pairs = h_blocks[b + 1] - h_blocks[b], pieces = (pairs + cp - 1) / cp;
            const int size = pieces ? (pairs + pieces - 1) / pieces : 0;
            for (int at = h_blocks[b]; at < h_blocks[b + 1]; at += size) h_chunks[nc++] = make_int4(b, at, std::min(size, h_blocks[b + 1] - at), 0);
        }
        h_cbegin[nb] = nc;
        s.n_chunks = nc;
        s.chunk_begin.assign(h_cbegin, h_cbegin + nb + 1);
        // How many CTAs of a whole-batch backward launch work on each block, for the data-parallel runs that
        // announce finished blocks: there CTA k takes the units k, k + grid, ... of the block-ordered numbering.
        int* h_expect = s.host<int>(s.off_bexpect);
        const int grid = ft_backward_grid(net, s, 0, nb, net->overlap_mode);
        s.expect_grid = grid;
        for (int blk = 0; blk < nb; blk++) h_expect[blk] = std::min(grid, net->nslabs * (h_cbegin[blk + 1] - h_cbegin[blk]));
    }
    *s.host<int>(s.off_status) = 0;
}

// The row lists of the tiled kernels depend on the indices only: build them right behind the copy, on
// the copy stream, where they run beside the step that is still computing; then mark the slot ready.
static int upload_launch_lists(b200_net* net, Slot& s, int32_t n) {
    const b200_net_desc& d = net->d;
    s.prepared = s.csr_built = false;
    s.n = n;
    if (net->tiled_ok && (net->fwd_tiled() || net->bwd_tiled())) {
        b200::FtArgs fa = ft_args(net, s);
        b200::TileArgs ta = tile_args(net, s, true);
        b200::ft_prepare_kernel<<<(2 * n + 7) / 8, 256, 0, net->copy_stream>>>(fa, ta);
        LAUNCHED(net);
        s.prepared = true;
        if (net->bwd_tiled() && s.n_chunks > 0) {
            b200::ft_csr_kernel<<<s.n_chunks, b200::kCsrThreads, b200::ft_csr_smem(d.ft_block_rows, d.nnz, s.chunk_len), net->copy_stream>>>(fa, ta);
            LAUNCHED(net);
            s.csr_built = true;
        }
    }
    CK(cudaEventRecord(s.ready, net->copy_stream));
    s.has_ready = true;
    s.has_consumed = false;
    s.n = n;
    return 0;
}

static int upload_finish(b200_net* net, Slot& s, int32_t n) {
    const b200_net_desc& d = net->d;
    const int O = d.n_out_buckets, nb = net->nblocks;
    int* h_buckets = s.host<int>(s.off_buckets);
    const uint16_t* h_stm = s.host<uint16_t>(s.off_stm);
    const uint16_t* h_nstm = s.host<uint16_t>(s.off_nstm);
    // visiting order of the dense weight-gradient kernel: positions grouped by output bucket (stable)
    std::vector<int> bucket_count(O, 0), block_count(nb, 0);
    {
        int* h_order = s.host<int>(s.off_order);
        std::vector<int> begin(O + 1, 0);
        for (int i = 0; i < n; i++) begin[h_buckets[i] + 1]++;
        for (int k = 0; k < O; k++) bucket_count[k] = begin[k + 1];
        for (int k = 0; k < O; k++) begin[k + 1] += begin[k];
        for (int i = 0; i < n; i++) h_order[begin[h_buckets[i]]++] = i;
    }
    // visiting order of the tiled feature-transformer kernels: (position, perspective)
    // pairs grouped by the table row block their features live in (stable)
    if (nb > 1) {
        int* h_pairs = s.host<int>(s.off_pairs);
        const int R = d.ft_block_rows, nnz = d.nnz;
        std::vector<int> begin(nb + 1, 0);
        std::vector<uint16_t> blk((size_t)2 * n);
#pragma omp parallel for schedule(static) if (n > 8192)
        for (int i = 0; i < n; i++) {
            for (int p = 0; p < 2; p++) {
                const uint16_t* list = (p ? h_nstm : h_stm) + (size_t)i * nnz;
                int b = 0;
                for (int k = 0; k < nnz; k++)
                    if (list[k] != 0xFFFFu) {
                        b = list[k] / R;
                        break;
                    }
                blk[(size_t)2 * i + p] = (uint16_t)b;
            }
        }
        for (size_t i = 0; i < blk.size(); i++) begin[blk[i] + 1]++;
        for (int k = 0; k < nb; k++) block_count[k] = begin[k + 1];
        for (int k = 0; k < nb; k++) begin[k + 1] += begin[k];
        for (size_t i = 0; i < blk.size(); i++) h_pairs[begin[blk[i]]++] = (int)i;
    } else {
        block_count[0] = 2 * n;
    }
    derive_tables(net, s, bucket_count.data(), block_count.data());
    CK(cudaMemcpyAsync(s.d_blob, s.h_blob, s.bytes, cudaMemcpyHostToDevice, net->copy_stream));
    net->h2d_bytes += (int64_t)s.bytes;
    return upload_launch_lists(net, s, n);
}

// Records in, batch prepared ON the device: 32 bytes per position cross PCIe instead of the packed lists,
// and the host only sizes the launches from two small histograms it reads back.
int b200_batch_upload_records_gpu(b200_net* net, int slot, const void* records, int32_t n, int32_t game, const int32_t* layout32,
                                  float scale, float blend) {
    if (!net || !records) return b200::fail(B200_ERR_ARG, "batch_upload_records_gpu: null argument");
    if (game < B200_GAME_CHESS768 || game > B200_GAME_ATAXX147) return b200::fail(B200_ERR_ARG, "batch_upload_records_gpu: unknown game %d", game);
    if (game == B200_GAME_CHESS_BUCKETS_MIRRORED && !layout32) return b200::fail(B200_ERR_ARG, "batch_upload_records_gpu: the king-bucket layout is missing");
    if (!(blend >= 0.f && blend <= 1.f) || !(scale > 0.f)) return b200::fail(B200_ERR_ARG, "batch_upload_records_gpu: bad scale or blend");
    const b200_net_desc& d = net->d;
    const int O = d.n_out_buckets, nb = net->nblocks, nbins = nb + O;
    if (O > 1 && game == B200_GAME_ATAXX147) return b200::fail(B200_ERR_UNSUPPORTED, "batch_upload_records_gpu: no output buckets for ataxx records");
    if (nb > b200::kPrepMaxBins || O > b200::kPrepMaxBins)
        return b200::fail(B200_ERR_UNSUPPORTED, "batch_upload_records_gpu: at most %d row blocks and output buckets; use b200_batch_upload_records",
                          b200::kPrepMaxBins);
    if (int rc = upload_begin(net, slot, n, "batch_upload_records_gpu")) return rc;
    Slot& s = net->slots[slot];
    const size_t B = d.max_batch;
    const int max_ctas = (int)((B + b200::kPrepPositions - 1) / b200::kPrepPositions);
    if (!s.d_records) {  // first use of this slot by the device path: its scratch, sized for the largest batch
        CK(cudaMalloc(&s.d_records, B * 32));
        CK(cudaMalloc(&s.d_pair_block, 2 * B * sizeof(uint16_t)));
        CK(cudaMalloc(&s.d_cta_hist, (size_t)max_ctas * nbins * sizeof(int)));
        CK(cudaMalloc(&s.d_totals, (size_t)2 * nbins * sizeof(int)));
        CK(cudaHostAlloc(&s.h_totals, ((size_t)2 * nbins + 1) * sizeof(int), cudaHostAllocDefault));
        CK(cudaEventCreateWithFlags(&s.totals_ready, cudaEventDisableTiming));
    }
    if (!net->d_win_rate) {
        CK(cudaMalloc(&net->d_win_rate, 65536 * sizeof(float)));
        CK(cudaMalloc(&net->d_expanded, 64 * sizeof(int)));
    }
    if (net->win_rate_scale != scale) {  // the same function the host mapper evaluates, for every possible score
        std::vector<float> table(65536);
        const float rscale = 1.0f / scale;
        for (int v = -32768; v < 32768; v++) table[v + 32768] = b200::blended_target((int16_t)v, 0, rscale, 0.0f);
        CK(cudaStreamSynchronize(net->copy_stream));
        CK(cudaMemcpy(net->d_win_rate, table.data(), table.size() * sizeof(float), cudaMemcpyHostToDevice));
        net->win_rate_scale = scale;
    }
    if (game == B200_GAME_CHESS_BUCKETS_MIRRORED && (!net->expanded_valid || memcmp(net->expanded_layout, layout32, sizeof net->expanded_layout))) {
        int32_t expanded[64];
        b200::expand_king_buckets(layout32, expanded);
        CK(cudaStreamSynchronize(net->copy_stream));
        CK(cudaMemcpy(net->d_expanded, expanded, sizeof expanded, cudaMemcpyHostToDevice));
        memcpy(net->expanded_layout, layout32, sizeof net->expanded_layout);
        net->expanded_valid = true;
    }
    // the records go through the slot's pinned block (its list sections are not used on the host here)
    memcpy(s.h_blob, records, (size_t)n * 32);
    CK(cudaMemcpyAsync(s.d_records, s.h_blob, (size_t)n * 32, cudaMemcpyHostToDevice, net->copy_stream));
    CK(cudaMemsetAsync(s.dev<int>(s.off_status), 0, sizeof(int), net->copy_stream));
    net->h2d_bytes += (int64_t)n * 32;
    b200::PrepArgs p{};
    p.records = s.d_records;
    p.n = n;
    p.nnz = d.nnz;
    p.n_inputs = d.n_inputs;
    p.game = game;
    p.n_out_buckets = O;
    p.block_rows = net->tiled_ok ? d.ft_block_rows : d.n_inputs;
    p.nblocks = nb;
    p.expanded = net->d_expanded;
    p.win_rate = net->d_win_rate;
    p.blend = blend;
    p.stm = s.dev<uint16_t>(s.off_stm);
    p.nstm = s.dev<uint16_t>(s.off_nstm);
    p.buckets = s.dev<int>(s.off_buckets);
    p.targets = s.dev<float>(s.off_targets);
    p.pair_block = s.d_pair_block;
    p.cta_hist = s.d_cta_hist;
    p.totals = s.d_totals;
    p.order = s.dev<int>(s.off_order);
    p.pair_order = s.dev<int>(s.off_pairs);
    p.status = s.dev<int>(s.off_status);
    const int ctas = (n + b200::kPrepPositions - 1) / b200::kPrepPositions;
    b200::prep_featurise_kernel<<<ctas, b200::kPrepPositions, 0, net->copy_stream>>>(p);
    LAUNCHED(net);
    b200::prep_scan_kernel<<<1, 512, 0, net->copy_stream>>>(p, ctas);
    LAUNCHED(net);
    CK(cudaMemcpyAsync(s.h_totals, s.d_totals, (size_t)2 * nbins * sizeof(int), cudaMemcpyDeviceToHost, net->copy_stream));
    CK(cudaMemcpyAsync(s.h_totals + 2 * nbins, s.dev<int>(s.off_status), sizeof(int), cudaMemcpyDeviceToHost, net->copy_stream));
    CK(cudaEventRecord(s.totals_ready, net->copy_stream));
    b200::prep_scatter_kernel<<<ctas, 2 * b200::kPrepPositions, 0, net->copy_stream>>>(p);
    LAUNCHED(net);
    // the host needs the bin totals to lay out chunks and tiles and to size the step's launches
    CK(cudaEventSynchronize(s.totals_ready));
    const int status = s.h_totals[2 * nbins];
    if (status & b200::kStatusTooManyPieces) return b200::fail(B200_ERR_DATA, "batch_upload_records_gpu: a record holds more than nnz=%d pieces", d.nnz);
    if (status & b200::kStatusBadBucket) return b200::fail(B200_ERR_DATA, "batch_upload_records_gpu: a record has no valid output bucket");
    derive_tables(net, s, s.h_totals + nb, s.h_totals);
    // only the derived tables travel: they sit behind the lists and the two orders in the slot's block
    const size_t tail = s.off_blocks;
    CK(cudaMemcpyAsync(s.d_blob + tail, s.h_blob + tail, s.bytes - tail, cudaMemcpyHostToDevice, net->copy_stream));
    net->h2d_bytes += (int64_t)(s.bytes - tail);
    return upload_launch_lists(net, s, n);
}

int b200_slot_read(b200_net* net, int slot, uint16_t* stm, uint16_t* nstm, int32_t* buckets, float* targets, int32_t* order,
                   int32_t* pair_order, int32_t* n) {
    if (int rc = check_slot(net, slot, "slot_read")) return rc;
    if (int rc = set_device(net)) return rc;
    const Slot& s = net->slots[slot];
    CK(cudaStreamSynchronize(net->copy_stream));
    const size_t count = (size_t)s.n, list = count * net->d.nnz * sizeof(uint16_t);
    if (stm) CK(cudaMemcpy(stm, s.d_blob + s.off_stm, list, cudaMemcpyDeviceToHost));
    if (nstm) CK(cudaMemcpy(nstm, s.d_blob + s.off_nstm, list, cudaMemcpyDeviceToHost));
    if (buckets) CK(cudaMemcpy(buckets, s.d_blob + s.off_buckets, count * 4, cudaMemcpyDeviceToHost));
    if (targets) CK(cudaMemcpy(targets, s.d_blob + s.off_targets, count * 4, cudaMemcpyDeviceToHost));
    if (order) CK(cudaMemcpy(order, s.d_blob + s.off_order, count * 4, cudaMemcpyDeviceToHost));
    if (pair_order) {
        if (net->nblocks > 1) {
            CK(cudaMemcpy(pair_order, s.d_blob + s.off_pairs, count * 8, cudaMemcpyDeviceToHost));
        } else {  // a single row block is visited in pair order and keeps no list
            for (size_t i = 0; i < 2 * count; i++) pair_order[i] = (int32_t)i;
        }
    }
    if (n) *n = s.n;
    return 0;
}

// ---- the training forward pass in pieces (b200_backward_begin runs them itself when the caller has not)

int b200_forward_begin(b200_net* net, int slot) {
    if (int rc = check_slot(net, slot, "forward_begin")) return rc;
    if (net->bwd_slot >= 0) return b200::fail(B200_ERR_STATE, "forward_begin: the backward pass of slot %d is not finished", net->bwd_slot);
    if (int rc = set_device(net)) return rc;
    Slot& s = net->slots[slot];
    CK(cudaStreamWaitEvent(net->stream, s.ready, 0));
    if (int rc = refresh_table(net)) return rc;
    if (!net->manual_grad_zero) {
        // every gradient is accumulated with reductions, so the buffer starts at zero; nothing before
        // the dense layers writes to it, so the clearing runs on a side stream beside the FT forward
        CK(cudaEventRecord(net->zero_fork, net->stream));
        CK(cudaStreamWaitEvent(net->zero_stream, net->zero_fork, 0));
        CK(cudaMemsetAsync(net->G, 0, (size_t)net->n_flat * 4, net->zero_stream));
        CK(cudaEventRecord(net->zero_done, net->zero_stream));
        net->zero_pending = true;
    }
    if (int rc = forward_prepare(net, s, true)) return rc;
    net->fwd_slot = slot;
    net->fwd_parts_done = 0;
    net->fwd_parts = 0;
    return 0;
}

int b200_forward_ft(b200_net* net, int slot, int part, int n_parts) {
    if (int rc = check_slot(net, slot, "forward_ft")) return rc;
    if (net->fwd_slot != slot) return b200::fail(B200_ERR_STATE, "forward_ft: call b200_forward_begin on slot %d first", slot);
    if (n_parts < 1 || part < 0 || part >= n_parts || part != net->fwd_parts_done)
        return b200::fail(B200_ERR_ARG, "forward_ft: parts must be run in order 0..n_parts-1 (got %d of %d)", part, n_parts);
    if (n_parts > 1 && (!net->fwd_tiled() || net->nblocks % n_parts))
        return b200::fail(B200_ERR_UNSUPPORTED, "forward_ft: %d parts need the tiled forward and must divide the %d row blocks", n_parts,
                          net->nblocks);
    if (int rc = set_device(net)) return rc;
    Slot& s = net->slots[slot];
    const int per = net->nblocks / n_parts;  // this part's run of row blocks
    if (int rc = forward_ft_blocks(net, s, part * per, n_parts > 1 ? (part + 1) * per : net->nblocks)) return rc;
    net->fwd_parts_done = part + 1;
    net->fwd_parts = n_parts;
    return 0;
}

// ---- the backward pass in three phases (b200_backward runs them back to back)

int b200_backward_begin(b200_net* net, int slot) {
    if (int rc = check_slot(net, slot, "backward_begin")) return rc;
    if (int rc = set_device(net)) return rc;
    Slot& s = net->slots[slot];
    const b200_net_desc& d = net->d;
    if (net->fwd_slot == slot) {  // the forward pass was started in pieces: every piece must be in
        if (net->fwd_parts_done < 1 || net->fwd_parts_done != net->fwd_parts)
            return b200::fail(B200_ERR_STATE, "backward_begin: run every b200_forward_ft part of slot %d first", slot);
    } else {
        if (net->fwd_slot >= 0) return b200::fail(B200_ERR_STATE, "backward_begin: a forward pass of slot %d is under way", net->fwd_slot);
        if (int rc = b200_forward_begin(net, slot)) return rc;
        if (int rc = b200_forward_ft(net, slot, 0, 1)) return rc;
    }
    net->fwd_slot = -1;
    if (int rc = forward_dense(net, s, true)) return rc;
    cudaEvent_t* ev = net->tev[net->steps_begun % b200_net::kTimingRing];
    CK(cudaEventRecord(ev[2], net->stream));
    if (net->bwd_tiled() && s.n_chunks > 0 && !s.csr_built) {  // normally built at upload
        b200::FtArgs fa = ft_args(net, s);
        b200::TileArgs ta = tile_args(net, s, true);
        b200::ft_csr_kernel<<<s.n_chunks, b200::kCsrThreads, b200::ft_csr_smem(d.ft_block_rows, d.nnz, s.chunk_len), net->stream>>>(fa, ta);
        LAUNCHED(net);
        s.csr_built = true;
    }
    {
        b200::DenseArgs da = dense_args(net, s, true);
        DISPATCH_M(d.dense_out[0], b200::dense_dx_kernel<MM><<<s.n_dtiles, 256, 0, net->stream>>>(da, net->dx));
        LAUNCHED(net);
    }
    if (int rc = launch_dense_grads(net, s)) return rc;
    CK(cudaEventRecord(ev[3], net->stream));
    net->bwd_slot = slot;
    net->bwd_parts_done = 0;
    net->last_n = s.n;
    return 0;
}

int b200_backward_ft(b200_net* net, int slot, int part, int n_parts) {
    if (int rc = check_slot(net, slot, "backward_ft")) return rc;
    if (net->bwd_slot != slot) return b200::fail(B200_ERR_STATE, "backward_ft: call b200_backward_begin on slot %d first", slot);
    const bool tiled = net->bwd_tiled();
    if (n_parts < 1 || part < 0 || part >= n_parts || part != net->bwd_parts_done)
        return b200::fail(B200_ERR_ARG, "backward_ft: parts must be run in order 0..n_parts-1 (got %d of %d)", part, n_parts);
    if (n_parts > 1 && (!tiled || net->nblocks % n_parts))
        return b200::fail(B200_ERR_UNSUPPORTED, "backward_ft: %d parts need the tiled backward and must divide the %d row blocks",
                          n_parts, net->nblocks);
    if (int rc = set_device(net)) return rc;
    Slot& s = net->slots[slot];
    const b200_net_desc& d = net->d;
    cudaEvent_t* ev = net->tev[net->steps_begun % b200_net::kTimingRing];
    const int per = net->nblocks / n_parts;
    const Tensor* l0w = net->find("l0w");
    {
        b200::FtArgs fa = ft_args(net, s);
        b200::TileArgs ta = tile_args(net, s, true);
        int grid = 0;
        bool any = true;
        if (tiled) {  // this part's run of blocks
            ta.first_block = part * per;
            ta.last_block = n_parts > 1 ? (part + 1) * per : net->nblocks;
            any = s.chunk_begin[ta.last_block] > s.chunk_begin[ta.first_block];
            grid = ft_backward_grid(net, s, ta.first_block, ta.last_block, net->sig_on);
            if (net->sig_on && grid != s.expect_grid)
                return b200::fail(B200_ERR_STATE, "backward_ft: the batch was uploaded before the exchange under the backward was switched on");
        }
        if (any) {
            int rc = d.pairwise ? launch_ft_backward<true>(net, fa, ta, tiled, grid) : launch_ft_backward<false>(net, fa, ta, tiled, grid);
            if (rc) return rc;
        }
    }
    if (part == n_parts - 1) CK(cudaEventRecord(ev[4], net->stream));
    if (d.factoriser_rows && !(net->sig_on && net->facc)) {  // (the overlapped exchange sums the reduced blocks itself)
        // sum of this part's copies of the factoriser rows; with one part: all copies, in order
        const Tensor* f = net->find("l0f");
        const int copies = (int)(l0w->n / f->n), per_part = copies / n_parts;
        if (copies % n_parts) return b200::fail(B200_ERR_UNSUPPORTED, "backward_ft: %d parts do not divide %d factoriser copies", n_parts, copies);
        b200::factoriser_grad_kernel<<<net->sm_count * 4, 256, 0, net->stream>>>(
            reinterpret_cast<const float4*>(net->G + l0w->off + (int64_t)part * per_part * f->n),
            reinterpret_cast<float4*>(net->G + f->off), (size_t)f->n / 4, per_part, part > 0);
        LAUNCHED(net);
    }
    if (part == n_parts - 1) CK(cudaEventRecord(ev[5], net->stream));
    net->bwd_parts_done = part + 1;
    net->bwd_parts = n_parts;
    return 0;
}

int b200_backward_end(b200_net* net, int slot) {
    if (int rc = check_slot(net, slot, "backward_end")) return rc;
    if (net->bwd_slot != slot || net->bwd_parts_done < 1 || net->bwd_parts_done != net->bwd_parts)
        return b200::fail(B200_ERR_STATE, "backward_end: run b200_backward_begin and every b200_backward_ft part first");
    if (int rc = set_device(net)) return rc;
    Slot& s = net->slots[slot];
    cudaEvent_t* ev = net->tev[net->steps_begun % b200_net::kTimingRing];
    CK(cudaEventRecord(ev[6], net->stream));
    // the status word travels with the step, not with the slot: once `consumed` is recorded the uploader may
    // clear and refill the slot while the update of this step is still to come
    if (net->status_slot >= 0)
        CK(cudaMemcpyAsync(net->d_status + net->updates % b200_net::kLossRing, s.dev<int>(s.off_status), sizeof(int),
                           cudaMemcpyDeviceToDevice, net->stream));
    CK(cudaEventRecord(s.consumed, net->stream));
    s.has_consumed = true;
    net->have_backward = true;
    net->step_open = true;
    net->bwd_slot = -1;
    return 0;
}

int b200_backward(b200_net* net, int slot) {
    if (int rc = b200_backward_begin(net, slot)) return rc;
    if (int rc = b200_backward_ft(net, slot, 0, 1)) return rc;
    return b200_backward_end(net, slot);
}

int b200_grad_part(b200_net* net, int part, int n_parts, int64_t* first_float, int64_t* n_floats) {
    if (!net || !first_float || !n_floats) return b200::fail(B200_ERR_ARG, "grad_part: null argument");
    const Tensor* l0w = net->find("l0w");
    if (n_parts < 1 || part < 0 || part > n_parts) return b200::fail(B200_ERR_ARG, "grad_part: part %d of %d", part, n_parts);
    if (part == n_parts) {  // the head: loss and every tensor but l0w
        *first_float = 0;
        *n_floats = l0w->off;
        return 0;
    }
    if (net->nblocks % n_parts) return b200::fail(B200_ERR_UNSUPPORTED, "grad_part: %d parts do not divide %d row blocks", n_parts, net->nblocks);
    const int64_t per = l0w->n / n_parts;
    *first_float = l0w->off + part * per;
    *n_floats = part == n_parts - 1 ? net->n_flat - *first_float : per;  // the last part takes the alignment tail
    return 0;
}

int b200_update_range(b200_net* net, float lr, float grad_factor, int64_t first_float, int64_t n_floats) {
    if (!net) return b200::fail(B200_ERR_ARG, "update_range: null net");
    if (!net->have_backward) return b200::fail(B200_ERR_STATE, "update_range: no gradients yet, call b200_backward first");
    if (first_float < 0 || n_floats < 1 || first_float + n_floats > net->n_flat || first_float % 4 || n_floats % 4)
        return b200::fail(B200_ERR_ARG, "update_range: [%lld, +%lld) is not a 4-float-aligned range of the flat buffer",
                          (long long)first_float, (long long)n_floats);
    if (int rc = set_device(net)) return rc;
    b200::AdamArgs a{};
    a.p = reinterpret_cast<float4*>(net->P);
    a.m = reinterpret_cast<float4*>(net->M);
    a.v = reinterpret_cast<float4*>(net->V);
    a.g = reinterpret_cast<const float4*>(net->G);
    a.first4 = first_float / 4;
    a.total4 = n_floats / 4;
    a.rate = lr;
    a.adj = grad_factor;
    fill_segments(net, a);
    const long long blocks = std::min<long long>((a.total4 + 255) / 256, net->sm_count * 16);
    b200::adamw_flat_kernel<<<(unsigned)blocks, 256, 0, net->stream>>>(a);
    LAUNCHED(net);
    net->table_dirty = true;
    return 0;
}

// ---- the data-parallel update over peer memory (one process per GPU)

int b200_exchange_export(b200_net* net, void* handles, int64_t bytes) {
    if (!net || !handles) return b200::fail(B200_ERR_ARG, "exchange_export: null argument");
    static_assert(3 * sizeof(cudaIpcMemHandle_t) == B200_EXCHANGE_HANDLE_BYTES, "handle size");
    if (bytes < B200_EXCHANGE_HANDLE_BYTES) return b200::fail(B200_ERR_ARG, "exchange_export: %d bytes are needed", B200_EXCHANGE_HANDLE_BYTES);
    if (int rc = set_device(net)) return rc;
    cudaIpcMemHandle_t h[3];
    CK(cudaIpcGetMemHandle(&h[0], net->G));
    CK(cudaIpcGetMemHandle(&h[1], net->P));
    CK(cudaIpcGetMemHandle(&h[2], net->xch_flags));
    memcpy(handles, h, sizeof h);
    return 0;
}

int b200_exchange_import(b200_net* net, int rank, int world, const void* handles, int64_t bytes) {
    if (!net || !handles) return b200::fail(B200_ERR_ARG, "exchange_import: null argument");
    if (world < 2 || world > b200::kMaxRanks || rank < 0 || rank >= world)
        return b200::fail(B200_ERR_ARG, "exchange_import: rank %d of %d (at most %d ranks)", rank, world, b200::kMaxRanks);
    if (bytes < (int64_t)world * B200_EXCHANGE_HANDLE_BYTES) return b200::fail(B200_ERR_ARG, "exchange_import: handles of %d ranks are needed", world);
    if (net->xch_world) return b200::fail(B200_ERR_STATE, "exchange_import: peers are already mapped");
    if (net->n_flat % (4 * world)) return b200::fail(B200_ERR_UNSUPPORTED, "exchange_import: the flat buffer does not split over %d ranks", world);
    if (int rc = set_device(net)) return rc;
    const cudaIpcMemHandle_t* h = static_cast<const cudaIpcMemHandle_t*>(handles);
    auto unmap_all = [&]() {
        for (int q = 0; q < world; q++)
            if (q != rank) {
                if (net->peer_g[q]) cudaIpcCloseMemHandle(net->peer_g[q]);
                if (net->peer_p[q]) cudaIpcCloseMemHandle(net->peer_p[q]);
                if (net->peer_flags[q]) cudaIpcCloseMemHandle(net->peer_flags[q]);
            }
        memset(net->peer_g, 0, sizeof net->peer_g);
        memset(net->peer_p, 0, sizeof net->peer_p);
        memset(net->peer_flags, 0, sizeof net->peer_flags);
    };
    for (int r = 0; r < world; r++) {
        if (r == rank) {
            net->peer_g[r] = net->G;
            net->peer_p[r] = net->P;
            net->peer_flags[r] = net->xch_flags;
            continue;
        }
        void* mapped[3] = {nullptr, nullptr, nullptr};
        cudaError_t e = cudaSuccess;
        for (int k = 0; k < 3 && e == cudaSuccess; k++) e = cudaIpcOpenMemHandle(&mapped[k], h[3 * r + k], cudaIpcMemLazyEnablePeerAccess);
        net->peer_g[r] = static_cast<float*>(mapped[0]);
        net->peer_p[r] = static_cast<float*>(mapped[1]);
        net->peer_flags[r] = static_cast<int*>(mapped[2]);
        if (e != cudaSuccess) {
            cudaGetLastError();
            unmap_all();
            return b200::fail(B200_ERR_CUDA, "exchange_import: cannot map the buffers of rank %d: %s", r, cudaGetErrorString(e));
        }
    }
    net->xch_rank = rank;
    net->xch_world = world;
    b200::PeerFlags f{};
    f.world = world;
    f.rank = rank;
    f.spin_limit = net->xch_spin_limit;
    for (int r = 0; r < world; r++) f.flags[r] = net->peer_flags[r];
    CK(cudaMemcpy(net->d_peers, &f, sizeof f, cudaMemcpyHostToDevice));
    return 0;
}

int b200_update_exchange_range(b200_net* net, float lr, float grad_factor, int64_t first_float, int64_t n_floats, int gather,
                               void* stream) {
    if (!net) return b200::fail(B200_ERR_ARG, "update_exchange: null net");
    if (!net->xch_world) return b200::fail(B200_ERR_STATE, "update_exchange: map the peers with b200_exchange_import first");
    if (first_float < 0 || n_floats < 1 || first_float + n_floats > net->n_flat || first_float % 4 || n_floats % 4)
        return b200::fail(B200_ERR_ARG, "update_exchange: [%lld, +%lld) is not a 4-float-aligned range of the flat buffer",
                          (long long)first_float, (long long)n_floats);
    if (int rc = set_device(net)) return rc;
    b200::ExchangeArgs x{};
    b200::AdamArgs& a = x.adam;
    a.p = reinterpret_cast<float4*>(net->P);
    a.m = reinterpret_cast<float4*>(net->M);
    a.v = reinterpret_cast<float4*>(net->V);
    a.g = nullptr;
    a.first4 = first_float / 4;
    a.total4 = n_floats / 4;
    a.rate = lr;
    a.adj = grad_factor;
    fill_segments(net, a);
    x.world = net->xch_world;
    x.store_peers = gather ? 1 : 0;
    x.head4 = kAlignFloats / 4;
    x.flags.world = net->xch_world;
    x.flags.rank = net->xch_rank;
    x.flags.spin_limit = net->xch_spin_limit;
    x.wait_ready = net->xch_wait_ready;
    for (int r = 0; r < x.world; r++) {
        x.g[r] = reinterpret_cast<const float4*>(net->peer_g[r]);
        x.p_out[r] = reinterpret_cast<float4*>(net->peer_p[r]);
        x.flags.flags[r] = net->peer_flags[r];
    }
    // On the net's own stream the kernel runs alone and takes the whole device.  On a caller's side
    // stream it runs beside the feature-transformer kernels, whose CTAs leave room for exactly one
    // such CTA per SM: more CTAs would take whole SMs away from them instead of filling the gaps.
    const long long cap = stream ? (net->exchange_ctas > 0 ? net->exchange_ctas : net->sm_count) : net->sm_count * 8;
    const long long blocks = std::min<long long>((a.total4 + 127) / 128, cap);
    cudaStream_t on = stream ? static_cast<cudaStream_t>(stream) : net->stream;
    if (net->exchange_bulk && !stream && x.store_peers) {
        // gradients fetched and weights sent by bulk copies: one CTA per SM over the tiles of this rank's share
#define BULK(W, T, S)                                                                                                           \
    do {                                                                                                                        \
        const long long tiles = (a.total4 + (T)-1) / (T);                                                                       \
        const unsigned ctas = (unsigned)std::min<long long>(net->sm_count, tiles);                                              \
        cudaFuncSetAttribute(b200::adamw_exchange_bulk_kernel<W, T, S>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                             (int)b200::exchange_bulk_smem<W, T, S>());                                                         \
        b200::adamw_exchange_bulk_kernel<W, T, S><<<ctas, T, b200::exchange_bulk_smem<W, T, S>(), on>>>(x);                     \
    } while (0)
        const int variant = net->exchange_bulk;
        if (x.world == 2) {
            if (variant == 2) BULK(2, 512, 3);
            else if (variant == 3) BULK(2, 128, 12);
            else BULK(2, 256, 6);
        } else if (x.world == 4) {
            BULK(4, 256, 5);
        } else {
            if (variant == 2) BULK(0, 512, 1);
            else if (variant == 3) BULK(0, 128, 6);
            else BULK(0, 256, 3);
        }
#undef BULK
        LAUNCHED(net);
        net->table_dirty = true;
        if (first_float == 0) net->loss_in_param = true;
        return 0;
    }
    switch (x.world) {
        case 2: b200::adamw_exchange_kernel<2><<<(unsigned)blocks, 128, 0, on>>>(x); break;
        case 4: b200::adamw_exchange_kernel<4><<<(unsigned)blocks, 128, 0, on>>>(x); break;
        case 8: b200::adamw_exchange_kernel<8><<<(unsigned)blocks, 128, 0, on>>>(x); break;
        default: b200::adamw_exchange_kernel<0><<<(unsigned)blocks, 128, 0, on>>>(x); break;
    }
    LAUNCHED(net);
    net->table_dirty = true;
    if (first_float == 0) net->loss_in_param = true;  // the range holds the loss: it now sits in P[0]
    return 0;
}

int b200_update_exchange(b200_net* net, float lr, float grad_factor) {
    if (!net) return b200::fail(B200_ERR_ARG, "update_exchange: null net");
    if (!net->xch_world) return b200::fail(B200_ERR_STATE, "update_exchange: map the peers with b200_exchange_import first");
    if (!net->have_backward) return b200::fail(B200_ERR_STATE, "update_exchange: no gradients yet, call b200_backward first");
    const int64_t per = net->n_flat / net->xch_world;
    if (int rc = set_device(net)) return rc;
    // fences without a collective: tell the peers that this rank's gradients are complete; the exchange
    // kernel waits for every peer's word before it reads; afterwards the same once more for "finished",
    // so that nobody overwrites gradients or reads weights while a peer's kernel is still at work
    b200::PeerFlags f{};
    f.world = net->xch_world;
    f.rank = net->xch_rank;
    f.spin_limit = net->xch_spin_limit;
    for (int r = 0; r < f.world; r++) f.flags[r] = net->peer_flags[r];
    const int step = ++net->xch_step;
    b200::peer_signal_kernel<<<1, 32, 0, net->stream>>>(f, b200::kFlagReady, step);
    LAUNCHED(net);
    net->xch_wait_ready = step;
    int rc = b200_update_exchange_range(net, lr, grad_factor, net->xch_rank * per, per, 1, nullptr);
    net->xch_wait_ready = 0;
    if (rc) return rc;
    b200::peer_signal_kernel<<<1, 32, 0, net->stream>>>(f, b200::kFlagDone, step);
    LAUNCHED(net);
    b200::peer_wait_kernel<<<1, 32, 0, net->stream>>>(f, b200::kFlagDone, step);
    LAUNCHED(net);
    net->loss_in_param = true;  // rank 0's share starts with the loss and stores it to every rank
    net->xch_fenced_used = true;
    return 0;
}

// One data-parallel step with the exchange under the backward pass (see adamw_exchange_overlap_kernel).
int b200_step_exchange(b200_net* net, int slot, float lr, float grad_factor) {
    if (!net) return b200::fail(B200_ERR_ARG, "step_exchange: null net");
    if (!net->xch_world) return b200::fail(B200_ERR_STATE, "step_exchange: map the peers with b200_exchange_import first");
    const b200_net_desc& d = net->d;
    const Tensor* l0w = net->find("l0w");
    const Tensor* l0f = d.factoriser_rows ? net->find("l0f") : nullptr;
    const int64_t block_floats = (int64_t)d.ft_block_rows * d.ft_out;
    if (!net->bwd_tiled() || net->nblocks > b200::kMaxSignalBlocks)
        return b200::fail(B200_ERR_UNSUPPORTED, "step_exchange: needs the tiled backward (ft_block_rows > 0) and at most %d row blocks",
                          b200::kMaxSignalBlocks);
    if (block_floats % (4 * net->xch_world)) return b200::fail(B200_ERR_UNSUPPORTED, "step_exchange: a row block does not split over %d ranks", net->xch_world);
    if (l0f && !net->facc) return b200::fail(B200_ERR_UNSUPPORTED, "step_exchange: the factoriser must have as many rows as a row block");
    if (int rc = b200_backward_begin(net, slot)) return rc;
    Slot& s = net->slots[slot];
    const int step = ++net->xch_step;

    b200::OverlapArgs o{};
    b200::ExchangeArgs& x = o.x;
    b200::AdamArgs& a = x.adam;
    a.p = reinterpret_cast<float4*>(net->P);
    a.m = reinterpret_cast<float4*>(net->M);
    a.v = reinterpret_cast<float4*>(net->V);
    a.rate = lr;
    a.adj = grad_factor;
    fill_segments(net, a);
    o.l0f_seg = -1;
    for (int i = 0; i < a.nseg; i++) {
        if (&net->tensors[i] == l0w) o.l0w_seg = i;
        if (&net->tensors[i] == l0f) o.l0f_seg = i;
    }
    x.world = net->xch_world;
    x.store_peers = 1;
    x.head4 = kAlignFloats / 4;
    x.flags.world = net->xch_world;
    x.flags.rank = net->xch_rank;
    x.flags.spin_limit = net->xch_spin_limit;
    for (int r = 0; r < x.world; r++) {
        x.g[r] = reinterpret_cast<const float4*>(net->peer_g[r]);
        x.p_out[r] = reinterpret_cast<float4*>(net->peer_p[r]);
        x.flags.flags[r] = net->peer_flags[r];
    }
    o.step = step;
    o.nblocks = net->nblocks;
    o.l0w4 = l0w->off / 4;
    o.block4 = block_floats / 4;
    o.l0f4 = l0f ? l0f->off / 4 : 0;
    o.facc = l0f ? reinterpret_cast<float4*>(net->facc) : nullptr;

    // the exchange kernel goes first, on its own stream: it is resident (or first in line for an SM) by the
    // time the backward's CTAs arrive, and it depends on them, never they on it
    CK(cudaEventRecord(net->xch_fork, net->stream));
    CK(cudaStreamWaitEvent(net->xch_stream, net->xch_fork, 0));
    const int ctas = std::min(net->overlap_ctas, net->sm_count - 1);
    switch (x.world) {
        case 2: b200::adamw_exchange_overlap_kernel<2><<<ctas, b200::kOverlapThreads, b200::kOverlapSmem, net->xch_stream>>>(o); break;
        case 4: b200::adamw_exchange_overlap_kernel<4><<<ctas, b200::kOverlapThreads, b200::kOverlapSmem, net->xch_stream>>>(o); break;
        case 8: b200::adamw_exchange_overlap_kernel<8><<<ctas, b200::kOverlapThreads, b200::kOverlapSmem, net->xch_stream>>>(o); break;
        default: b200::adamw_exchange_overlap_kernel<0><<<ctas, b200::kOverlapThreads, b200::kOverlapSmem, net->xch_stream>>>(o); break;
    }
    LAUNCHED(net);
    b200::PeerFlags f = x.flags;
    // ... and behind it the closing fence: every rank's kernel has finished before anyone reuses gradients or weights
    b200::peer_signal_kernel<<<1, 32, 0, net->xch_stream>>>(f, b200::kFlagDone, step);
    LAUNCHED(net);
    b200::peer_wait_kernel<<<1, 32, 0, net->xch_stream>>>(f, b200::kFlagDone, step);
    LAUNCHED(net);
    CK(cudaEventRecord(net->xch_join, net->xch_stream));

    // the backward, announcing its row blocks as they finish
    net->sig_on = true;
    net->sig_value = step;
    {
        b200::TileArgs ta = tile_args(net, s, true);
        b200::bucket_presignal_kernel<<<1, 256, 0, net->stream>>>(ta.sig, net->nblocks);
        LAUNCHED(net);
    }
    int rc = b200_backward_ft(net, slot, 0, 1);
    net->sig_on = false;
    if (rc) return rc;
    b200::peer_signal_kernel<<<1, 32, 0, net->stream>>>(f, b200::kFlagReady, step);  // bias and dense gradients too
    LAUNCHED(net);
    if (int rc2 = b200_backward_end(net, slot)) return rc2;
    CK(cudaStreamWaitEvent(net->stream, net->xch_join, 0));
    net->loss_in_param = true;  // every rank reduced the loss into float 0 of its parameter buffer
    net->xch_fenced_used = true;
    net->table_dirty = true;
    return b200_update_end(net);
}

int b200_grad_zero_range(b200_net* net, int64_t first_float, int64_t n_floats) {
    if (!net) return b200::fail(B200_ERR_ARG, "grad_zero_range: null net");
    if (first_float < 0 || n_floats < 1 || first_float + n_floats > net->n_flat)
        return b200::fail(B200_ERR_ARG, "grad_zero_range: [%lld, +%lld) is outside the flat buffer", (long long)first_float, (long long)n_floats);
    if (int rc = set_device(net)) return rc;
    CK(cudaMemsetAsync(net->G + first_float, 0, (size_t)n_floats * 4, net->stream));
    return 0;
}

int b200_update_end(b200_net* net) {
    if (!net) return b200::fail(B200_ERR_ARG, "update_end: null net");
    if (!net->have_backward) return b200::fail(B200_ERR_STATE, "update_end: no gradients yet");
    if (int rc = set_device(net)) return rc;
    const int ring = (int)(net->updates % b200_net::kLossRing);
    CK(cudaMemcpyAsync(net->h_loss + ring, net->loss_in_param ? net->P : net->G, sizeof(float), cudaMemcpyDeviceToHost, net->stream));
    net->loss_in_param = false;
    if (net->status_slot >= 0) {
        CK(cudaMemcpyAsync(net->h_status + ring, net->d_status + ring, sizeof(int), cudaMemcpyDeviceToHost, net->stream));
    } else {
        net->h_status[ring] = 0;
    }
    if (net->xch_fenced_used) {
        // report the word with this step, then clear it: a later good step starts clean
        CK(cudaMemcpyAsync(net->h_xstatus + 4 * ring, net->xch_flags + b200::kFlagTimeout, 4 * sizeof(int), cudaMemcpyDeviceToHost, net->stream));
        CK(cudaMemsetAsync(net->xch_flags + b200::kFlagTimeout, 0, 4 * sizeof(int), net->stream));
    }
    CK(cudaEventRecord(net->loss_ev[ring], net->stream));
    net->updates++;
    net->opt_step++;
    {   // Ranger: every k-th step the fast weights are pulled towards the slow ones, which then follow
        b200::LookaheadArgs la{};
        la.p = reinterpret_cast<float4*>(net->P);
        la.slow = reinterpret_cast<float4*>(net->S);
        la.total4 = net->n_flat / 4;
        la.nseg = (int)net->tensors.size();
        bool any = false;
        for (int i = 0; i < la.nseg; i++) {
            const Tensor& t = net->tensors[i];
            la.begin4[i] = t.off / 4;
            la.end4[i] = (t.off + t.n + 3) / 4;
            const bool due = t.opt_kind == B200_OPT_RANGER && net->opt_step % t.lookahead_k == 0;
            la.alpha[i] = due ? t.alpha : -1.f;
            la.one_minus[i] = 1.0f - t.alpha;
            any = any || due;
        }
        if (any && net->S) {
            b200::lookahead_kernel<<<net->sm_count * 8, 256, 0, net->stream>>>(la);
            LAUNCHED(net);
            net->table_dirty = true;
        }
    }
    if (int rc = refresh_table(net)) return rc;
    if (net->step_open) {  // close the timed step begun by the matching backward
        CK(cudaEventRecord(net->tev[net->steps_begun % b200_net::kTimingRing][7], net->stream));
        net->steps_begun++;
        net->steps_done = net->steps_begun;
        net->step_open = false;
    }
    return 0;
}

int b200_update(b200_net* net, float lr, float grad_factor) {
    if (!net) return b200::fail(B200_ERR_ARG, "update: null net");
    if (int rc = b200_update_range(net, lr, grad_factor, 0, net->n_flat)) return rc;
    return b200_update_end(net);
}

int b200_step(b200_net* net, int slot, float lr, float grad_factor) {
    if (int rc = b200_backward(net, slot)) return rc;
    return b200_update(net, lr, grad_factor);
}

int b200_grad_buffer(b200_net* net, void** device_ptr, int64_t* n_floats) {
    if (!net || !device_ptr || !n_floats) return b200::fail(B200_ERR_ARG, "grad_buffer: null argument");
    *device_ptr = net->G;
    *n_floats = net->n_flat;
    return 0;
}

int b200_flat_buffer(b200_net* net, int kind, void** device_ptr, int64_t* n_floats) {
    if (!net || !device_ptr || !n_floats) return b200::fail(B200_ERR_ARG, "flat_buffer: null argument");
    float* base = kind_base(net, kind);
    if (!base) return b200::fail(B200_ERR_ARG, "flat_buffer: unknown kind %d", kind);
    *device_ptr = base;
    *n_floats = net->n_flat;
    return 0;
}

int b200_loss_of(b200_net* net, int steps_back, float* loss_sum) {
    if (!net || !loss_sum) return b200::fail(B200_ERR_ARG, "loss: null argument");
    if (steps_back < 0 || steps_back >= b200_net::kLossRing - 1)
        return b200::fail(B200_ERR_ARG, "loss: only the last %d updates are kept", b200_net::kLossRing - 1);
    if (net->updates <= steps_back) return b200::fail(B200_ERR_STATE, "loss: that update has not run yet");
    if (int rc = set_device(net)) return rc;
    const int ring = (int)((net->updates - 1 - steps_back) % b200_net::kLossRing);
    CK(cudaEventSynchronize(net->loss_ev[ring]));
    *loss_sum = net->h_loss[ring];
    if (net->h_xstatus[4 * ring]) {
        const int* x = net->h_xstatus + 4 * ring;
        const int base = x[1], value = x[2], who = x[3];
        net->h_xstatus[4 * ring] = 0;
        if (value == 0)
            return b200::fail(B200_ERR_STATE, "data-parallel exchange: a peer did not reach the fence in time (reported by another rank); "
                                              "the update of this step is not valid");
        return b200::fail(B200_ERR_STATE,
                          "data-parallel exchange: a peer did not reach the fence in time (rank %d never announced %s%d of step %d); the "
                          "update of this step is not valid",
                          who, base >= b200::kFlagBucket ? "row block " : base >= b200::kFlagDone ? "the end of its exchange, fence " : "its gradients, fence ",
                          base >= b200::kFlagBucket ? (base - b200::kFlagBucket) / b200::kMaxRanks : base, value);
    }
    if (net->h_status[ring] & b200::kStatusOutsideBlock) {
        net->h_status[ring] = 0;
        return b200::fail(B200_ERR_DATA,
                          "a feature index fell outside the row block of its position (ft_block_rows=%d): those "
                          "features were ignored; create the network with ft_block_rows=0 for such inputs",
                          net->d.ft_block_rows);
    }
    return 0;
}

int b200_loss(b200_net* net, float* loss_sum) { return b200_loss_of(net, 0, loss_sum); }

int b200_forward(b200_net* net, int slot, float* out_host) {
    if (int rc = check_slot(net, slot, "forward")) return rc;
    if (!out_host) return b200::fail(B200_ERR_ARG, "forward: null output");
    if (int rc = set_device(net)) return rc;
    Slot& s = net->slots[slot];
    CK(cudaStreamWaitEvent(net->stream, s.ready, 0));
    if (int rc = refresh_table(net)) return rc;
    if (int rc = forward_part(net, s, false)) return rc;
    CK(cudaEventRecord(s.consumed, net->stream));
    s.has_consumed = true;
    net->last_n = s.n;
    CK(cudaMemcpyAsync(out_host, net->out, (size_t)s.n * sizeof(float), cudaMemcpyDeviceToHost, net->stream));
    CK(cudaStreamSynchronize(net->stream));
    return 0;
}

int b200_sync(b200_net* net) {
    if (!net) return b200::fail(B200_ERR_ARG, "sync: null net");
    if (int rc = set_device(net)) return rc;
    CK(cudaStreamSynchronize(net->copy_stream));
    CK(cudaStreamSynchronize(net->stream));
    return 0;
}

int b200_get_timings(b200_net* net, b200_timings* out) {
    if (!net || !out) return b200::fail(B200_ERR_ARG, "get_timings: null argument");
    if (int rc = set_device(net)) return rc;
    memset(out, 0, sizeof *out);
    const int64_t first = std::max(net->timing_origin, net->steps_done - b200_net::kTimingRing);
    const int64_t count = net->steps_done - first;
    net->timing_origin = net->steps_done;
    if (count < 1) return b200::fail(B200_ERR_STATE, "get_timings: no complete step since the last call");
    CK(cudaStreamSynchronize(net->stream));
    // events: 0 start, 1 FT forward, 2 dense forward, 3 dx, 4 FT backward, 5 factoriser sums,
    // 6 dense weight gradients, 7 update
    double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int64_t i = first; i < net->steps_done; i++) {
        cudaEvent_t* ev = net->tev[i % b200_net::kTimingRing];
        float ms = 0.f;
        for (int k = 0; k < 7; k++) {
            CK(cudaEventElapsedTime(&ms, ev[k], ev[k + 1]));
            acc[k] += ms;
        }
        CK(cudaEventElapsedTime(&ms, ev[0], ev[7]));
        acc[7] += ms;
    }
    const double inv = 1.0 / (double)count;
    out->ft_forward = (float)(acc[0] * inv);
    out->dense_forward = (float)(acc[1] * inv);
    out->dense_backward = (float)((acc[2] + acc[5]) * inv);
    out->ft_backward = (float)(acc[3] * inv);
    out->factoriser_grad = (float)(acc[4] * inv);
    out->optimiser = (float)(acc[6] * inv);
    out->total = (float)(acc[7] * inv);
    out->steps = (int32_t)count;
    return 0;
}

int b200_net_get_stat(b200_net* net, const char* key, int64_t* value) {
    if (!net || !key || !value) return b200::fail(B200_ERR_ARG, "get_stat: null argument");
    if (!strcmp(key, "launches")) *value = net->launches;
    else if (!strcmp(key, "h2d_bytes")) *value = net->h2d_bytes;
    else if (!strcmp(key, "flat_floats")) *value = net->n_flat;
    else if (!strcmp(key, "ft_tiled")) *value = (net->fwd_tiled() ? 1 : 0) + (net->bwd_tiled() ? 2 : 0);
    else if (!strcmp(key, "slow_weights")) *value = net->S ? 1 : 0;
    else if (!strcmp(key, "optimiser_steps")) *value = net->opt_step;
    else return b200::fail(B200_ERR_ARG, "get_stat: unknown key '%s'", key);
    return 0;
}

int b200_net_get_activation(b200_net* net, int which, float* host, int64_t n) {
    if (!net || !host) return b200::fail(B200_ERR_ARG, "get_activation: null argument");
    const int64_t B = net->last_n;
    const float* src = nullptr;
    int64_t want = 0;
    switch (which) {
        case 0: src = net->x; want = B * net->D1(); break;
        case 1: src = net->u; want = net->d.pairwise ? B * 2 * net->d.ft_out : 0; break;
        case 2: src = net->dx; want = B * net->D1(); break;
        case 3: src = net->out; want = B; break;
        default: return b200::fail(B200_ERR_ARG, "get_activation: unknown buffer %d", which);
    }
    if (!src || want == 0) return b200::fail(B200_ERR_STATE, "get_activation: buffer %d is not used by this network", which);
    if (n != want) return b200::fail(B200_ERR_ARG, "get_activation: buffer %d holds %lld values, %lld asked", which, (long long)want, (long long)n);
    if (int rc = set_device(net)) return rc;
    CK(cudaStreamSynchronize(net->stream));
    CK(cudaMemcpy(host, src, n * sizeof(float), cudaMemcpyDeviceToHost));
    return 0;
}

}  // extern "C"
