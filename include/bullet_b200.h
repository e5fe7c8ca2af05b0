/*
 * bullet_b200 — C ABI of the B200-native NNUE training step.
 *
 * This header is the whole drop-in boundary: plain pointers and sizes, no C++ or
 * torch types.  A binding for bullet's Rust crates declares exactly these symbols
 * in an `extern "C"` block; each entry point names the piece of jw1912/bullet it
 * stands in for (paths relative to that project).
 *
 * Conventions
 *   - every function returns 0 on success, a negative B200_ERR_* otherwise;
 *     b200_last_error() then holds a message for the calling thread.  Nothing
 *     aborts, throws across the boundary, or traps on the device.
 *   - a b200_net is bound to one CUDA device and is not re-entrant; different
 *     nets (GPUs) may be driven from different host threads at the same time.
 *   - host pointers are borrowed for the duration of the call only.
 *   - weights are column-major `rows x cols` (docs/4-saved-networks.md:21-31):
 *     l0w[feature * H + row]; dense layer i: l{i}w[col * (O*M_i) + bucket*M_i + row].
 *   - there is no CPU fallback: without a usable CUDA device every entry point
 *     that needs one fails with B200_ERR_CUDA.
 */
#ifndef BULLET_B200_H
#define BULLET_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_ERR_ARG (-1)         /* bad argument, unknown tensor name, size mismatch   */
#define B200_ERR_STATE (-2)       /* call order violated (e.g. step on an empty slot)    */
#define B200_ERR_CUDA (-3)        /* a CUDA runtime call failed; message has the code    */
#define B200_ERR_DATA (-4)        /* batch data violates the declared input structure    */
#define B200_ERR_UNSUPPORTED (-5) /* network shape outside what the kernels implement    */

#define B200_ACT_NONE 0
#define B200_ACT_CRELU 1
#define B200_ACT_SCRELU 2

#define B200_KIND_WEIGHT 0
#define B200_KIND_MOMENTUM 1
#define B200_KIND_VELOCITY 2
#define B200_KIND_GRAD 3
#define B200_KIND_SLOW 4 /* Ranger's slow weights (only while a tensor uses Ranger) */

#define B200_NUM_SLOTS 3 /* staging slots for double/triple-buffered upload */

/* Feature-transformer kernel selection: b200_net_set_option "ft_mode" sets both passes,
 * "ft_fwd_mode" / "ft_bwd_mode" one of them */
#define B200_FT_AUTO 0
#define B200_FT_GATHER 1 /* row gather straight from the table in L2/HBM, global vector atomics */
#define B200_FT_TILED 2  /* table block staged in shared memory, positions grouped by block */

typedef struct b200_net b200_net;

/* The recognised form of the graph built by bullet's ModelBuilder closure
 * (examples/simple.rs:25-56, examples/progression/4_multi_layer.rs:66-87):
 * l0 affine on both sparse perspectives -> activation [-> pairwise_mul] ->
 * concat -> 1..3 dense affines, each followed by select(output bucket) and an
 * activation -> sigmoid -> squared error, summed over the batch. */
typedef struct b200_net_desc {
    int32_t n_inputs;        /* sparse inputs per perspective (SparseInputType::num_inputs)   */
    int32_t nnz;             /* index slots per position (SparseInputType::max_active), <= 64 */
    int32_t ft_out;          /* rows of l0 (hidden size H), multiple of 8                     */
    int32_t ft_act;          /* B200_ACT_CRELU or B200_ACT_SCRELU                             */
    int32_t pairwise;        /* 1: crelu then pairwise_mul (model/builder.rs:390-393)         */
    int32_t factoriser_rows; /* 0, or rows of l0f with l0w + l0f.repeat(n) as the table       */
    int32_t n_out_buckets;   /* OutputBuckets::BUCKETS                                        */
    int32_t n_dense;         /* 1..3                                                          */
    int32_t dense_out[3];    /* rows per bucket; <= 32; the last must be 1                    */
    int32_t dense_act[3];    /* activation after select; the last must be B200_ACT_NONE       */
    int32_t ft_block_rows;   /* >0 promises that the valid features of one perspective of one
                                position all fall in one aligned block of this many table rows
                                (768 for king-bucketed chess inputs); 0 promises nothing      */
    int32_t max_batch;       /* largest batch a slot will ever hold                           */
} b200_net_desc;

/* crates/trainer/src/optimiser/adam.rs:20-33 — same fields, same defaults. */
typedef struct b200_adamw_params {
    float decay, beta1, beta2, min_weight, max_weight;
} b200_adamw_params;

/* Device time of the phases of a step (milliseconds, CUDA events on the compute stream). */
typedef struct b200_timings {
    float ft_forward, dense_forward, dense_backward, ft_backward, factoriser_grad, optimiser, total;
    int32_t steps; /* complete steps averaged */
} b200_timings;

const char* b200_last_error(void);
int b200_version(void);

/* ---- life cycle.  Stands in for Device::new + Function::new/prealloc
 * (crates/gpu/src/function.rs:73,180) and Optimiser::new
 * (crates/trainer/src/optimiser.rs:98-133): allocates every buffer the step
 * needs, once.  `stream` is a cudaStream_t to run on, or NULL for a private one. */
int b200_net_create(int device, void* stream, const b200_net_desc* desc, b200_net** out);
int b200_net_destroy(b200_net* net);
/* Tuning switches (no counterpart in the reference; every one has a measured default):
 *   "ft_mode" / "ft_fwd_mode" / "ft_bwd_mode"  B200_FT_*; "ft_bwd_wide" 0 = two 512-thread backward CTAs per SM;
 *   "ft_once" 0 = table rows and activations through ordinary (L1-allocating) loads;
 *   "ft_bwd_grab" rows a warp of the tiled backward takes from the row counter at a time (0 = by block size);
 *   "exchange_bulk" 1 = the peer exchange moves gradients and weights with bulk asynchronous copies;
 *   "overlap_ctas", "overlap_mode", "exchange_ctas", "exchange_wait_ms", "exchange_step", "manual_grad_zero": see the
 *   data-parallel entry points below. */
int b200_net_set_option(b200_net* net, const char* key, int64_t value);

/* ---- tensors by reference id ("l0w","l0b","l0f","l1w",...).  Stands in for
 * Optimiser::load_weights_from_host / Buffer::to_host
 * (crates/trainer/src/optimiser.rs:208-216).  `kind` selects weight, momentum,
 * velocity or (read-only) the batch-summed gradient of the last backward pass. */
int b200_net_tensor_size(b200_net* net, const char* name, int64_t* n);
int b200_net_set_tensor(b200_net* net, const char* name, int kind, const float* host, int64_t n);
int b200_net_get_tensor(b200_net* net, const char* name, int kind, float* host, int64_t n);
/* Optimiser::set_params_for_weight (crates/trainer/src/optimiser.rs:204-206); NULL name = all. */
int b200_net_set_adamw(b200_net* net, const char* name, const b200_adamw_params* params);

/* The other update rules of the reference, per tensor or (NULL name) for all.  RAdam
 * (crates/trainer/src/optimiser/radam.rs:20-52,295-314): rectified Adam; the host evaluates the step size and
 * whether the second moment divides the update from the step count, the kernel is AdamW's with those two
 * applied; defaults beta 0.9 / 0.999, threshold 5, decay 0, no clipping (pass -FLT_MAX / FLT_MAX).  Ranger
 * (ranger.rs:45-167): RAdam plus lookahead: every k-th step w = alpha * w + (1 - alpha) * slow and slow = w,
 * the slow weights starting at zero as in the reference; defaults decay 0.01, beta 0.99 / 0.999, clip +-1.98,
 * alpha 0.5, k 6.  Setting a rule resets the step count.  The slow weights are tensor kind B200_KIND_SLOW
 * and travel in `slow.bin` of a checkpoint. */
#define B200_OPT_ADAMW 0
#define B200_OPT_RADAM 1
#define B200_OPT_RANGER 2
typedef struct b200_optimiser_params {
    int32_t kind; /* B200_OPT_* */
    float decay, beta1, beta2, min_weight, max_weight;
    float n_sma_threshold; /* RAdam, Ranger */
    float alpha;           /* Ranger */
    int32_t k;             /* Ranger */
} b200_optimiser_params;
int b200_net_set_optimiser(b200_net* net, const char* name, const b200_optimiser_params* params);

/* ---- batch upload.  Stands in for PreparedBatchHost::copy_to_device_async
 * (crates/trainer/src/run/dataloader.rs:41-61): takes the mapper's output in
 * the reference layout (i32 [n][nnz] per perspective, -1 in unused slots, i32
 * bucket and f32 target per position; crates/bullet_lib/src/value.rs:77-117),
 * packs it to u16 in pinned memory and starts one asynchronous copy.  Blocks
 * only while `slot` is still being read by an earlier step. */
int b200_batch_upload(b200_net* net, int slot, const int32_t* stm, const int32_t* nstm, const int32_t* buckets,
                      const float* targets, int32_t n);
/* The same from raw 32-byte position records: the featuriser (`game`), MaterialCount<n_out_buckets>
 * (crates/bullet_lib/src/game/outputs.rs:24-31; networks with output buckets take chess records) and
 * the target blend of ValueTrainerState::make_mapper (crates/bullet_lib/src/value.rs:77-117) run on
 * all host cores and write the packed lists straight into the pinned staging block.  `layout32` is the
 * king-bucket layout of ChessBucketsMirrored (32 entries), NULL for the other games. */
#define B200_GAME_CHESS768 0
#define B200_GAME_CHESS_BUCKETS_MIRRORED 1
#define B200_GAME_ATAXX147 2
int b200_batch_upload_records(b200_net* net, int slot, const void* records, int32_t n, int32_t game, const int32_t* layout32,
                              float scale, float blend);

/* The same with the preparation on the DEVICE: the raw records (32 bytes per position) are copied and a kernel runs
 * the featuriser, the output bucket and the target blend; two more group the positions by output bucket and the
 * (position, perspective) pairs by table row block, in the same stable order the host path produces.  The slot
 * ends up bit-identical to b200_batch_upload_records' (lists, buckets, targets, both orders), so training results
 * are identical too.  The call waits once for two small histograms (it needs them to size the step's launches);
 * everything runs on the library's copy stream, beside a step that is still computing.  What it replaces in the
 * reference: the per-position mapper closure of ValueTrainerState::make_mapper (crates/bullet_lib/src/value.rs:77-117)
 * run by the loader threads (crates/trainer/src/model/inputs.rs:86-109) plus the copy of its five arrays.
 * At most 256 row blocks and 256 output buckets. */
int b200_batch_upload_records_gpu(b200_net* net, int slot, const void* records, int32_t n, int32_t game, const int32_t* layout32,
                                  float scale, float blend);

/* Debug/inspection: copies what a slot holds on the device to the host (any pointer may be NULL): the packed index
 * lists [n][nnz], buckets [n], targets [n], the positions grouped by output bucket [n] and the (position,
 * perspective) pairs (id = 2 * position + perspective) grouped by row block [2n]; *n = positions in the slot. */
int b200_slot_read(b200_net* net, int slot, uint16_t* stm, uint16_t* nstm, int32_t* buckets, float* targets, int32_t* order,
                   int32_t* pair_order, int32_t* n);

/* ---- the step.  b200_step = Function::execute on the backward graph followed by
 * Optimiser::update (crates/trainer/src/run.rs:185-192).  The split form lets a
 * data-parallel host all-reduce the flat gradient buffer between the halves:
 * gradients are batch SUMS and `grad_factor` (1/global batch) is applied in the
 * update, as in crates/trainer/src/run.rs:130-131.  All calls only enqueue. */
int b200_step(b200_net* net, int slot, float lr, float grad_factor);
int b200_backward(b200_net* net, int slot);
int b200_update(b200_net* net, float lr, float grad_factor);
/* Device address and length (floats) of the flat gradient buffer; its FIRST
 * element is the summed loss, so one all-reduce carries both. */
int b200_grad_buffer(b200_net* net, void** device_ptr, int64_t* n_floats);

/* The data-parallel update over peer memory, one process per GPU of one box (new; the reference is
 * single-GPU).  b200_exchange_export writes three CUDA IPC handles (gradient buffer, parameter buffer,
 * fence counters; B200_EXCHANGE_HANDLE_BYTES bytes); the host gathers the handles of all ranks, in
 * rank order, and hands them to b200_exchange_import, which maps every peer's buffers (at most 8
 * ranks; the flat buffer must split into world x 4 floats).  b200_update_exchange then replaces the
 * all-reduce + b200_update pair: ONE kernel sums this rank's 1/world share of the gradients over all
 * ranks with peer loads, applies AdamW+clip to it and stores the new weights into every rank's
 * parameter buffer (reduce-scatter + AdamW + all-gather).  Momentum and velocity stay sharded.
 * It fences itself: small kernels around it exchange counters with the peers (release stores over
 * NVLink, bounded local polling), so every rank's b200_backward is complete before its gradients are
 * read and every rank's kernel has finished before anyone goes on.  All ranks must call it the same
 * number of times.  A peer that does not arrive within about four seconds ("exchange_wait_ms") makes the wait
 * give up: the kernel returns without touching parameters, optimiser state or any peer's memory, raises a word
 * on every rank, the stream carries on, and b200_loss reports B200_ERR_STATE for that step on every rank (the
 * rank that waited also says which rank and which fence were missing).  b200_update_end follows as usual. */
#define B200_EXCHANGE_HANDLE_BYTES 192
int b200_exchange_export(b200_net* net, void* handles, int64_t bytes);
int b200_exchange_import(b200_net* net, int rank, int world, const void* handles, int64_t bytes);
int b200_update_exchange(b200_net* net, float lr, float grad_factor);
/* One whole data-parallel step (= b200_backward + b200_update_exchange + b200_update_end) with the exchange
 * hidden under the feature-transformer backward.  The backward's work is ordered by table row block (king
 * bucket) and announces every finished block to all ranks; the exchange runs at the same time on a few SMs
 * of its own ("overlap_ctas", default 20) and takes the blocks as they arrive: peer loads of this rank's 1/world
 * share, AdamW, peer stores of the new weights.  The factoriser gradient is formed from the reduced blocks by
 * the share's owner; bias, dense layers and loss are reduced by every rank for itself after the backward.
 * Needs the tiled backward, row blocks that split over world x 4 floats, and a factoriser (if any) of exactly
 * one row block; otherwise B200_ERR_UNSUPPORTED, and the caller uses the calls above.  Momentum and velocity of
 * l0w and l0f stay sharded (share r of every block with rank r), those of the small tensors are complete on
 * every rank.  The gradient of l0f is not formed in the gradient buffer.  Fences and time-outs as above.
 * b200_net_set_option("exchange_step", n) resynchronises the ranks' step counters after a failed step. */
int b200_step_exchange(b200_net* net, int slot, float lr, float grad_factor);
/* The same kernel on any 4-float-aligned range, on `stream` (a cudaStream_t, NULL = the net's), for a
 * host that exchanges slice by slice beside the backward and the next forward.  gather = 1: the range is
 * this rank's own share of a slice; the new weights are stored to every rank.  gather = 0: every rank
 * runs the same range and keeps the result to itself (the small tensors, which all ranks need at once).
 * This form does NOT fence itself: the caller orders every launch between two cross-rank barriers on
 * `stream` (any tiny collective).  b200_grad_zero_range clears a range of the gradient buffer
 * on the net's stream; with b200_net_set_option("manual_grad_zero", 1) the library no longer clears the
 * whole buffer at the start of a step, because peers may still be reading parts of it. */
int b200_update_exchange_range(b200_net* net, float lr, float grad_factor, int64_t first_float, int64_t n_floats, int gather,
                               void* stream);
int b200_grad_zero_range(b200_net* net, int64_t first_float, int64_t n_floats);

/* The training forward pass in pieces, for a host that overlaps an exchange of freshly updated
 * weights with it (a sharded optimiser gathers l0w slice by slice): b200_forward_begin waits for
 * the batch, zeroes the gradients and builds the row lists; b200_forward_ft runs the feature
 * transformer for the part-th of n_parts equal runs of table row blocks, in order, reading only
 * that run's rows of l0w (plus l0b and l0f); b200_backward_begin on the same slot then carries on
 * from the dense layers.  Without these calls b200_backward_begin runs the whole forward itself. */
int b200_forward_begin(b200_net* net, int slot);
int b200_forward_ft(b200_net* net, int slot, int part, int n_parts);
/* First float of a tensor inside the flat buffers (b200_flat_buffer); tensors lie in name order
 * with l0w last, each starting on a 256-byte boundary. */
int b200_net_tensor_offset(b200_net* net, const char* name, int64_t* first_float);

/* The same step in phases, for a host that overlaps the gradient exchange with the backward
 * pass.  b200_backward = begin + ft(0, 1) + end; b200_update = update_range(whole buffer) + end.
 *   b200_backward_begin  zeroes the gradients, runs the forward, the loss and the backward
 *                        down to the gradient at the feature transformer's output;
 *   b200_backward_ft     feature-transformer backward for the part-th of n_parts equal runs of
 *                        table row blocks, in order (n_parts > 1 needs the tiled backward and
 *                        must divide the number of row blocks); when it returns, part's slice
 *                        of the l0w gradient is complete on the stream and may be all-reduced;
 *   b200_backward_end    the dense layers' weight gradients; afterwards the head is complete;
 *   b200_grad_part       flat range [first, first + count) of the gradient buffer that part
 *                        covers; part == n_parts names the head: the loss and every tensor
 *                        except l0w;
 *   b200_update_range    AdamW+clip on a 4-float-aligned range of the flat buffer;
 *   b200_update_end      after all ranges: rebuilds the derived tables, queues the loss read. */
int b200_backward_begin(b200_net* net, int slot);
int b200_backward_ft(b200_net* net, int slot, int part, int n_parts);
int b200_backward_end(b200_net* net, int slot);
int b200_grad_part(b200_net* net, int part, int n_parts, int64_t* first_float, int64_t* n_floats);
int b200_update_range(b200_net* net, float lr, float grad_factor, int64_t first_float, int64_t n_floats);
int b200_update_end(b200_net* net);
/* Device address and length of one of the four flat buffers (B200_KIND_*), all of the same
 * layout and length (a multiple of 1024 floats); float 0 is used only in the gradient buffer.
 * A data-parallel host that shards the optimiser reduce-scatters the gradients, runs
 * b200_update_range on its own shard only, and all-gathers the weight buffer before
 * b200_update_end; momentum and velocity then stay sharded until it gathers them too. */
int b200_flat_buffer(b200_net* net, int kind, void** device_ptr, int64_t* n_floats);
/* Summed loss of the most recent update/step (run.rs:212-221); waits for it. */
int b200_loss(b200_net* net, float* loss_sum);
/* The same for an earlier update: steps_back = 1 is the update before the most recent one (at
 * most 2).  Reading step n-1's loss right after enqueuing step n keeps the GPU busy while the
 * host waits, where b200_loss would drain it every step. */
int b200_loss_of(b200_net* net, int steps_back, float* loss_sum);
/* Forward only: network output per position (ModelEvaluator, crates/trainer/src/model/evaluator.rs:22-81). */
int b200_forward(b200_net* net, int slot, float* out_host);
int b200_sync(b200_net* net);
/* Average device time per phase over the complete steps (backward + update) enqueued since
 * the previous call, at most the last 256; waits for them.  ft_forward and ft_backward each
 * span exactly one kernel launch. */
int b200_get_timings(b200_net* net, b200_timings* out);
/* Counters: "launches" (kernels launched so far), "h2d_bytes" (batch bytes copied so far),
 * "flat_floats" (length of the flat parameter buffer), "ft_tiled" (bit 0: the forward runs the
 * tiled kernel, bit 1: the backward does). */
int b200_net_get_stat(b200_net* net, const char* key, int64_t* value);
/* Debug/inspection: copy an internal activation buffer of the last pass to the host.
 * which: 0 = dense-stack input x [n][D1], 1 = pairwise crelu outputs u [n][2][H],
 *        2 = gradient at x [n][D1], 3 = network outputs [n]. */
int b200_net_get_activation(b200_net* net, int which, float* host, int64_t n);

/* ---- checkpoints in the reference's on-disk format: `dir`/weights.bin, momentum.bin and
 * velocity.bin, each a sequence of records (ASCII id, '\n', u64 LE count, f32 LE values) in name
 * order, as Optimiser::write_to_checkpoint / load_from_checkpoint read and write them
 * (crates/trainer/src/optimiser.rs:218-236, crates/trainer/src/model/weights.rs:404-467).
 * The directory must exist; in the reference it is `<checkpoint>/optimiser_state`. */
int b200_checkpoint_save(b200_net* net, const char* dir);
int b200_checkpoint_load(b200_net* net, const char* dir);

/* ---- network export in the reference's SavedFormat scheme
 * (crates/trainer/src/model/weights.rs:183-335; ModelWeights::to_quantised_buffer weights.rs:158-177;
 * save_quantised / save_unquantised crates/bullet_lib/src/value/save.rs:45-88).
 * One entry is custom bytes (id == NULL) or a weight id whose values pass, in this order, through
 * the optional factoriser merge (the transform of examples/progression/3_input_buckets.rs:46-53:
 * value + l0f repeated over the input buckets), the optional transpose (weights.rs:254-269, using
 * the weight's column-major shape) and quantisation: round-half-away-from-zero or truncation of
 * f64(multiplier) * f64(value), stored little-endian.  A value that does not fit its target type
 * fails the export with B200_ERR_DATA ("Failed quantisation from f32 to i16!"); nothing is clamped. */
#define B200_QUANT_FLOAT 0
#define B200_QUANT_I8 1
#define B200_QUANT_I16 2
#define B200_QUANT_I32 3
typedef struct b200_saved_format {
    const char* id;           /* weight to write, or NULL for custom bytes                        */
    const void* custom;       /* id == NULL: bytes copied as they are (header, padding, ...)      */
    int64_t custom_len;
    int32_t quant;            /* B200_QUANT_*                                                     */
    int32_t multiplier;       /* i16 range for the i8 and i16 targets, as in the reference        */
    int32_t round;            /* 1: round half away from zero; 0: truncate                        */
    int32_t transpose;        /* 1: write the transposed matrix                                   */
    int32_t merge_factoriser; /* 1: add l0f, repeated over the input buckets, before the rest     */
} b200_saved_format;
/* Shape(rows, cols) of a weight, column-major as in the reference (l0w: ft_out x n_inputs). */
int b200_net_tensor_shape(b200_net* net, const char* name, int64_t* rows, int64_t* cols);
/* QuantTarget::quantise (weights.rs:281-331) on host values; `out` holds n * b200_quant_size(quant) bytes. */
int64_t b200_quant_size(int32_t quant);
int b200_quantise(const float* values, int64_t n, int32_t quant, int32_t multiplier, int32_t round, void* out);
/* SavedFormat::transpose_impl (weights.rs:254-269): out[cols * i + j] = in[rows * j + i]. */
int b200_transpose(const float* in, int64_t rows, int64_t cols, float* out);
/* to_quantised_buffer: size of, and the bytes of, the concatenated entries; `pad` pads to 64 bytes. */
int b200_saved_format_size(b200_net* net, const b200_saved_format* fmt, int32_t n_fmt, int32_t pad, int64_t* bytes);
int b200_saved_format_write(b200_net* net, const b200_saved_format* fmt, int32_t n_fmt, int32_t pad, void* out, int64_t out_bytes);
/* save_quantised (padded) and save_unquantised (the named weights as raw f32, no transforms) to a file;
 * in the reference these are `<checkpoint>/quantised.bin` and `<checkpoint>/raw.bin`. */
int b200_save_quantised(b200_net* net, const b200_saved_format* fmt, int32_t n_fmt, const char* path);
int b200_save_unquantised(b200_net* net, const b200_saved_format* fmt, int32_t n_fmt, const char* path);

/* ---- operator level: the feature-transformer forward on caller-owned DEVICE memory, without a
 * b200_net.  For both perspectives of n positions: the sparse affine of SparseMatmul::evaluate
 * (crates/compiler/src/tensor/operation/linear/sparse.rs:86-119), the bias
 * (crates/compiler/src/model/builder.rs:145-147), the activation (autograd/dfo.rs:47-88), the
 * optional pairwise product (model/builder.rs:390-393) and the stm|nstm concat (builder.rs:375-388).
 * Needs the block structure (ft_block_rows > 0 dividing n_inputs) and ft_out a multiple of 64.
 * Groups the positions by row block on the device, in scratch memory taken from cudaMalloc for
 * the duration of the call; runs on `stream` (NULL = default stream) and waits for it. */
typedef struct b200_ft_op {
    int32_t n_inputs, nnz, ft_out, ft_act, pairwise, ft_block_rows;
    int32_t n;                /* positions */
    const float* table;       /* [n_inputs][ft_out] weights, l0w layout (plus the factoriser if any) */
    const float* bias;        /* [ft_out] */
    const uint16_t* idx_stm;  /* [n][nnz] packed indices, 0xFFFF = empty (b200_pack_indices_u16) */
    const uint16_t* idx_nstm;
    float* x;                 /* out: [n][2*ft_out], or [n][ft_out] with pairwise */
    float* u;                 /* out, pairwise only: crelu outputs [n][2][ft_out] */
} b200_ft_op;
int b200_op_ft_forward(int device, void* stream, const b200_ft_op* op);

/* The same operator for callers that must not allocate.  (No counterpart in the reference: its
 * runtime allocates every buffer through its own Buffer type.)  Use it from code that runs
 * beside a training loop on the same GPU, or after all device memory has been handed out:
 * cudaMalloc/cudaFree stall every stream of the device, and a fixed memory budget leaves
 * nothing to allocate.  The grouping scratch is a fixed array inside the library (about 4.6 MB
 * on every GPU that loads it), so n is limited to B200_OP_NOALLOC_MAX_POSITIONS (half of it
 * when nnz > 32); larger n is refused with B200_ERR_ARG.  No cudaMalloc, cudaFree or other allocating call is made.
 * The first call on a device looks up the array's address: make it before any stream capture.
 * Calls on one device share the array, so calls whose GPU work overlaps race: serialise them. */
#define B200_OP_NOALLOC_MAX_POSITIONS 16384
int b200_op_ft_forward_noalloc(int device, void* stream, const b200_ft_op* op);

/* ---- bandwidth probes: the measured denominators for kernels whose table stays in L2.  kind 0: every SM
 * reads a buffer of `bytes` bytes `reps` times with 16-byte loads (a buffer well below the L2 size measures L2,
 * one far above it measures HBM); kind 1: 16-byte vector reductions (red.global.add.v4.f32) into it; kinds 2
 * and 3: reductions of 4 and 8 bytes per lane, a warp covering one contiguous run.  Allocates
 * the buffer for the duration of the call and returns GB/s of the best of three timed rounds.  (No counterpart
 * in the reference.) */
int b200_probe_bandwidth(int device, int kind, int64_t bytes, int reps, double* gb_per_s);

/* ---- host featurisers (no device needed).  Records are the 32-byte layouts of
 * bulletformat's ChessBoard / AtaxxBoard as restated in examples/tests/test4.rs:8-36
 * and examples/ataxx.rs:8-31.  Outputs use the mapper's layout with -1 in every
 * unused slot.  Return the largest feature count seen. */
int b200_map_chess768(const void* records, int32_t n, int32_t* stm, int32_t* nstm, int32_t nnz);
/* ChessBucketsMirrored::{new,map_features} (crates/bullet_lib/src/game/inputs/chess_buckets.rs:57-88) */
int b200_map_chess_buckets_mirrored(const void* records, int32_t n, const int32_t* layout32, int32_t* stm,
                                    int32_t* nstm, int32_t nnz);
/* Ataxx147::map_features (crates/bullet_lib/src/game/inputs/ataxx147.rs:18-27) */
int b200_map_ataxx147(const void* records, int32_t n, int32_t* stm, int32_t* nstm, int32_t nnz);
/* MaterialCount<N>::bucket (crates/bullet_lib/src/game/outputs.rs:24-31) */
int b200_material_count(const void* records, int32_t n, int32_t n_buckets, int32_t* out);
/* target = blend*result/2 + (1-blend)*sigmoid(score/scale) (crates/bullet_lib/src/value.rs:103-115).
 * The score is multiplied by the fp32 reciprocal of `scale`, as value.rs:69,108 does (`rscale * score`), for
 * every game, ataxx records included.  The raw-API ataxx example divides instead
 * (examples/ataxx.rs:58: exp(-score / 400.0)); 1/400 is not exact in fp32, so a target made this way can differ
 * from that example's by one unit in the last place. */
int b200_make_targets(const void* records, int32_t n, float scale, float blend, float* out);
/* Host threads (OpenMP) used by the featurisers and by the packing inside the uploads; n < 1 = one per
 * core.  One-process-per-GPU launchers often set OMP_NUM_THREADS=1, which leaves the packing serial. */
int b200_set_host_threads(int32_t n);
/* The packed index format of a staging slot: u16 per slot, 0xFFFF for "no feature". */
int b200_pack_indices_u16(const int32_t* idx, int64_t count, uint16_t* out);
int b200_unpack_indices_u16(const uint16_t* packed, int64_t count, int32_t* out);

#ifdef __cplusplus
}
#endif
#endif /* BULLET_B200_H */
