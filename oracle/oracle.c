/*
 * CPU oracle for the NNUE training step.  TEST INFRASTRUCTURE ONLY: the shipped
 * library never links, loads or calls this file; it exists so that the CUDA
 * path can be checked against an independent restatement of the reference's
 * CPU graph interpreter, and so that the benchmark has a CPU figure to print.
 *
 * Every function restates, in plain C and in the reference's own evaluation
 * order, one piece of jw1912/bullet (paths are relative to that project):
 *
 *   sparse affine forward      crates/compiler/src/tensor/operation/linear/sparse.rs:86-119
 *   sparse affine backward     crates/compiler/src/tensor/operation/linear/sparse.rs:151-187,253-271
 *   dense matmul               crates/compiler/src/tensor/operation/linear/matmul.rs:62-93
 *   select / select-pad        crates/compiler/src/tensor/operation/index/select.rs:12-26,93-110
 *   reduce / broadcast         crates/compiler/src/tensor/operation/linear/reduce.rs:96-120,
 *                              crates/compiler/src/tensor/operation/index/broadcast.rs:66-80
 *   activations + derivatives  crates/compiler/src/tensor/operation/autograd/dfo.rs:47-119
 *   AdamW + clip               crates/trainer/src/optimiser/adam.rs:35-52,117-136
 *   featurisers                crates/bullet_lib/src/game/inputs/{chess768,chess_buckets,ataxx147}.rs,
 *                              crates/bullet_lib/src/game/outputs.rs:24-31
 *   batch mapper               crates/bullet_lib/src/value.rs:77-117
 *   record iteration           examples/tests/test4.rs:8-36, examples/ataxx.rs:8-31
 *
 * Parity pins: the op-level functions are checked against the reference's own
 * unit-test vectors (sparse.rs:286-313, matmul.rs:133-174, select.rs:172-222,
 * reduce.rs:201-244, broadcast.rs tests); AdamW, the featurisers, the mapper
 * and the activation derivatives have no test in the reference, so for those
 * parity is unpinned and rests on the cited source text alone.
 *
 * Arithmetic type: `real` is float (REAL_IS_DOUBLE undefined) or double (the
 * arbiter build).  Compile with -ffp-contract=off so a*b+c is two roundings,
 * as in the reference's Rust.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#ifdef REAL_IS_DOUBLE
typedef double real;
#define R_EXP exp
#define R_SQRT sqrt
#else
typedef float real;
#define R_EXP expf
#define R_SQRT sqrtf
#endif

int orc_real_bytes(void) { return (int)sizeof(real); }

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ ops */

/* sparse.rs:86-119.  W is column-major with `stride` floats per input column;
 * out[b*rows+r] = sum over valid slots, in slot order, starting from 0. */
void orc_sparse_matmul(const real* W, const int32_t* idx, real* out, int batch, int rows, int cols,
                       int stride, int offset, int nnz) {
    for (int b = 0; b < batch; b++)
        for (int r = 0; r < rows; r++) {
            real sum = 0;
            for (int n = 0; n < nnz; n++) {
                int32_t j = idx[(size_t)nnz * b + n];
                if (j >= 0 && j < cols) sum = sum + W[(size_t)stride * j + offset + r];
            }
            out[(size_t)rows * b + r] = sum;
        }
}

/* sparse.rs:151-187: zero the table, then add g[b,r] once per valid slot. */
void orc_sparse_matmul_bwd(const real* g, const int32_t* idx, real* out, int batch, int rows, int cols,
                           int stride, int offset, int nnz) {
    memset(out, 0, sizeof(real) * (size_t)stride * cols);
    for (int b = 0; b < batch; b++)
        for (int r = 0; r < rows; r++)
            for (int n = 0; n < nnz; n++) {
                int32_t j = idx[(size_t)nnz * b + n];
                if (j >= 0 && j < cols) {
                    size_t at = (size_t)stride * j + offset + r;
                    out[at] = g[(size_t)rows * b + r] + out[at];
                }
            }
}

/* sparse.rs:253-271: every (grad, indices) pair fills its own zeroed table,
 * the tables are then added to the output one after the other. */
void orc_sparse_matmul_bwd_multi(int npairs, const real* const* g, const int32_t* const* idx, const int* offsets,
                                 real* out, int batch, int rows, int cols, int stride, int nnz) {
    size_t n = (size_t)stride * cols;
    real* tmp = (real*)malloc(sizeof(real) * n);
    memset(out, 0, sizeof(real) * n);
    for (int p = 0; p < npairs; p++) {
        orc_sparse_matmul_bwd(g[p], idx[p], tmp, batch, rows, cols, stride, offsets[p], nnz);
        for (size_t i = 0; i < n; i++) out[i] = out[i] + tmp[i];
    }
    free(tmp);
}

/* matmul.rs:62-93, generic over element type through two instantiations. */
#define ORC_MATMUL(NAME, T)                                                                                   \
    void NAME(const T* l, const T* r, T* o, int b, int m, int n, int k, int lhs_col_mjr, int rhs_col_mjr) {   \
        for (int bi = 0; bi < b; bi++)                                                                        \
            for (int ki = 0; ki < k; ki++)                                                                    \
                for (int mi = 0; mi < m; mi++) {                                                              \
                    T sum = 0;                                                                                \
                    for (int ni = 0; ni < n; ni++) {                                                          \
                        size_t a = (size_t)m * n * bi + (lhs_col_mjr ? m * ni + mi : n * mi + ni);            \
                        size_t c = (size_t)n * k * bi + (rhs_col_mjr ? n * ki + ni : k * ni + ki);            \
                        T prod = l[a] * r[c];                                                                 \
                        sum = sum + prod;                                                                     \
                    }                                                                                         \
                    o[(size_t)m * k * bi + m * ki + mi] = sum;                                                \
                }                                                                                             \
    }
ORC_MATMUL(orc_matmul, real)
ORC_MATMUL(orc_matmul_i32, int32_t)

/* select.rs:12-26 */
#define ORC_SELECT(NAME, T)                                                                    \
    void NAME(const T* in, const int32_t* indices, T* out, int batch, int inner, int divisor) { \
        int sub = inner / divisor;                                                             \
        for (int o = 0; o < batch; o++)                                                        \
            memcpy(out + (size_t)sub * o, in + (size_t)inner * o + (size_t)sub * indices[o],   \
                   sizeof(T) * sub);                                                           \
    }
ORC_SELECT(orc_select, real)
ORC_SELECT(orc_select_i32, int32_t)

/* select.rs:93-110 */
#define ORC_SELECT_PAD(NAME, T)                                                                \
    void NAME(const T* in, const int32_t* indices, T* out, int batch, int inner, int divisor) { \
        int sub = inner / divisor;                                                             \
        for (int o = 0; o < batch; o++) {                                                      \
            for (int i = 0; i < inner; i++) out[(size_t)inner * o + i] = 0;                    \
            memcpy(out + (size_t)inner * o + (size_t)sub * indices[o], in + (size_t)sub * o,   \
                   sizeof(T) * sub);                                                           \
        }                                                                                      \
    }
ORC_SELECT_PAD(orc_select_pad, real)
ORC_SELECT_PAD(orc_select_pad_i32, int32_t)

/* reduce.rs:96-120 (sum only): acc starts from element 0, adds k = 1..dimen. */
#define ORC_REDUCE(NAME, T)                                                        \
    void NAME(const T* in, T* out, int outer, int dimen, int inner) {              \
        size_t os = (size_t)dimen * inner;                                         \
        for (int i = 0; i < outer; i++)                                            \
            for (int j = 0; j < inner; j++) {                                      \
                T acc = in[i * os + j];                                            \
                for (int k = 1; k < dimen; k++) acc = acc + in[i * os + (size_t)k * inner + j]; \
                out[(size_t)i * inner + j] = acc;                                  \
            }                                                                      \
    }
ORC_REDUCE(orc_reduce_sum, real)
ORC_REDUCE(orc_reduce_sum_i32, int32_t)

/* broadcast.rs:66-80 */
#define ORC_BROADCAST(NAME, T)                                                     \
    void NAME(const T* in, T* out, int outer, int inner, int repeats) {            \
        for (int i = 0; i < outer; i++)                                            \
            for (int j = 0; j < inner; j++) {                                      \
                size_t ld = (size_t)inner * i;                                     \
                for (int r = 0; r < repeats; r++) out[ld * repeats + (size_t)inner * r + j] = in[ld + j]; \
            }                                                                      \
    }
ORC_BROADCAST(orc_broadcast, real)
ORC_BROADCAST(orc_broadcast_i32, int32_t)

/* dfo.rs:47-119.  act: 0 identity, 1 crelu, 2 screlu. */
static inline real act_fwd(int act, real x) {
    if (act == 0) return x;
    real c = x > 0 ? x : 0;
    c = c < 1 ? c : 1;
    return act == 2 ? c * c : c;
}
/* derivative as a function of the OUTPUT y (strict inequalities on both sides) */
static inline real act_bwd_from_output(int act, real y) {
    if (act == 0) return 1;
    real pos = y > 0 ? 1 : 0;
    real lt1 = ((real)1 - y) > 0 ? 1 : 0;
    real c = pos * lt1;
    if (act == 1) return c;
    real half = c * R_SQRT(y);
    return half + half;
}
void orc_act_forward(int act, const real* x, real* y, int n) {
    for (int i = 0; i < n; i++) y[i] = act_fwd(act, x[i]);
}
void orc_act_backward(int act, const real* y, const real* gy, real* gx, int n) {
    for (int i = 0; i < n; i++) gx[i] = gy[i] * act_bwd_from_output(act, y[i]);
}
static inline real sigmoid_r(real x) { return (real)1 / ((real)1 + R_EXP(-x)); }

/* adam.rs:35-52 with adj*grad as the gradient (adam.rs:121-131). */
void orc_adamw(real* p, real* m, real* v, const real* grad, size_t n, real adj, real rate, real decay, real beta1,
               real beta2, real wmin, real wmax) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        real g = adj * grad[i];
        real pi = p[i];
        pi = pi * ((real)1 - decay * rate);
        m[i] = beta1 * m[i] + ((real)1 - beta1) * g;
        v[i] = beta2 * v[i] + ((real)1 - beta2) * g * g;
        real val = m[i] / (R_SQRT(v[i]) + (real)0.00000001f);
        pi = pi - rate * val;
        pi = pi > wmin ? pi : wmin;
        pi = pi < wmax ? pi : wmax;
        p[i] = pi;
    }
}

/* radam.rs:35-52 with adj*grad as the gradient.  `rate` is the learning rate already multiplied by the step
 * size that RAdam::update computes on the host (orc_radam_step below); `use_denom` is its n_sma test. */
void orc_radam(real* p, real* m, real* v, const real* grad, size_t n, real adj, real rate, int use_denom, real decay,
               real beta1, real beta2, real wmin, real wmax) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        real g = adj * grad[i];
        real pi = p[i];
        pi = pi * ((real)1 - decay * rate);
        m[i] = beta1 * m[i] + ((real)1 - beta1) * g;
        v[i] = beta2 * v[i] + ((real)1 - beta2) * g * g;
        real val = m[i];
        if (use_denom) val = val / (R_SQRT(v[i]) + (real)0.00000001f);
        pi = pi - rate * val;
        pi = pi > wmin ? pi : wmin;
        pi = pi < wmax ? pi : wmax;
        p[i] = pi;
    }
}

/* radam.rs:295-314: always in f32, as the reference's host code; returns the step size, *use_denom the flag. */
float orc_radam_step(int step_count, float beta1, float beta2, float n_sma_threshold, int* use_denom) {
    const float step = (float)step_count;
    const float beta2_t = powf(beta2, step);
    const float n_sma_max = 2.0f / (1.0f - beta2) - 1.0f;
    const float n_sma = n_sma_max - 2.0f * step * beta2_t / (1.0f - beta2_t);
    const float denom = 1.0f - powf(beta1, step);
    *use_denom = n_sma > n_sma_threshold;
    if (*use_denom) {
        const float p1 = (n_sma - 4.0f) / (n_sma_max - 4.0f);
        const float p2 = (n_sma - 2.0f) / n_sma;
        const float p3 = n_sma_max / (n_sma_max - 2.0f);
        return sqrtf((1.0f - beta2_t) * p1 * p2 * p3) / denom;
    }
    return 1.0f / denom;
}

/* ranger.rs:23-43: new = alpha * w + (1 - alpha) * slow, written to both. */
void orc_lookahead(real* w, real* slow, size_t n, real alpha) {
    const real one_minus = (real)((float)1 - (float)alpha);
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) {
        real lhs = alpha * w[i];
        real rhs = one_minus * slow[i];
        real nw = lhs + rhs;
        w[i] = nw;
        slow[i] = nw;
    }
}

/* ------------------------------------------------------------ featurisers */

typedef struct {
    uint64_t occ;
    uint8_t pcs[16];
    int16_t score;
    uint8_t result;
    uint8_t ksq;
    uint8_t opp_ksq;
    uint8_t extra[3];
} orc_chess_board; /* examples/tests/test4.rs:8-18 */

typedef struct {
    uint64_t bbs[3];
    int16_t score;
    uint8_t result;
    uint8_t origstm;
    uint16_t fullm;
    uint8_t halfm;
    uint8_t extra;
} orc_ataxx_board; /* examples/ataxx.rs:8-18 */

/* chess768.rs:20-30 over the piece iteration of test4.rs:23-36.
 * mode 0: plain 768; mode 1: mirrored king buckets (chess_buckets.rs:57-66,82-88)
 * with `layout32` the 32-entry half-board bucket table.  Writes the reference
 * layout: features in iteration order, then -1 in EVERY unused slot (the
 * reference writes one terminator and leaves the rest to a recycled buffer). */
static int chess_features(const orc_chess_board* pos, int mode, const int32_t* layout32, int32_t* stm, int32_t* ntm,
                          int nnz) {
    int expanded[64];
    int sflip = 0, nflip = 0, sb = 0, nb = 0;
    if (mode == 1) {
        static const int fold[8] = {0, 1, 2, 3, 3, 2, 1, 0};
        for (int i = 0; i < 64; i++) expanded[i] = layout32[(i / 8) * 4 + fold[i % 8]];
        sflip = (pos->ksq % 8 > 3) ? 7 : 0;
        nflip = (pos->opp_ksq % 8 > 3) ? 7 : 0;
        sb = 768 * expanded[pos->ksq];
        nb = 768 * expanded[pos->opp_ksq];
    }
    uint64_t occ = pos->occ;
    int cnt = 0;
    while (occ) {
        int sq = __builtin_ctzll(occ);
        int piece = (pos->pcs[cnt / 2] >> (4 * (cnt % 2))) & 15;
        occ &= occ - 1;
        int c = (piece & 8) > 0;
        int pc = 64 * (piece & 7);
        int s = (c ? 384 : 0) + pc + sq;
        int n = (c ? 0 : 384) + pc + (sq ^ 56);
        if (cnt < nnz) {
            stm[cnt] = sb + (s ^ sflip);
            ntm[cnt] = nb + (n ^ nflip);
        }
        cnt++;
    }
    for (int i = cnt; i < nnz; i++) stm[i] = ntm[i] = -1;
    return cnt;
}

/* returns the largest feature count seen, or -1 if one exceeded nnz */
int orc_map_chess(const void* records, int n, int mode, const int32_t* layout32, int32_t* stm, int32_t* ntm, int nnz) {
    const orc_chess_board* r = (const orc_chess_board*)records;
    int worst = 0;
    for (int i = 0; i < n; i++) {
        int c = chess_features(&r[i], mode, layout32, stm + (size_t)i * nnz, ntm + (size_t)i * nnz, nnz);
        if (c > nnz) return -1;
        if (c > worst) worst = c;
    }
    return worst;
}

/* ataxx147.rs:18-27 over the iteration of examples/ataxx.rs:23-30 */
int orc_map_ataxx147(const void* records, int n, int32_t* stm, int32_t* ntm, int nnz) {
    const orc_ataxx_board* r = (const orc_ataxx_board*)records;
    int worst = 0;
    for (int i = 0; i < n; i++) {
        int cnt = 0;
        for (int pc = 0; pc < 3; pc++) {
            uint64_t occ = r[i].bbs[pc];
            while (occ) {
                int sq = __builtin_ctzll(occ);
                occ &= occ - 1;
                int s = 49 * pc + sq;
                int t = pc == 2 ? s : 49 * (1 - pc) + sq;
                if (cnt < nnz) {
                    stm[(size_t)i * nnz + cnt] = s;
                    ntm[(size_t)i * nnz + cnt] = t;
                }
                cnt++;
            }
        }
        if (cnt > nnz) return -1;
        for (int k = cnt; k < nnz; k++) stm[(size_t)i * nnz + k] = ntm[(size_t)i * nnz + k] = -1;
        if (cnt > worst) worst = cnt;
    }
    return worst;
}

/* outputs.rs:24-31 */
void orc_material_count(const void* records, int n, int nbuckets, int32_t* out) {
    const orc_chess_board* r = (const orc_chess_board*)records;
    int divisor = (32 + nbuckets - 1) / nbuckets;
    for (int i = 0; i < n; i++) out[i] = (uint8_t)((uint8_t)__builtin_popcountll(r[i].occ) - 2) / (uint8_t)divisor;
}

/* value.rs:103-115 with the plain sigmoid score model; always float, as the
 * reference computes targets in f32 on the host.  `stride` is the record size
 * and score/result sit at the same offsets in both record types. */
void orc_make_targets(const void* records, int n, int stride, int score_off, int result_off, float scale, float blend,
                      float* out) {
    const uint8_t* base = (const uint8_t*)records;
    float rscale = 1.0f / scale;
    for (int i = 0; i < n; i++) {
        int16_t sc;
        memcpy(&sc, base + (size_t)i * stride + score_off, 2);
        uint8_t res = base[(size_t)i * stride + result_off];
        float score = 1.0f / (1.0f + expf(-(rscale * (float)sc)));
        float result = (float)res / 2.0f;
        out[i] = blend * result + (1.0f - blend) * score;
    }
}

/* --------------------------------------------------------------- whole net */

typedef struct {
    int32_t n_inputs;        /* sparse inputs per perspective */
    int32_t nnz;             /* index slots per position */
    int32_t ft_out;          /* H: feature-transformer rows */
    int32_t ft_act;          /* 1 crelu, 2 screlu */
    int32_t pairwise;        /* 1: crelu halves multiplied, output H per position */
    int32_t factoriser_rows; /* 0, or the row count of l0f that tiles the inputs */
    int32_t n_out_buckets;   /* O */
    int32_t n_dense;         /* 1..3 dense layers after the concat */
    int32_t dense_out[3];    /* rows per bucket of each dense layer */
    int32_t dense_act[3];    /* activation after each dense layer (0 for the last) */
    int32_t ft_block_rows;   /* scheduling hint of the GPU library; unused here */
    int32_t max_batch;       /* capacity hint of the GPU library; unused here */
} orc_net_desc;

typedef struct {
    real* l0w;   /* [n_inputs][H] column-major: l0w[f*H + r] */
    real* l0b;   /* [H] */
    real* l0f;   /* [factoriser_rows][H] or NULL */
    real* lw[3]; /* [(O*M_i)][K_i] column-major: lw[c*(O*M_i) + row] */
    real* lb[3]; /* [O*M_i] */
} orc_tensors;

typedef struct {
    real decay, beta1, beta2, wmin, wmax;
} orc_adamw_params;

static int dense_in(const orc_net_desc* d, int layer) {
    if (layer == 0) return d->pairwise ? d->ft_out : 2 * d->ft_out;
    return d->dense_out[layer - 1];
}

/* Grow-only scratch buffers reused across calls: the large temporaries (gradient tables,
 * activations) would otherwise be mapped, faulted in and unmapped on every step, which
 * costs more than the arithmetic.  Not thread-safe across concurrent oracle calls. */
#define ORC_SCRATCH_SLOTS 8
static real* scratch_buf[ORC_SCRATCH_SLOTS];
static size_t scratch_len[ORC_SCRATCH_SLOTS];
static real* scratch(int slot, size_t n) {
    if (scratch_len[slot] < n) {
        free(scratch_buf[slot]);
        scratch_buf[slot] = (real*)malloc(sizeof(real) * n);
        scratch_len[slot] = n;
    }
    return scratch_buf[slot];
}
static void zero_parallel(real* p, size_t n) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) p[i] = 0;
}

/* Forward + backward of one batch.  Gradients are batch SUMS (the 1/B factor
 * lives in AdamW, crates/trainer/src/run.rs:130-131).  `out` (may be NULL)
 * receives the network output per position; `grads` may be NULL for a
 * forward-only call.  OpenMP threads split work only along axes that the
 * interpreter's sums do not run over (positions for per-position math, output
 * columns for the batch reductions), so every sum keeps the interpreter's
 * sequential order and the result does not depend on the thread count. */
int orc_net_grad(const orc_net_desc* d, const orc_tensors* w, const int32_t* stm, const int32_t* nstm,
                 const int32_t* buckets, const float* targets, int B, orc_tensors* grads, real* loss_out, real* out) {
    const int H = d->ft_out, NI = d->n_inputs, NNZ = d->nnz, O = d->n_out_buckets;
    const int half = H / 2;
    const int D1 = d->pairwise ? H : 2 * H;
    const int persp = d->pairwise ? half : H; /* outputs per perspective */
    const int nd = d->n_dense;
    if (nd < 1 || nd > 3 || d->dense_out[nd - 1] != 1 || B < 1) return -1;
    for (int l = 0; l < nd; l++)
        if (d->dense_out[l] > 64) return -1;

    /* W_eff = l0w + repeat(l0f): builder.rs:421-424, broadcast.rs:66-80 */
    const real* W = w->l0w;
    real* weff = NULL;
    if (d->factoriser_rows > 0) {
        size_t blk = (size_t)d->factoriser_rows * H;
        weff = scratch(0, (size_t)NI * H);
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < (size_t)NI * H; i++) weff[i] = w->l0w[i] + w->l0f[i % blk];
        W = weff;
    }

    real* u = scratch(1, (size_t)B * 2 * H); /* FT activation outputs, stm then nstm */
    real* x = scratch(2, (size_t)B * D1);    /* dense-stack input */
    real* a[3] = {0, 0, 0};                                    /* selected + activated outputs per layer */
    for (int l = 0; l < nd; l++) a[l] = (real*)malloc(sizeof(real) * (size_t)B * d->dense_out[l]);
    real* lossv = (real*)malloc(sizeof(real) * B);
    real* sig = (real*)malloc(sizeof(real) * B);

#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; b++) {
        const int32_t* lists[2] = {stm + (size_t)b * NNZ, nstm + (size_t)b * NNZ};
        for (int p = 0; p < 2; p++) {
            real* up = u + ((size_t)b * 2 + p) * H;
            for (int r = 0; r < H; r++) {
                real sum = 0;
                for (int n = 0; n < NNZ; n++) {
                    int32_t j = lists[p][n];
                    if (j >= 0 && j < NI) sum = sum + W[(size_t)H * j + r];
                }
                sum = sum + w->l0b[r]; /* builder.rs:145-147: bias after the matmul */
                up[r] = act_fwd(d->pairwise ? 1 : d->ft_act, sum);
            }
            real* xp = x + (size_t)b * D1 + (size_t)p * persp;
            if (d->pairwise)
                for (int j = 0; j < half; j++) xp[j] = up[j] * up[j + half];
            else
                for (int r = 0; r < H; r++) xp[r] = up[r];
        }
        /* dense stack on the selected bucket rows; the first layer is evaluated
         * as two half-width products that are then added (rewriterules.rs:211-265) */
        const int k = buckets[b];
        const real* in = x + (size_t)b * D1;
        for (int l = 0; l < nd; l++) {
            const int K = dense_in(d, l), M = d->dense_out[l], OM = O * M;
            real* al = a[l] + (size_t)b * M;
            for (int r = 0; r < M; r++) {
                const int row = k * M + r;
                real z;
                if (l == 0) {
                    real s0 = 0, s1 = 0;
                    for (int c = 0; c < K / 2; c++) s0 = s0 + w->lw[l][(size_t)c * OM + row] * in[c];
                    for (int c = K / 2; c < K; c++) s1 = s1 + w->lw[l][(size_t)c * OM + row] * in[c];
                    z = s0 + s1;
                } else {
                    z = 0;
                    for (int c = 0; c < K; c++) z = z + w->lw[l][(size_t)c * OM + row] * in[c];
                }
                z = z + w->lb[l][row];
                al[r] = act_fwd(d->dense_act[l], z);
            }
            in = al;
        }
        real o = a[nd - 1][b];
        if (out) out[b] = o;
        real s = sigmoid_r(o);
        real diff = s - (real)targets[b];
        sig[b] = s;
        lossv[b] = diff * diff;
    }
    /* reduce.rs:109-118: first element, then add the rest in order */
    real loss = lossv[0];
    for (int b = 1; b < B; b++) loss = loss + lossv[b];
    if (loss_out) *loss_out = loss;

    if (grads) {
        const size_t nl0 = (size_t)NI * H;
        real* dz[3] = {0, 0, 0}; /* gradient at each dense layer's selected pre-activation */
        for (int l = 0; l < nd; l++) dz[l] = (real*)malloc(sizeof(real) * (size_t)B * d->dense_out[l]);
        real* du = scratch(3, (size_t)B * 2 * H); /* gradient at the FT pre-activation */

        /* phase A, per position: everything that does not sum over the batch */
#pragma omp parallel
        {
            real* dx = (real*)malloc(sizeof(real) * D1);
#pragma omp for schedule(static)
            for (int b = 0; b < B; b++) {
                const int k = buckets[b];
                real s = sig[b];
                real diff = s - (real)targets[b];
                /* binary.rs:105-107 applied to diff*diff, then sigmoid from its output */
                real gin[64], tmp[64];
                gin[0] = (diff + diff) * (s * ((real)1 - s));
                for (int l = nd - 1; l >= 0; l--) {
                    const int K = dense_in(d, l), M = d->dense_out[l], OM = O * M;
                    const real* al = a[l] + (size_t)b * M;
                    real* dzl = dz[l] + (size_t)b * M;
                    for (int r = 0; r < M; r++) dzl[r] = gin[r] * act_bwd_from_output(d->dense_act[l], al[r]);
                    real* gout = l == 0 ? dx : tmp;
                    for (int c = 0; c < K; c++) {
                        real acc = 0;
                        for (int r = 0; r < M; r++) acc = acc + w->lw[l][(size_t)c * OM + k * M + r] * dzl[r];
                        gout[c] = acc;
                    }
                    if (l != 0)
                        for (int c = 0; c < K; c++) gin[c] = tmp[c];
                }
                for (int p = 0; p < 2; p++) {
                    const real* up = u + ((size_t)b * 2 + p) * H;
                    const real* dxp = dx + (size_t)p * persp;
                    real* dup = du + ((size_t)b * 2 + p) * H;
                    if (d->pairwise) {
                        for (int j = 0; j < half; j++) {
                            dup[j] = (dxp[j] * up[j + half]) * act_bwd_from_output(1, up[j]);
                            dup[j + half] = (dxp[j] * up[j]) * act_bwd_from_output(1, up[j + half]);
                        }
                    } else {
                        for (int r = 0; r < H; r++) dup[r] = dxp[r] * act_bwd_from_output(d->ft_act, up[r]);
                    }
                }
            }
            free(dx);
        }

        /* phase B: batch reductions, each output element summed over b in order */
        for (int l = 0; l < nd; l++) {
            const int K = dense_in(d, l), M = d->dense_out[l], OM = O * M;
            memset(grads->lw[l], 0, sizeof(real) * (size_t)OM * K);
            memset(grads->lb[l], 0, sizeof(real) * (size_t)OM);
            const real* inp = l == 0 ? x : a[l - 1];
#pragma omp parallel for schedule(static)
            for (int c = 0; c < K; c++)
                for (int b = 0; b < B; b++) {
                    const real xv = inp[(size_t)b * K + c];
                    const real* dzl = dz[l] + (size_t)b * M;
                    real* g = grads->lw[l] + (size_t)c * OM + buckets[b] * M;
                    for (int r = 0; r < M; r++) g[r] = g[r] + dzl[r] * xv;
                }
            for (int b = 0; b < B; b++)
                for (int r = 0; r < M; r++)
                    grads->lb[l][buckets[b] * M + r] = grads->lb[l][buckets[b] * M + r] + dz[l][(size_t)b * M + r];
        }
        /* the two perspectives fill separate zeroed tables which are then added
         * to a zeroed output one after the other (sparse.rs:253-271) */
        real* tab[2];
        for (int p = 0; p < 2; p++) {
            tab[p] = scratch(4 + p, nl0);
            zero_parallel(tab[p], nl0);
        }
        memset(grads->l0b, 0, sizeof(real) * H);
        {
            const int chunk = 64;
            const int nchunks = (H + chunk - 1) / chunk;
#pragma omp parallel for schedule(dynamic, 1)
            for (int ci = 0; ci < nchunks; ci++) {
                const int r0 = ci * chunk, r1 = r0 + chunk < H ? r0 + chunk : H;
                for (int b = 0; b < B; b++)
                    for (int p = 0; p < 2; p++) {
                        const real* dup = du + ((size_t)b * 2 + p) * H;
                        const int32_t* list = (p ? nstm : stm) + (size_t)b * NNZ;
                        for (int r = r0; r < r1; r++) grads->l0b[r] = grads->l0b[r] + dup[r];
                        for (int n = 0; n < NNZ; n++) {
                            int32_t j = list[n];
                            if (j >= 0 && j < NI) {
                                real* row = tab[p] + (size_t)H * j;
                                for (int r = r0; r < r1; r++) row[r] = dup[r] + row[r];
                            }
                        }
                    }
            }
        }
#pragma omp parallel for schedule(static)
        for (size_t i = 0; i < nl0; i++) grads->l0w[i] = ((real)0 + tab[0][i]) + tab[1][i];
        /* factoriser gradient = sum over the tiled copies (broadcast.rs:18-20 -> reduce.rs:96-120) */
        if (d->factoriser_rows > 0) {
            size_t blk = (size_t)d->factoriser_rows * H;
            int reps = (int)(nl0 / blk);
#pragma omp parallel for schedule(static)
            for (size_t i = 0; i < blk; i++) {
                real acc = grads->l0w[i];
                for (int r = 1; r < reps; r++) acc = acc + grads->l0w[(size_t)r * blk + i];
                grads->l0f[i] = acc;
            }
        }
        for (int l = 0; l < nd; l++) free(dz[l]);
    }

    for (int l = 0; l < nd; l++) free(a[l]);
    free(lossv);
    free(sig);
    (void)weff;
    return 0;
}

static void adam_tensor(real* p, real* m, real* v, const real* g, size_t n, real adj, real rate,
                        const orc_adamw_params* hp) {
    if (p) orc_adamw(p, m, v, g, n, adj, rate, hp->decay, hp->beta1, hp->beta2, hp->wmin, hp->wmax);
}

/* One AdamW step over every tensor (crates/trainer/src/optimiser.rs:162-194).
 * `hp` holds 9 entries in the order l0w l0b l0f l1w l1b l2w l2b l3w l3b. */
void orc_net_update(const orc_net_desc* d, orc_tensors* w, orc_tensors* m, orc_tensors* v, const orc_tensors* g,
                    real adj, real rate, const orc_adamw_params* hp) {
    size_t nl0 = (size_t)d->n_inputs * d->ft_out;
    adam_tensor(w->l0w, m->l0w, v->l0w, g->l0w, nl0, adj, rate, &hp[0]);
    adam_tensor(w->l0b, m->l0b, v->l0b, g->l0b, d->ft_out, adj, rate, &hp[1]);
    if (d->factoriser_rows > 0)
        adam_tensor(w->l0f, m->l0f, v->l0f, g->l0f, (size_t)d->factoriser_rows * d->ft_out, adj, rate, &hp[2]);
    for (int l = 0; l < d->n_dense; l++) {
        size_t rows = (size_t)d->n_out_buckets * d->dense_out[l];
        adam_tensor(w->lw[l], m->lw[l], v->lw[l], g->lw[l], rows * dense_in(d, l), adj, rate, &hp[3 + 2 * l]);
        adam_tensor(w->lb[l], m->lb[l], v->lb[l], g->lb[l], rows, adj, rate, &hp[4 + 2 * l]);
    }
}
