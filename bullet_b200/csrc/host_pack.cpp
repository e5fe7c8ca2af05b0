// Host-side featurisers and index packing (no CUDA in this file).
//
// These replace the closure that ValueTrainerState::make_mapper builds around a
// SparseInputType (crates/bullet_lib/src/value.rs:77-117 in the reference): they walk
// 32-byte position records and emit the per-perspective feature lists, the output
// bucket and the blended target.  Unlike the reference, which writes a single -1
// terminator into a recycled buffer, every unused slot is set to -1, so that a
// kernel that skips invalid slots and one that stops at the first agree.
#include <cmath>
#include <cstring>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../../include/bullet_b200.h"
#include "common.h"
#include "host_map.h"

namespace {

// Records are independent: the loops below run over all host cores for large batches.  A record
// with too many pieces is remembered (the first one) and reported after the loop.
constexpr int kParallelFrom = 4096;

template <bool BUCKETED>
int map_chess(const void* records, int32_t n, const int32_t* layout32, int32_t* stm, int32_t* nstm, int32_t nnz) {
    int32_t expanded[64] = {0};
    if (BUCKETED) b200::expand_king_buckets(layout32, expanded);
    const b200::ChessRecord* rec = static_cast<const b200::ChessRecord*>(records);
    int worst = 0, bad = n;
#pragma omp parallel for schedule(static) reduction(max : worst) reduction(min : bad) if (n >= kParallelFrom)
    for (int32_t i = 0; i < n; i++) {
        const int count = b200::map_chess_record<BUCKETED, int32_t>(rec[i], expanded, stm + static_cast<size_t>(i) * nnz,
                                                                    nstm + static_cast<size_t>(i) * nnz, nnz, -1);
        if (count < 0) bad = i < bad ? i : bad;
        if (count > worst) worst = count;
    }
    if (bad < n) return b200::fail(B200_ERR_DATA, "record %d holds more than nnz=%d pieces", bad, nnz);
    return worst;
}

}  // namespace

extern "C" {

int b200_map_chess768(const void* records, int32_t n, int32_t* stm, int32_t* nstm, int32_t nnz) {
    if (!records || !stm || !nstm || n < 0 || nnz < 1) return b200::fail(B200_ERR_ARG, "map_chess768: bad argument");
    return map_chess<false>(records, n, nullptr, stm, nstm, nnz);
}

int b200_map_chess_buckets_mirrored(const void* records, int32_t n, const int32_t* layout32, int32_t* stm,
                                    int32_t* nstm, int32_t nnz) {
    if (!records || !layout32 || !stm || !nstm || n < 0 || nnz < 1)
        return b200::fail(B200_ERR_ARG, "map_chess_buckets_mirrored: bad argument");
    return map_chess<true>(records, n, layout32, stm, nstm, nnz);
}

int b200_map_ataxx147(const void* records, int32_t n, int32_t* stm, int32_t* nstm, int32_t nnz) {
    if (!records || !stm || !nstm || n < 0 || nnz < 1) return b200::fail(B200_ERR_ARG, "map_ataxx147: bad argument");
    const b200::AtaxxRecord* rec = static_cast<const b200::AtaxxRecord*>(records);
    int worst = 0, bad = n;
#pragma omp parallel for schedule(static) reduction(max : worst) reduction(min : bad) if (n >= kParallelFrom)
    for (int32_t i = 0; i < n; i++) {
        const int count = b200::map_ataxx_record<int32_t>(rec[i], stm + static_cast<size_t>(i) * nnz,
                                                          nstm + static_cast<size_t>(i) * nnz, nnz, -1);
        if (count < 0) bad = i < bad ? i : bad;
        if (count > worst) worst = count;
    }
    if (bad < n) return b200::fail(B200_ERR_DATA, "record %d holds more than nnz=%d cells", bad, nnz);
    return worst;
}

int b200_material_count(const void* records, int32_t n, int32_t n_buckets, int32_t* out) {
    if (!records || !out || n < 0 || n_buckets < 1) return b200::fail(B200_ERR_ARG, "material_count: bad argument");
    const b200::ChessRecord* rec = static_cast<const b200::ChessRecord*>(records);
#pragma omp parallel for schedule(static) if (n >= kParallelFrom)
    for (int32_t i = 0; i < n; i++) out[i] = b200::material_bucket(rec[i].occ, n_buckets);
    return 0;
}

int b200_make_targets(const void* records, int32_t n, float scale, float blend, float* out) {
    if (!records || !out || n < 0 || !(blend >= 0.f && blend <= 1.f))
        return b200::fail(B200_ERR_ARG, "make_targets: bad argument");
    const b200::ChessRecord* rec = static_cast<const b200::ChessRecord*>(records);
    const float rscale = 1.0f / scale;
#pragma omp parallel for schedule(static) if (n >= kParallelFrom)
    for (int32_t i = 0; i < n; i++) out[i] = b200::blended_target(rec[i].score, rec[i].result, rscale, blend);
    return 0;
}

// How many host threads the featurisers and the batch packing use (OpenMP); n < 1 = the runtime's own
// choice.  Launchers that start one process per GPU often pin every process to one thread.
int b200_set_host_threads(int32_t n) {
#ifdef _OPENMP
    omp_set_num_threads(n >= 1 ? n : omp_get_num_procs());
#else
    (void)n;
#endif
    return 0;
}

int b200_pack_indices_u16(const int32_t* idx, int64_t count, uint16_t* out) {
    if (!idx || !out || count < 0) return b200::fail(B200_ERR_ARG, "pack_indices: bad argument");
    for (int64_t i = 0; i < count; i++) {
        const uint32_t v = static_cast<uint32_t>(idx[i]);  // negatives become huge
        out[i] = v < 0xFFFFu ? static_cast<uint16_t>(v) : 0xFFFFu;
    }
    return 0;
}

int b200_unpack_indices_u16(const uint16_t* packed, int64_t count, int32_t* out) {
    if (!packed || !out || count < 0) return b200::fail(B200_ERR_ARG, "unpack_indices: bad argument");
    for (int64_t i = 0; i < count; i++) out[i] = packed[i] == 0xFFFFu ? -1 : static_cast<int32_t>(packed[i]);
    return 0;
}

}  // extern "C"
