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

#include "../../include/bullet_b200.h"
#include "common.h"

namespace {

#pragma pack(push, 1)
struct ChessRecord {  // bulletformat ChessBoard as restated in examples/tests/test4.rs:8-18
    uint64_t occ;
    uint8_t pcs[16];
    int16_t score;
    uint8_t result;
    uint8_t ksq;
    uint8_t opp_ksq;
    uint8_t extra[3];
};
struct AtaxxRecord {  // examples/ataxx.rs:8-18
    uint64_t bbs[3];
    int16_t score;
    uint8_t result;
    uint8_t origstm;
    uint16_t fullm;
    uint8_t halfm;
    uint8_t extra;
};
#pragma pack(pop)
static_assert(sizeof(ChessRecord) == 32 && sizeof(AtaxxRecord) == 32, "record layout");

// Per 4-bit piece code: base feature for the side to move and for the other side
// (chess768.rs:21-28: colour swaps the 384 halves, the other side sees sq ^ 56).
struct PieceBase {
    int16_t stm[16], ntm[16];
    constexpr PieceBase() : stm(), ntm() {
        for (int code = 0; code < 16; code++) {
            const int theirs = (code >> 3) & 1, type = code & 7;
            stm[code] = static_cast<int16_t>(384 * theirs + 64 * type);
            ntm[code] = static_cast<int16_t>(384 * (1 - theirs) + 64 * type);
        }
    }
};
constexpr PieceBase kPieceBase;

struct Perspective {
    int32_t base = 0;  // 768 * bucket
    int32_t flip = 0;  // 7 when the king stands on files e..h
};

template <bool BUCKETED>
int map_chess(const void* records, int32_t n, const int32_t* layout32, int32_t* stm, int32_t* nstm, int32_t nnz) {
    int32_t expanded[64] = {0};
    if (BUCKETED) {
        for (int sq = 0; sq < 64; sq++) {
            const int file = sq & 7, folded = file < 4 ? file : 7 - file;
            expanded[sq] = 768 * layout32[(sq >> 3) * 4 + folded];
        }
    }
    const ChessRecord* rec = static_cast<const ChessRecord*>(records);
    int worst = 0;
    for (int32_t i = 0; i < n; i++) {
        const ChessRecord& r = rec[i];
        Perspective us, them;
        if (BUCKETED) {
            us.base = expanded[r.ksq & 63];
            us.flip = (r.ksq & 7) > 3 ? 7 : 0;
            them.base = expanded[r.opp_ksq & 63];
            them.flip = (r.opp_ksq & 7) > 3 ? 7 : 0;
        }
        int32_t* s = stm + static_cast<size_t>(i) * nnz;
        int32_t* t = nstm + static_cast<size_t>(i) * nnz;
        int count = 0;
        for (uint64_t bb = r.occ; bb; bb &= bb - 1, count++) {
            if (count >= nnz) return b200::fail(B200_ERR_DATA, "record %d holds more than nnz=%d pieces", i, nnz);
            const int sq = __builtin_ctzll(bb);
            const int code = (r.pcs[count >> 1] >> ((count & 1) * 4)) & 15;
            s[count] = us.base + ((kPieceBase.stm[code] + sq) ^ us.flip);
            t[count] = them.base + ((kPieceBase.ntm[code] + (sq ^ 56)) ^ them.flip);
        }
        for (int k = count; k < nnz; k++) s[k] = t[k] = -1;
        if (count > worst) worst = count;
    }
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
    const AtaxxRecord* rec = static_cast<const AtaxxRecord*>(records);
    // own stones, their stones, blocked cells: the other side swaps the first two planes
    static const int other_plane[3] = {49, 0, 98};
    int worst = 0;
    for (int32_t i = 0; i < n; i++) {
        int32_t* s = stm + static_cast<size_t>(i) * nnz;
        int32_t* t = nstm + static_cast<size_t>(i) * nnz;
        int count = 0;
        for (int plane = 0; plane < 3; plane++)
            for (uint64_t bb = rec[i].bbs[plane]; bb; bb &= bb - 1, count++) {
                if (count >= nnz) return b200::fail(B200_ERR_DATA, "record %d holds more than nnz=%d cells", i, nnz);
                const int sq = __builtin_ctzll(bb);
                s[count] = 49 * plane + sq;
                t[count] = other_plane[plane] + sq;
            }
        for (int k = count; k < nnz; k++) s[k] = t[k] = -1;
        if (count > worst) worst = count;
    }
    return worst;
}

int b200_material_count(const void* records, int32_t n, int32_t n_buckets, int32_t* out) {
    if (!records || !out || n < 0 || n_buckets < 1) return b200::fail(B200_ERR_ARG, "material_count: bad argument");
    const ChessRecord* rec = static_cast<const ChessRecord*>(records);
    const int divisor = (32 + n_buckets - 1) / n_buckets;
    for (int32_t i = 0; i < n; i++) out[i] = (__builtin_popcountll(rec[i].occ) - 2) / divisor;
    return 0;
}

int b200_make_targets(const void* records, int32_t n, float scale, float blend, float* out) {
    if (!records || !out || n < 0 || !(blend >= 0.f && blend <= 1.f))
        return b200::fail(B200_ERR_ARG, "make_targets: bad argument");
    // score and result sit at the same offsets in both record types
    const ChessRecord* rec = static_cast<const ChessRecord*>(records);
    const float rscale = 1.0f / scale;
    for (int32_t i = 0; i < n; i++) {
        const float wr = 1.0f / (1.0f + std::exp(-(rscale * static_cast<float>(rec[i].score))));
        out[i] = blend * (static_cast<float>(rec[i].result) / 2.0f) + (1.0f - blend) * wr;
    }
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
