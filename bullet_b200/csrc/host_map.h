// Per-record featurisers shared by the stand-alone mappers (host_pack.cpp) and the upload that
// maps records straight into a pinned staging slot (net.cu).  No CUDA here.
//
// Reference (jw1912/bullet): Chess768::map_features crates/bullet_lib/src/game/inputs/chess768.rs:20-30,
// ChessBucketsMirrored crates/bullet_lib/src/game/inputs/chess_buckets.rs:57-88,
// Ataxx147 crates/bullet_lib/src/game/inputs/ataxx147.rs:18-27, MaterialCount
// crates/bullet_lib/src/game/outputs.rs:24-31, the target blend of
// ValueTrainerState::make_mapper crates/bullet_lib/src/value.rs:103-115; record layouts as restated
// in examples/tests/test4.rs:8-36 and examples/ataxx.rs:8-18.
#pragma once
#include <cmath>
#include <cstdint>

namespace b200 {

#pragma pack(push, 1)
struct ChessRecord {  // bulletformat ChessBoard
    uint64_t occ;
    uint8_t pcs[16];
    int16_t score;
    uint8_t result;
    uint8_t ksq;
    uint8_t opp_ksq;
    uint8_t extra[3];
};
struct AtaxxRecord {
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

// 64-square table of 768 * bucket from the reference's 32-entry half-board layout
inline void expand_king_buckets(const int32_t* layout32, int32_t (&expanded)[64]) {
    for (int sq = 0; sq < 64; sq++) {
        const int file = sq & 7, folded = file < 4 ? file : 7 - file;
        expanded[sq] = 768 * layout32[(sq >> 3) * 4 + folded];
    }
}

// One chess record -> its two feature lists; unused slots get `empty`.  Returns the number of
// pieces, or -1 if the record holds more than nnz.
template <bool BUCKETED, typename T>
inline int map_chess_record(const ChessRecord& r, const int32_t* expanded, T* s, T* t, int nnz, T empty) {
    int32_t us_base = 0, us_flip = 0, them_base = 0, them_flip = 0;
    if (BUCKETED) {
        us_base = expanded[r.ksq & 63];
        us_flip = (r.ksq & 7) > 3 ? 7 : 0;  // the king on files e..h mirrors the board
        them_base = expanded[r.opp_ksq & 63];
        them_flip = (r.opp_ksq & 7) > 3 ? 7 : 0;
    }
    int count = 0;
    for (uint64_t bb = r.occ; bb; bb &= bb - 1, count++) {
        if (count >= nnz) return -1;
        const int sq = __builtin_ctzll(bb);
        const int code = (r.pcs[count >> 1] >> ((count & 1) * 4)) & 15;
        s[count] = static_cast<T>(us_base + ((kPieceBase.stm[code] + sq) ^ us_flip));
        t[count] = static_cast<T>(them_base + ((kPieceBase.ntm[code] + (sq ^ 56)) ^ them_flip));
    }
    for (int k = count; k < nnz; k++) s[k] = t[k] = empty;
    return count;
}

// own stones, their stones, blocked cells: the other side swaps the first two planes
template <typename T>
inline int map_ataxx_record(const AtaxxRecord& r, T* s, T* t, int nnz, T empty) {
    const int other_plane[3] = {49, 0, 98};
    int count = 0;
    for (int plane = 0; plane < 3; plane++)
        for (uint64_t bb = r.bbs[plane]; bb; bb &= bb - 1, count++) {
            if (count >= nnz) return -1;
            const int sq = __builtin_ctzll(bb);
            s[count] = static_cast<T>(49 * plane + sq);
            t[count] = static_cast<T>(other_plane[plane] + sq);
        }
    for (int k = count; k < nnz; k++) s[k] = t[k] = empty;
    return count;
}

inline int32_t material_bucket(uint64_t occ, int n_buckets) {
    const int divisor = (32 + n_buckets - 1) / n_buckets;
    return (__builtin_popcountll(occ) - 2) / divisor;
}

// score and result sit at the same offsets in both record types
inline float blended_target(int16_t score, uint8_t result, float rscale, float blend) {
    const float wr = 1.0f / (1.0f + std::exp(-(rscale * static_cast<float>(score))));
    return blend * (static_cast<float>(result) / 2.0f) + (1.0f - blend) * wr;
}

}  // namespace b200
