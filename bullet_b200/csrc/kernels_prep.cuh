// Batch preparation on the device, from raw 32-byte position records: the featurisers, the output
// bucket, the target blend, and the two stable groupings (positions by output bucket, (position,
// perspective) pairs by table row block) that the host otherwise builds while packing.
//
// Reference semantics (jw1912/bullet): Chess768::map_features
// crates/bullet_lib/src/game/inputs/chess768.rs:20-30, ChessBucketsMirrored
// crates/bullet_lib/src/game/inputs/chess_buckets.rs:57-88, Ataxx147
// crates/bullet_lib/src/game/inputs/ataxx147.rs:18-27, MaterialCount
// crates/bullet_lib/src/game/outputs.rs:24-31, the mapper's layout and target blend
// crates/bullet_lib/src/value.rs:77-117; record layouts as restated in examples/tests/test4.rs:8-36
// and examples/ataxx.rs:8-18.  The host mappers (host_map.h) are the same functions; a GPU test holds
// the two against each other bit for bit, including the order inside every group.
//
// Three launches on the copy stream:
//   prep_featurise_kernel  one thread per position: lists, bucket, target, the block of each of its two
//                          pairs; per CTA a histogram of buckets and of blocks
//   prep_scan_kernel       one CTA: per bin, the running sum over the CTAs (a CTA's first place inside
//                          the bin) and the bin totals, which the host reads to size the launches
//   prep_scatter_kernel    same CTAs: every position and pair goes to bin base + CTA base + its rank
//                          among the earlier ones of its CTA, i.e. a stable counting sort
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kPrepPositions = 256;  // positions per CTA of the featurise and scatter kernels
constexpr int kPrepMaxBins = 256;    // most row blocks (and most output buckets) the device path groups by
constexpr int kStatusTooManyPieces = 2, kStatusBadBucket = 4;

struct PrepArgs {
    const uint4* records;   // [n] raw records (32 bytes = two uint4 each)
    int n, nnz, n_inputs, game, n_out_buckets, block_rows, nblocks;
    const int* expanded;    // [64] 768 * king bucket of every square (king-bucketed chess inputs)
    const float* win_rate;  // [65536] sigmoid(score / scale) for every 16-bit score, index score + 32768
    float blend;
    uint16_t* stm;          // out [n][nnz], 0xFFFF = empty
    uint16_t* nstm;
    int* buckets;           // out [n]
    float* targets;         // out [n]
    uint16_t* pair_block;   // scratch [2n]
    int* cta_hist;          // scratch [nctas][nblocks + n_out_buckets]: counts, then first places
    int* totals;            // out [2 * (nblocks + n_out_buckets)]: bin totals, then bin bases
    int* order;             // out [n] positions grouped by output bucket
    int* pair_order;        // out [2n] pairs grouped by row block
    int* status;
};

// game codes as in bullet_b200.h: 0 chess 768, 1 king-bucketed mirrored chess, 2 ataxx 147
static __global__ void __launch_bounds__(kPrepPositions) prep_featurise_kernel(PrepArgs p) {
    __shared__ int hist[2 * kPrepMaxBins];
    const int nbins = p.nblocks + p.n_out_buckets;
    for (int k = threadIdx.x; k < nbins; k += blockDim.x) hist[k] = 0;
    __syncthreads();
    const int i = blockIdx.x * kPrepPositions + threadIdx.x;
    if (i < p.n) {
        const uint4 lo = p.records[2 * i], hi = p.records[2 * i + 1];
        // both record types keep score (i16) at byte 24 and the result at byte 26
        const int score = (int)(short)(hi.z & 0xffffu);
        const int result = (int)((hi.z >> 16) & 0xffu);
        uint16_t* s = p.stm + (size_t)i * p.nnz;
        uint16_t* t = p.nstm + (size_t)i * p.nnz;
        int count = 0, bad = 0, first_s = -1, first_t = -1;
        auto put = [&](int fs, int ft) {
            if (count >= p.nnz) {
                bad = 1;
                return;
            }
            const uint16_t a = (unsigned)fs < (unsigned)p.n_inputs ? (uint16_t)fs : (uint16_t)0xFFFFu;
            const uint16_t b = (unsigned)ft < (unsigned)p.n_inputs ? (uint16_t)ft : (uint16_t)0xFFFFu;
            s[count] = a;
            t[count] = b;
            if (first_s < 0 && a != 0xFFFFu) first_s = a;
            if (first_t < 0 && b != 0xFFFFu) first_t = b;
            count++;
        };
        unsigned long long occ = 0;
        if (p.game == 2) {
            const unsigned long long planes[3] = {(unsigned long long)lo.x | ((unsigned long long)lo.y << 32),
                                                  (unsigned long long)lo.z | ((unsigned long long)lo.w << 32),
                                                  (unsigned long long)hi.x | ((unsigned long long)hi.y << 32)};
            const int other_plane[3] = {49, 0, 98};
            for (int plane = 0; plane < 3; plane++)
                for (unsigned long long bb = planes[plane]; bb; bb &= bb - 1) {
                    const int sq = __ffsll((long long)bb) - 1;
                    put(49 * plane + sq, other_plane[plane] + sq);
                }
        } else {
            occ = (unsigned long long)lo.x | ((unsigned long long)lo.y << 32);
            // 16 bytes of 4-bit piece codes, two per byte, in ascending square order of the occupancy
            const unsigned pcs[4] = {lo.z, lo.w, hi.x, hi.y};
            const int ksq = (int)((hi.z >> 24) & 0xffu), opp_ksq = (int)(hi.w & 0xffu);
            int us_base = 0, us_flip = 0, them_base = 0, them_flip = 0;
            if (p.game == 1) {
                us_base = p.expanded[ksq & 63];
                us_flip = (ksq & 7) > 3 ? 7 : 0;  // the king on files e..h mirrors the board
                them_base = p.expanded[opp_ksq & 63];
                them_flip = (opp_ksq & 7) > 3 ? 7 : 0;
            }
            int piece = 0;
            for (unsigned long long bb = occ; bb; bb &= bb - 1, piece++) {
                const int sq = __ffsll((long long)bb) - 1;
                const int code = (int)((pcs[(piece >> 3) & 3] >> ((piece & 7) * 4)) & 15u);
                const int theirs = (code >> 3) & 1, type = code & 7;
                put(us_base + ((384 * theirs + 64 * type + sq) ^ us_flip),
                    them_base + ((384 * (1 - theirs) + 64 * type + (sq ^ 56)) ^ them_flip));
            }
        }
        for (int k = count; k < p.nnz; k++) s[k] = t[k] = (uint16_t)0xFFFFu;
        int bucket = 0;
        if (p.n_out_buckets > 1) {
            const int divisor = (32 + p.n_out_buckets - 1) / p.n_out_buckets;
            bucket = (__popcll(occ) - 2) / divisor;
            if ((unsigned)bucket >= (unsigned)p.n_out_buckets) {
                bad |= 2;
                bucket = 0;
            }
        }
        if (bad) atomicOr(p.status, (bad & 1 ? kStatusTooManyPieces : 0) | (bad & 2 ? kStatusBadBucket : 0));
        p.buckets[i] = bucket;
        // blend * result / 2 + (1 - blend) * sigmoid(score / scale), every operation rounded on its own as the
        // host compiler does it (no fused multiply-add)
        const float wr = p.win_rate[score + 32768];
        p.targets[i] = __fadd_rn(__fmul_rn(p.blend, __fdiv_rn((float)result, 2.0f)), __fmul_rn(__fsub_rn(1.0f, p.blend), wr));
        const int bs = first_s < 0 ? 0 : first_s / p.block_rows, bt = first_t < 0 ? 0 : first_t / p.block_rows;
        p.pair_block[2 * i] = (uint16_t)bs;
        p.pair_block[2 * i + 1] = (uint16_t)bt;
        atomicAdd(&hist[bs], 1);
        atomicAdd(&hist[bt], 1);
        atomicAdd(&hist[p.nblocks + bucket], 1);
    }
    __syncthreads();
    for (int k = threadIdx.x; k < nbins; k += blockDim.x) p.cta_hist[(size_t)blockIdx.x * nbins + k] = hist[k];
}

// grid = 1, block = 512 threads; nctas = CTAs of the featurise kernel
static __global__ void __launch_bounds__(512) prep_scan_kernel(PrepArgs p, int nctas) {
    const int nbins = p.nblocks + p.n_out_buckets;
    for (int k = threadIdx.x; k < nbins; k += blockDim.x) {
        int run = 0;
        for (int c = 0; c < nctas; c++) {
            const int v = p.cta_hist[(size_t)c * nbins + k];
            p.cta_hist[(size_t)c * nbins + k] = run;
            run += v;
        }
        p.totals[k] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {  // bin bases: blocks and output buckets are two separate groupings
        int run = 0;
        for (int k = 0; k < p.nblocks; k++) {
            p.totals[nbins + k] = run;
            run += p.totals[k];
        }
        run = 0;
        for (int k = p.nblocks; k < nbins; k++) {
            p.totals[nbins + k] = run;
            run += p.totals[k];
        }
    }
}

// grid = CTAs of the featurise kernel, block = 2 * kPrepPositions threads: thread s takes the CTA's s-th pair
// (pair ids ascend with the thread index), the first kPrepPositions threads also take a position each.
static __global__ void __launch_bounds__(2 * kPrepPositions) prep_scatter_kernel(PrepArgs p) {
    constexpr int NW = 2 * kPrepPositions / 32;
    __shared__ int warp_count[NW][kPrepMaxBins];
    const int nbins = p.nblocks + p.n_out_buckets;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned below = (1u << lane) - 1u;
    const int* cta_base = p.cta_hist + (size_t)blockIdx.x * nbins;
    const int* bin_base = p.totals + nbins;
    // pass 0: pairs by row block; pass 1: positions by output bucket
    for (int pass = 0; pass < 2; pass++) {
        const int bins = pass ? p.n_out_buckets : p.nblocks, first_bin = pass ? p.nblocks : 0;
        const int items = pass ? kPrepPositions : 2 * kPrepPositions;
        const int limit = pass ? p.n : 2 * p.n;
        for (int k = threadIdx.x; k < NW * kPrepMaxBins; k += blockDim.x) (&warp_count[0][0])[k] = 0;
        __syncthreads();
        const int id = blockIdx.x * items + threadIdx.x;
        const bool live = (int)threadIdx.x < items && id < limit;
        const int key = live ? (pass ? p.buckets[id] : (int)p.pair_block[id]) : bins;  // dead threads share a key of their own
        const unsigned same = __match_any_sync(0xffffffffu, key);
        const int rank = __popc(same & below);
        if (live && rank == 0) warp_count[warp][key] = __popc(same);
        __syncthreads();
        if (live) {
            int before = 0;
            for (int w = 0; w < warp; w++) before += warp_count[w][key];
            const int place = bin_base[first_bin + key] + cta_base[first_bin + key] + before + rank;
            (pass ? p.order : p.pair_order)[place] = id;
        }
        __syncthreads();
    }
}

}  // namespace b200
