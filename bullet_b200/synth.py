"""Seeded synthetic positions in the reference's on-disk record formats.

No public data set is used anywhere in this repository: every measured batch comes from
these generators.  The records have the 32-byte layouts the reference reads
(`ChessBoard`, examples/tests/test4.rs:8-18; `AtaxxBoard`, examples/ataxx.rs:8-18), so the
featurisers see exactly what they would see when reading a data file.

PRNG: numpy `Generator(PCG64(seed))`.  Only reproducibility matters here, because the CPU
oracle and the GPU path consume the same generated arrays.

Chess: piece count k ~ U{2..32}; two kings plus k-2 pieces of uniform type P..Q and
uniform colour on distinct uniform squares; a pawn drawn on rank 1 or 8 is redrawn as a
uniform N/B/R/Q.  The record is side-to-move relative: our king (colour bit 0) sits at
`ksq`, the opponent's at `opp_ksq ^ 56` (the opponent's own frame is stored).
Ataxx: blocked count ~ U{0..8} placed point-symmetrically (pairs sq, 48-sq; the centre
cell takes the odd one), then U{2..free} stones of uniform colour on the free cells.
Targets: score ~ N(0, 400) cp, rounded and clipped to +-3000; with s = sigmoid(score/400)
the game result is a win with probability s^2, a loss with (1-s)^2, else a draw, stored
as 2 / 0 / 1 in `result`; the mapper then blends 0.5*result/2 + 0.5*s.
"""
from __future__ import annotations

import numpy as np

CHESS_DTYPE = np.dtype(
    [("occ", "<u8"), ("pcs", "u1", (16,)), ("score", "<i2"), ("result", "u1"), ("ksq", "u1"),
     ("opp_ksq", "u1"), ("extra", "u1", (3,))]
)
ATAXX_DTYPE = np.dtype(
    [("bbs", "<u8", (3,)), ("score", "<i2"), ("result", "u1"), ("origstm", "u1"), ("fullm", "<u2"),
     ("halfm", "u1"), ("extra", "u1")]
)
assert CHESS_DTYPE.itemsize == 32 and ATAXX_DTYPE.itemsize == 32


def _scores_results(rng: np.random.Generator, n: int):
    score = np.clip(np.rint(rng.normal(0.0, 400.0, n)), -3000, 3000).astype(np.int16)
    s = 1.0 / (1.0 + np.exp(-score.astype(np.float64) / 400.0))
    r = rng.random(n)
    result = np.where(r < s * s, 2, np.where(r < s * s + (1 - s) * (1 - s), 0, 1)).astype(np.uint8)
    return score, result


def chess_records(n: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    k = rng.integers(2, 33, n)                                  # pieces on the board
    order = np.argsort(rng.random((n, 64)), axis=1)[:, :32]     # distinct uniform squares
    ptype = rng.integers(0, 5, (n, 32))                         # P N B R Q
    redraw = rng.integers(1, 5, (n, 32))                        # N B R Q for pawns on ranks 1/8
    colour = rng.integers(0, 2, (n, 32))
    rank = order // 8
    ptype = np.where((ptype == 0) & ((rank == 0) | (rank == 7)), redraw, ptype)
    ptype[:, 0], colour[:, 0] = 5, 0                            # our king
    ptype[:, 1], colour[:, 1] = 5, 1                            # their king
    code = (colour << 3) | ptype
    active = np.arange(32)[None, :] < k[:, None]
    # pieces are stored in ascending square order of the occupancy bitboard
    sq_sorted_key = np.where(active, order, 64)
    perm = np.argsort(sq_sorted_key, axis=1, kind="stable")
    sq = np.take_along_axis(order, perm, axis=1)
    code = np.take_along_axis(code, perm, axis=1)
    act = np.take_along_axis(active, perm, axis=1)
    code = np.where(act, code, 0).astype(np.uint8)
    occ = np.zeros(n, dtype=np.uint64)
    for j in range(32):
        occ |= np.where(act[:, j], np.uint64(1) << sq[:, j].astype(np.uint64), np.uint64(0))
    rec = np.zeros(n, dtype=CHESS_DTYPE)
    rec["occ"] = occ
    rec["pcs"] = code[:, 0::2] | (code[:, 1::2] << 4)
    rec["score"], rec["result"] = _scores_results(rng, n)
    rec["ksq"] = order[:, 0]
    rec["opp_ksq"] = order[:, 1] ^ 56
    return rec


def ataxx_records(n: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    nblocked = rng.integers(0, 9, n)
    pair_order = np.argsort(rng.random((n, 24)), axis=1)        # the 24 symmetric pairs (sq, 48-sq)
    blocked = np.zeros((n, 49), dtype=bool)
    rows = np.arange(n)
    for j in range(4):
        use = (nblocked // 2) > j
        sqs = pair_order[:, j]
        blocked[rows[use], sqs[use]] = True
        blocked[rows[use], 48 - sqs[use]] = True
    blocked[rows[nblocked % 2 == 1], 24] = True
    free = 49 - blocked.sum(axis=1)
    stones = 2 + (rng.random(n) * (free - 1)).astype(np.int64)   # U{2..free}
    key = np.where(blocked, 2.0, rng.random((n, 49)))
    rankpos = np.argsort(np.argsort(key, axis=1), axis=1)
    has_stone = rankpos < stones[:, None]
    colour = rng.integers(0, 2, (n, 49)).astype(bool)
    weights = (np.uint64(1) << np.arange(49, dtype=np.uint64))[None, :]
    rec = np.zeros(n, dtype=ATAXX_DTYPE)
    bbs = np.zeros((n, 3), dtype=np.uint64)
    bbs[:, 0] = (np.where(has_stone & ~colour, weights, np.uint64(0))).sum(axis=1, dtype=np.uint64)
    bbs[:, 1] = (np.where(has_stone & colour, weights, np.uint64(0))).sum(axis=1, dtype=np.uint64)
    bbs[:, 2] = (np.where(blocked, weights, np.uint64(0))).sum(axis=1, dtype=np.uint64)
    rec["bbs"] = bbs
    rec["score"], rec["result"] = _scores_results(rng, n)
    return rec


def records(game: str, n: int, seed: int) -> np.ndarray:
    if game in ("chess768", "chess_buckets"):
        return chess_records(n, seed)
    if game == "ataxx147":
        return ataxx_records(n, seed)
    raise ValueError(game)


def init_weights(desc, seed: int, ft_fan_in: int | None = None) -> dict:
    """Seeded uniform +-1/sqrt(fan_in) weights, zero biases and zero factoriser.

    The reference draws Normal(0, sqrt(2/fan_in)) from its own generator
    (crates/compiler/src/model/builder.rs:108-119); parity runs load the same explicit arrays
    into the oracle and the GPU, so only the law's scale matters.  `ft_fan_in` overrides the
    feature transformer's fan-in; king-bucketed nets default to 32 active inputs, as
    examples/progression/4_multi_layer.rs:69 does.
    """
    rng = np.random.default_rng(seed ^ 0x5EED)
    if ft_fan_in is None:
        ft_fan_in = 32 if desc.n_inputs > 768 else desc.n_inputs
    out = {}
    for name, (rows, cols) in desc.tensor_shapes().items():
        if name.endswith("b") or name == "l0f":
            out[name] = np.zeros(rows * cols, dtype=np.float32)
        else:
            lim = 1.0 / np.sqrt(ft_fan_in if name == "l0w" else cols)
            out[name] = rng.uniform(-lim, lim, rows * cols).astype(np.float32)
    return out
