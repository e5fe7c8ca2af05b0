"""Network descriptions for the NNUE training step and the five benchmark configurations.

A `NetDesc` is the recognised form of the graph that bullet's builder closure emits
(examples/simple.rs:25-56, examples/progression/4_multi_layer.rs:66-87 in the reference):
two sparse perspective inputs through one shared affine feature transformer, an
activation (CReLU / SCReLU, optionally pairwise-multiplied halves), the stm|nstm concat,
then up to three output-bucketed dense layers and a sigmoid-MSE loss.
"""
from __future__ import annotations

import ctypes
import dataclasses
from dataclasses import dataclass, field

ACT_NONE, ACT_CRELU, ACT_SCRELU = 0, 1, 2

#: tensor names in flat-buffer order (name-sorted, as the reference's BTreeMap iterates them,
#: crates/trainer/src/model/weights.rs:95-110)
TENSOR_ORDER = ("l0b", "l0f", "l0w", "l1b", "l1w", "l2b", "l2w", "l3b", "l3w")


@dataclass
class AdamWParams:
    """crates/trainer/src/optimiser/adam.rs:20-33 (same field meaning and defaults)."""

    decay: float = 0.01
    beta1: float = 0.9
    beta2: float = 0.999
    min_weight: float = -1.98
    max_weight: float = 1.98


@dataclass
class RAdamParams:
    """crates/trainer/src/optimiser/radam.rs:19-32 (same defaults; clip None = no clipping)."""

    beta1: float = 0.9
    beta2: float = 0.999
    n_sma_threshold: float = 5.0
    decay: float = 0.0
    clip: tuple | None = None


@dataclass
class RangerParams:
    """crates/trainer/src/optimiser/ranger.rs:137-151 (same defaults)."""

    decay: float = 0.01
    beta1: float = 0.99
    beta2: float = 0.999
    min_weight: float = -1.98
    max_weight: float = 1.98
    alpha: float = 0.5
    k: int = 6


@dataclass
class NetDesc:
    n_inputs: int                 # sparse inputs per perspective
    nnz: int                      # index slots per position (max active features)
    ft_out: int                   # feature-transformer rows H
    ft_act: int                   # ACT_CRELU or ACT_SCRELU
    pairwise: bool = False        # crelu(lo) * crelu(hi) per perspective
    factoriser_rows: int = 0      # 0, or rows of l0f tiled over the inputs (768 for chess)
    n_out_buckets: int = 1
    dense_out: tuple = (1,)       # rows per bucket of each dense layer; last must be 1
    dense_act: tuple = (ACT_NONE,)
    ft_block_rows: int = 0        # >0: every position's features of one perspective fall in one
                                  # aligned block of this many table rows (king-bucketed inputs)
    max_batch: int = 16384

    @property
    def n_dense(self) -> int:
        return len(self.dense_out)

    @property
    def dense_in0(self) -> int:
        return self.ft_out if self.pairwise else 2 * self.ft_out

    def dense_in(self, layer: int) -> int:
        return self.dense_in0 if layer == 0 else self.dense_out[layer - 1]

    def tensor_shapes(self) -> dict:
        """name -> (rows, cols), column-major (docs/4-saved-networks.md:21-31 in the reference)."""
        shapes = {"l0w": (self.ft_out, self.n_inputs), "l0b": (self.ft_out, 1)}
        if self.factoriser_rows:
            shapes["l0f"] = (self.ft_out, self.factoriser_rows)
        for i in range(self.n_dense):
            rows = self.n_out_buckets * self.dense_out[i]
            shapes[f"l{i + 1}w"] = (rows, self.dense_in(i))
            shapes[f"l{i + 1}b"] = (rows, 1)
        return {k: shapes[k] for k in TENSOR_ORDER if k in shapes}

    def n_params(self) -> int:
        return sum(r * c for r, c in self.tensor_shapes().values())

    def validate(self) -> None:
        if self.ft_act not in (ACT_CRELU, ACT_SCRELU):
            raise ValueError("ft_act must be CReLU or SCReLU")
        if self.pairwise and (self.ft_act != ACT_CRELU or self.ft_out % 2):
            raise ValueError("pairwise_mul needs CReLU and an even ft_out")
        if not 1 <= self.n_dense <= 3 or self.dense_out[-1] != 1 or self.dense_act[-1] != ACT_NONE:
            raise ValueError("one to three dense layers, the last with one row per bucket and no activation")
        if len(self.dense_act) != self.n_dense:
            raise ValueError("dense_act and dense_out differ in length")
        if self.factoriser_rows and self.n_inputs % self.factoriser_rows:
            raise ValueError("factoriser rows must tile the inputs")


class CNetDesc(ctypes.Structure):
    """Binary layout shared by `b200_net_desc` (include/bullet_b200.h) and the oracle."""

    _fields_ = [
        ("n_inputs", ctypes.c_int32),
        ("nnz", ctypes.c_int32),
        ("ft_out", ctypes.c_int32),
        ("ft_act", ctypes.c_int32),
        ("pairwise", ctypes.c_int32),
        ("factoriser_rows", ctypes.c_int32),
        ("n_out_buckets", ctypes.c_int32),
        ("n_dense", ctypes.c_int32),
        ("dense_out", ctypes.c_int32 * 3),
        ("dense_act", ctypes.c_int32 * 3),
        ("ft_block_rows", ctypes.c_int32),
        ("max_batch", ctypes.c_int32),
    ]

    @classmethod
    def from_desc(cls, d: NetDesc) -> "CNetDesc":
        d.validate()
        out = cls()
        out.n_inputs, out.nnz, out.ft_out, out.ft_act = d.n_inputs, d.nnz, d.ft_out, d.ft_act
        out.pairwise, out.factoriser_rows = int(d.pairwise), d.factoriser_rows
        out.n_out_buckets, out.n_dense = d.n_out_buckets, d.n_dense
        for i in range(3):
            out.dense_out[i] = d.dense_out[i] if i < d.n_dense else 0
            out.dense_act[i] = d.dense_act[i] if i < d.n_dense else 0
        out.ft_block_rows, out.max_batch = d.ft_block_rows, d.max_batch
        return out


#: 32-entry half-board king-bucket table for the "768x16" inputs: two ranks and one mirrored
#: file per bucket.  Expanded to 64 squares by ChessBucketsMirrored::new
#: (crates/bullet_lib/src/game/inputs/chess_buckets.rs:57-66); a king on files e-h mirrors the
#: board (chess_buckets.rs:83).
KING_BUCKETS_16 = tuple((rank // 2) * 4 + f for rank in range(8) for f in range(4))


@dataclass
class BenchConfig:
    name: str
    desc: NetDesc
    game: str                     # "chess768" | "chess_buckets" | "ataxx147"
    batch: int
    lr: float = 1e-3
    adamw: AdamWParams = field(default_factory=AdamWParams)
    seed: int = 0

    def with_batch(self, batch: int) -> "BenchConfig":
        return dataclasses.replace(self, batch=batch, desc=dataclasses.replace(self.desc, max_batch=batch))


def config(i: int) -> BenchConfig:
    """The five configurations of the headline benchmark, by index."""
    if i == 0:  # examples/simple.rs shape: 768 -> 128 SCReLU, concat -> 1
        d = NetDesc(n_inputs=768, nnz=32, ft_out=128, ft_act=ACT_SCRELU, ft_block_rows=768, max_batch=16384)
        return BenchConfig("c0-simple-768x128", d, "chess768", 16384, seed=1000)
    if i == 1:  # 768x16 king buckets + factoriser -> 1024 SCReLU -> 8 output buckets
        d = NetDesc(n_inputs=12288, nnz=32, ft_out=1024, ft_act=ACT_SCRELU, factoriser_rows=768,
                    n_out_buckets=8, ft_block_rows=768, max_batch=16384)
        return BenchConfig("c1-768x16-1024-ob8", d, "chess_buckets", 16384, seed=1001)
    if i == 2:  # examples/ataxx.rs shape with CReLU: 147 -> 256, concat -> 1
        d = NetDesc(n_inputs=147, nnz=49, ft_out=256, ft_act=ACT_CRELU, ft_block_rows=147, max_batch=32768)
        return BenchConfig("c2-ataxx-147x256", d, "ataxx147", 32768, seed=1002)
    if i in (3, 4):  # examples/progression/4_multi_layer.rs shape at H = 2048
        batch = 16384 if i == 3 else 131072
        d = NetDesc(n_inputs=12288, nnz=32, ft_out=2048, ft_act=ACT_CRELU, pairwise=True, factoriser_rows=768,
                    n_out_buckets=8, dense_out=(16, 32, 1), dense_act=(ACT_SCRELU, ACT_SCRELU, ACT_NONE),
                    ft_block_rows=768, max_batch=batch)
        name = "c3-768x16-2048pw-16-32-1-ob8" if i == 3 else "c4-768x16-2048pw-16-32-1-ob8-dp"
        return BenchConfig(name, d, "chess_buckets", batch, seed=1003)
    raise ValueError(f"no config {i}")
