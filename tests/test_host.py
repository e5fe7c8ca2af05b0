"""CPU tests of the host side: the C-ABI library loads and exports what the header declares,
featurisers and index packing are bit-exact against the oracle and the reference layout."""
import os
import re

import numpy as np
import pytest

from bullet_b200 import _lib, config, synth
from bullet_b200.configs import KING_BUCKETS_16, NetDesc
from bullet_b200.net import featurise, pack_indices, unpack_indices

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_rust_declarations_cover_the_header():
    header = open(os.path.join(ROOT, "include", "bullet_b200.h")).read()
    rust = open(os.path.join(ROOT, "bindings", "rust", "b200-sys", "src", "lib.rs")).read()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header))
    bound = set(re.findall(r"pub fn (b200_[a-z0-9_]+)\s*\(", rust))
    assert declared == bound
    for struct in ("b200_net_desc", "b200_adamw_params", "b200_timings", "b200_ft_op", "b200_saved_format"):
        assert f"pub struct {struct}" in rust


def test_rust_trainer_source_calls_only_declared_symbols():
    """bindings/rust/b200 (the recogniser and the train loop for bullet's own crates) is source only:
    at least every entry point it calls must exist in the header, and it must cover the step."""
    header = open(os.path.join(ROOT, "include", "bullet_b200.h")).read()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header))
    src_dir = os.path.join(ROOT, "bindings", "rust", "b200", "src")
    used = set()
    for name in os.listdir(src_dir):
        used |= set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", open(os.path.join(src_dir, name)).read()))
    used -= {"b200_net_desc", "b200_adamw_params"}
    assert used and used <= declared, used - declared
    assert {"b200_net_create", "b200_batch_upload", "b200_step", "b200_loss", "b200_checkpoint_save"} <= used


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "bullet_b200.h")).read()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.SYMBOLS)
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.b200_version() >= 1


@pytest.mark.parametrize("ci", [0, 1, 2, 3])
def test_featurisers_bit_exact_vs_oracle(oracle32, ci):
    c = config(ci)
    rec = synth.records(c.game, 4096, seed=c.seed + 7)
    ours = featurise(c.game, rec, c.desc)
    ref = oracle32.map_batch(c.game, rec, c.desc)
    for a, b, what in zip(ours, ref, ("stm", "nstm", "buckets", "targets")):
        assert a.dtype == b.dtype and np.array_equal(a, b), what


def test_reference_layout_properties():
    # crates/bullet_lib/src/value.rs:77-91: features first, then the terminator; ours fills every free slot
    c = config(3)
    rec = synth.records(c.game, 2000, seed=3)
    stm, nstm, buckets, targets = featurise(c.game, rec, c.desc)
    counts = np.array([bin(int(o)).count("1") for o in rec["occ"]])
    for idx in (stm, nstm):
        valid = idx >= 0
        assert (valid.sum(1) == counts).all()
        assert (valid[:, :-1] >= valid[:, 1:]).all()          # valid slots form a prefix
        assert idx[valid].max() < c.desc.n_inputs
        first_block = idx[:, :1] // 768
        assert ((idx // 768 == first_block) | ~valid).all()    # one king bucket per perspective
    assert (buckets == (counts - 2) // 4).all() and buckets.max() <= 7
    assert ((targets >= 0) & (targets <= 1)).all()


def test_fixture_records_from_the_reference(oracle32):
    # first 1024 records of the reference's examples/tests/batch.bf
    rec = np.fromfile(os.path.join(ROOT, "tests", "golden", "batch_head.bf"), dtype=synth.CHESS_DTYPE)
    assert len(rec) == 1024
    d768 = NetDesc(n_inputs=768, nnz=32, ft_out=16, ft_act=2)
    stm, nstm, _, _ = featurise("chess768", rec, d768)
    ostm, onstm = oracle32.map_chess(rec, 32)
    assert np.array_equal(stm, ostm) and np.array_equal(nstm, onstm)
    # our king is piece code 5 on `ksq`: feature 64*5 + ksq from our side
    assert ((stm == (320 + rec["ksq"].astype(np.int32))[:, None]).sum(1) == 1).all()
    # their king, seen from their side, stands on `opp_ksq` (chess_buckets.rs:82-88 relies on this frame)
    assert ((nstm == (320 + rec["opp_ksq"].astype(np.int32))[:, None]).sum(1) == 1).all()
    dbk = config(3).desc
    bstm, bnstm, buckets, _ = featurise("chess_buckets", rec, dbk)
    ob = oracle32.map_chess(rec, 32, KING_BUCKETS_16)
    assert np.array_equal(bstm, ob[0]) and np.array_equal(bnstm, ob[1])
    # un-bucketing and un-mirroring gives back the plain 768 features
    flip = np.where(rec["ksq"] % 8 > 3, 7, 0)[:, None]
    assert np.array_equal(np.where(bstm >= 0, (bstm % 768) ^ flip, -1), stm)


def test_index_packing_round_trip_is_bit_exact():
    c = config(1)
    rec = synth.records(c.game, 3000, seed=5)
    stm, nstm, _, _ = featurise(c.game, rec, c.desc)
    for idx in (stm, nstm):
        packed = pack_indices(idx)
        assert packed.dtype == np.uint16 and packed.shape == idx.shape
        assert np.array_equal(unpack_indices(packed), idx)
        assert ((packed == 0xFFFF) == (idx == -1)).all()
    # anything that is not a representable feature becomes "empty", as the kernels skip it anyway
    odd = np.array([0, 65534, 65535, 70000, -1, -7], dtype=np.int32)
    assert unpack_indices(pack_indices(odd)).tolist() == [0, 65534, -1, -1, -1, -1]
    assert pack_indices(np.zeros(0, np.int32)).size == 0


def test_too_many_features_is_an_error():
    rec = synth.records("chess768", 64, seed=1)
    d = NetDesc(n_inputs=768, nnz=4, ft_out=16, ft_act=2)
    with pytest.raises(_lib.B200Error) as e:
        featurise("chess768", rec, d)
    assert e.value.code == -4


def test_net_create_without_gpu_fails_loudly():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from bullet_b200.net import Net

    with pytest.raises(_lib.B200Error) as e:
        Net(config(0).desc)
    assert e.value.code == -3
