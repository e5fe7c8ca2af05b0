"""Network export (SavedFormat): C library against the numpy restatement and hand-computed cases.

Reference: crates/trainer/src/model/weights.rs:158-335, crates/bullet_lib/src/value/save.rs:24-88.
"""
import dataclasses
import os

import numpy as np
import pytest

from bullet_b200 import _lib, config, synth
from bullet_b200.saved_format import SavedFormat, quantise, transpose
from oracle import saved_format as ref


def test_quantise_hand_cases():
    # 255 * 0.5 = 127.5 -> 128 rounded (half away from zero), 127 truncated; negatives mirror
    v = np.array([0.5, -0.5, 0.25, -0.25, 0.0, 1.0 / 255.0], dtype=np.float32)
    assert quantise(v, "i16", 255, round=True).tolist() == [128, -128, 64, -64, 0, 1]
    assert quantise(v, "i16", 255, round=False).tolist() == [127, -127, 63, -63, 0, 1]
    # exact ties at small multipliers
    t = np.array([0.25, -0.25, 0.75, -0.75, 1.25], dtype=np.float32)
    assert quantise(t, "i8", 2, round=True).tolist() == [1, -1, 2, -2, 3]
    assert quantise(t, "i8", 2, round=False).tolist() == [0, 0, 1, -1, 2]
    # i8 takes an i16 multiplier: 0.99 * 128 = 126.72
    assert quantise(np.array([0.99, -0.99], dtype=np.float32), "i8", 128, round=True).tolist() == [127, -127]
    assert quantise(v, "f32", 1).tobytes() == v.tobytes()
    assert quantise(np.array([], dtype=np.float32), "i32", 7).size == 0


@pytest.mark.parametrize("target,mult", [("i8", 64), ("i16", 255), ("i16", 255 * 64), ("i32", 65536)])
@pytest.mark.parametrize("rnd", [False, True])
def test_quantise_matches_oracle(target, mult, rnd):
    rng = np.random.default_rng(hash((target, mult, rnd)) % 2**32)
    info = np.iinfo(ref.DTYPES[target])
    v = rng.uniform(-0.98, 0.98, 20000).astype(np.float32) * np.float32(min(1.0, info.max / mult))
    v[:64] = (np.arange(64, dtype=np.float32) - 32.0 + 0.5) / np.float32(mult)  # near-ties
    assert quantise(v, target, mult, round=rnd).tobytes() == ref.quantise(v, target, mult, rnd)


@pytest.mark.parametrize("bad", [1.0, -1.01, float("nan"), float("inf")])
def test_quantise_that_does_not_fit_fails(bad):
    v = np.array([0.1, bad], dtype=np.float32)
    with pytest.raises(ref.QuantisationError):
        ref.quantise(v, "i8", 128, True)
    with pytest.raises(_lib.B200Error) as e:
        quantise(v, "i8", 128, round=True)
    assert e.value.code == -4 and "Failed quantisation from f32 to i8!" in str(e.value)


def test_quantise_argument_errors():
    v = np.zeros(4, dtype=np.float32)
    out = np.zeros(4, dtype=np.int32)
    lib = _lib.load()
    assert lib.b200_quantise(v.ctypes.data, 4, 9, 1, 0, out.ctypes.data) == -1
    assert lib.b200_quantise(v.ctypes.data, 4, 2, 40000, 0, out.ctypes.data) == -1  # an i16 multiplier
    assert lib.b200_quantise(None, 4, 2, 1, 0, out.ctypes.data) == -1
    assert [lib.b200_quant_size(q) for q in (0, 1, 2, 3, 4)] == [4, 1, 2, 4, 0]


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 5), (16, 2048), (128, 7)])
def test_transpose_matches_oracle(rows, cols):
    w = np.random.default_rng(rows * 31 + cols).normal(size=rows * cols).astype(np.float32)
    got = transpose(w, rows, cols)
    assert np.array_equal(got, ref.transpose_impl(rows, cols, w))
    # column-major rows x cols -> row-major rows x cols
    assert np.array_equal(got.reshape(rows, cols), w.reshape(cols, rows).T)


def test_builder_mirrors_the_reference_rules():
    f = SavedFormat.id("l1w").round().quantise("i16", 64).transpose()
    assert (f.weight, f.quant, f.multiplier, f.rounded, f.transposed) == ("l1w", 2, 64, True, True)
    with pytest.raises(ValueError):
        SavedFormat.custom(b"x").round()
    with pytest.raises(ValueError):
        SavedFormat.custom(b"x").quantise("i8", 1)


def _net_and_weights():
    from bullet_b200 import Net

    c = config(3)
    desc = dataclasses.replace(c.desc, ft_out=128, max_batch=64)
    w = synth.init_weights(desc, seed=5)
    w["l0f"] = np.random.default_rng(1).uniform(-0.3, 0.3, w["l0f"].size).astype(np.float32)
    net = Net(desc)
    net.load_weights(w)
    return net, desc, w


FORMATS = [  # examples/progression/4_multi_layer.rs:47-63 with a header in front
    (SavedFormat.custom(b"NNUE\x01"), {"custom": b"NNUE\x01"}),
    (SavedFormat.id("l0w").merge_factoriser().round().quantise("i16", 255),
     {"id": "l0w", "merge_factoriser": True, "round": True, "quant": "i16", "multiplier": 255}),
    (SavedFormat.id("l0b").round().quantise("i16", 255), {"id": "l0b", "round": True, "quant": "i16", "multiplier": 255}),
    (SavedFormat.id("l1w").transpose().round().quantise("i8", 64),
     {"id": "l1w", "transpose": True, "round": True, "quant": "i8", "multiplier": 64}),
    (SavedFormat.id("l1b"), {"id": "l1b"}),
    (SavedFormat.id("l2w").transpose(), {"id": "l2w", "transpose": True}),
    (SavedFormat.id("l2b"), {"id": "l2b"}),
    (SavedFormat.id("l3w").transpose().quantise("i32", 1 << 16), {"id": "l3w", "transpose": True, "quant": "i32", "multiplier": 1 << 16}),
    (SavedFormat.id("l3b"), {"id": "l3b"}),
]


@pytest.mark.gpu
def test_export_of_a_network_matches_the_oracle(tmp_path):
    net, desc, w = _net_and_weights()
    shapes = {k: net.tensor_shape(k) for k in w}
    assert shapes["l0w"] == (desc.ft_out, desc.n_inputs) and shapes["l0f"] == (desc.ft_out, 768)
    assert shapes["l1w"] == (8 * 16, desc.ft_out) and shapes["l1b"] == (8 * 16, 1)
    ours = [f for f, _ in FORMATS]
    theirs = [d for _, d in FORMATS]
    for pad in (False, True):
        want = ref.to_quantised_buffer(w, shapes, theirs, pad)
        assert net.to_quantised_buffer(ours, pad) == want
    bare = ref.to_quantised_buffer(w, shapes, theirs, False)
    assert len(want) % 64 == 0 and len(want) - len(bare) < 64 and want[len(bare):] == (b"bullet" * 11)[:len(want) - len(bare)]
    # the checkpoint folder of save.rs:24-43
    path = str(tmp_path / "net-10")
    net.save_to_checkpoint(path, ours)
    assert open(os.path.join(path, "quantised.bin"), "rb").read() == want
    assert open(os.path.join(path, "raw.bin"), "rb").read() == ref.unquantised_buffer(w, theirs)
    assert sorted(os.listdir(os.path.join(path, "optimiser_state"))) == ["momentum.bin", "velocity.bin", "weights.bin"]
    # the weights moved through a training step are what gets exported
    from bullet_b200.net import featurise

    game = config(3).game
    net.upload(0, *featurise(game, synth.records(game, 64, seed=9), desc))
    net.step(0, 1e-2, 1.0 / 64)
    net.loss()
    w2 = net.tensors(0)
    assert net.to_quantised_buffer(ours, True) == ref.to_quantised_buffer(w2, shapes, theirs, True)
    net.close()


@pytest.mark.gpu
def test_export_fails_loudly_when_a_weight_does_not_fit():
    net, desc, w = _net_and_weights()
    w["l0b"][3] = 200.0  # 200 * 255 > i16
    net.load_weights(w)
    with pytest.raises(_lib.B200Error) as e:
        net.to_quantised_buffer([SavedFormat.id("l0b").round().quantise("i16", 255)])
    assert e.value.code == -4 and "i16" in str(e.value)
    with pytest.raises(_lib.B200Error):
        net.to_quantised_buffer([SavedFormat.id("nope")])
    with pytest.raises(_lib.B200Error):  # the factoriser goes with tables it tiles
        net.to_quantised_buffer([SavedFormat.id("l1b").merge_factoriser()])
    net.close()
