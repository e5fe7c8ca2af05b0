"""CPU tests that pin the oracle: the reference's own known-answer vectors, an independent
autograd cross-check of the whole-net backward pass, and AdamW against its formula."""
import json
import os

import numpy as np
import pytest

from bullet_b200 import synth
from bullet_b200.configs import ACT_CRELU, ACT_NONE, ACT_SCRELU, AdamWParams, NetDesc, config

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))


def test_kat_sparse_matmul(oracle32):
    g = GOLD["sparse_matmul"]
    out = oracle32.sparse_matmul(g["weights"], g["indices"], g["batch"], g["rows"], g["cols"], g["stride"],
                                 g["offset"], g["nnz"])
    assert out.tolist() == g["expected"]


def test_kat_sparse_matmul_bwd(oracle32):
    g = GOLD["sparse_matmul_bwd_multi"]
    out = oracle32.sparse_matmul_bwd_multi([(g["grads"], g["indices"], g["offset"])], g["batch"], g["rows"],
                                           g["cols"], g["stride"], g["nnz"])
    assert out.tolist() == g["expected"]


def test_kat_matmul_layouts(oracle32):
    g = GOLD["matmul"]
    for case in g["cases"]:
        out = oracle32.matmul(g["lhs"], g["rhs"], g["batch"], g["m"], g["n"], g["k"], case["lhs_col_mjr"],
                              case["rhs_col_mjr"], integer=True)
        assert out.tolist() == case["expected"]


def test_kat_select_and_pad(oracle32):
    g = GOLD["select"]
    assert oracle32.select(g["input"], g["indices"], g["batch"], g["inner"], g["divisor"], True).tolist() == \
        g["expected"]
    g = GOLD["select_pad"]
    assert oracle32.select_pad(g["input"], g["indices"], g["batch"], g["inner"], g["divisor"], True).tolist() == \
        g["expected"]
    g = GOLD["select_inverse"]
    x = np.arange(64)
    idx = np.tile(np.arange(4), 4)
    padded = oracle32.select_pad(x, idx, g["batch"], g["inner"], g["divisor"], True)
    assert oracle32.select(padded, idx, g["batch"], g["inner"], g["divisor"], True).tolist() == x.tolist()


def test_kat_reduce_and_broadcast(oracle32):
    x = np.arange(64)
    assert oracle32.reduce_sum(x, 1, 8, 8, True).tolist() == [224 + 8 * i for i in range(8)]
    assert oracle32.reduce_sum(x, 8, 2, 4, True).tolist() == [4 + 2 * (i % 4) + 16 * (i // 4) for i in range(32)]
    assert oracle32.reduce_sum(x, 16, 4, 1, True).tolist() == [6 + 16 * i for i in range(16)]
    b = GOLD["broadcast"]
    y = np.arange(8)
    assert oracle32.broadcast(y, 1, 8, 2, True).tolist() == b["shape2"]["rows"]
    assert oracle32.broadcast(y, 2, 4, 2, True).tolist() == b["shape2"]["cols"]
    assert oracle32.broadcast(y, 1, 8, 2, True).tolist() == b["shape3"]["leading"]
    assert oracle32.broadcast(y, 2, 4, 2, True).tolist() == b["shape3"]["middle"]
    assert oracle32.broadcast(y, 4, 2, 2, True).tolist() == b["shape3"]["trailing"]


def test_activation_rules(oracle32):
    # dfo.rs:56-88: strict inequalities, derivative taken from the OUTPUT value
    x = np.array([-1.0, 0.0, 0.25, 1.0, 2.0], dtype=np.float32)
    assert oracle32.act_forward(ACT_CRELU, x).tolist() == [0.0, 0.0, 0.25, 1.0, 1.0]
    assert oracle32.act_forward(ACT_SCRELU, x).tolist() == [0.0, 0.0, 0.0625, 1.0, 1.0]
    ones = np.ones(5, dtype=np.float32)
    assert oracle32.act_backward(ACT_CRELU, oracle32.act_forward(ACT_CRELU, x), ones).tolist() == [0, 0, 1, 0, 0]
    assert oracle32.act_backward(ACT_SCRELU, oracle32.act_forward(ACT_SCRELU, x), ones).tolist() == \
        [0, 0, 0.5, 0, 0]


def test_adamw_formula(oracle32, oracle64):
    rng = np.random.default_rng(3)
    n = 1000
    hp = AdamWParams(max_weight=0.05, min_weight=-0.05)
    p0, g = rng.normal(0, 0.05, n), rng.normal(0, 1, n)
    m0, v0 = rng.normal(0, 0.1, n), rng.random(n)
    adj, lr = 1.0 / 16384, 1e-3
    # every scalar reaches the kernel as an f32 (adam.rs:97-110 formats them into the source)
    f = lambda v: float(np.float32(v))  # noqa: E731
    gg = f(adj) * g
    pe = p0 * (1 - f(hp.decay) * f(lr))
    me = f(hp.beta1) * m0 + (1 - f(hp.beta1)) * gg
    ve = f(hp.beta2) * v0 + (1 - f(hp.beta2)) * gg * gg
    pe = np.clip(pe - f(lr) * me / (np.sqrt(ve) + f(1e-8)), f(hp.min_weight), f(hp.max_weight))
    for orc, tol in ((oracle64, 1e-12), (oracle32, 1e-6)):
        p, m, v = (np.array(a, dtype=orc.real) for a in (p0, m0, v0))
        orc.adamw(p, m, v, np.array(g, dtype=orc.real), adj, lr, hp)
        np.testing.assert_allclose(p, pe, rtol=tol, atol=tol)
        np.testing.assert_allclose(m, me, rtol=tol, atol=tol)
        np.testing.assert_allclose(v, ve, rtol=tol, atol=tol)
    assert np.any(pe == f(hp.max_weight)) and np.any(pe == f(hp.min_weight))


def _small_nets():
    yield "simple", NetDesc(n_inputs=768, nnz=32, ft_out=16, ft_act=ACT_SCRELU), "chess768"
    yield "ataxx", NetDesc(n_inputs=147, nnz=49, ft_out=24, ft_act=ACT_CRELU), "ataxx147"
    yield "bucketed", NetDesc(n_inputs=12288, nnz=32, ft_out=32, ft_act=ACT_SCRELU, factoriser_rows=768,
                              n_out_buckets=8), "chess_buckets"
    yield "pairwise", NetDesc(n_inputs=12288, nnz=32, ft_out=64, ft_act=ACT_CRELU, pairwise=True,
                              factoriser_rows=768, n_out_buckets=8, dense_out=(16, 32, 1),
                              dense_act=(ACT_SCRELU, ACT_SCRELU, ACT_NONE)), "chess_buckets"


@pytest.mark.parametrize("name,desc,game", list(_small_nets()), ids=[n for n, _, _ in _small_nets()])
def test_net_grad_matches_autograd(oracle64, oracle32, name, desc, game):
    from tests import torch_ref

    B = 96
    rec = synth.records(game, B, seed=11)
    stm, nstm, buckets, targets = oracle64.map_batch(game, rec, desc)
    w = synth.init_weights(desc, seed=5, ft_fan_in=8)
    rng = np.random.default_rng(9)
    for k in w:  # non-zero biases and factoriser so every path carries signal
        if k.endswith("b") or k == "l0f":
            w[k] = rng.normal(0, 0.05, w[k].size).astype(np.float32)
    loss64, g64, out64 = oracle64.net_grad(desc, w, stm, nstm, buckets, targets)
    tl, tg, tout = torch_ref.grads(desc, w, stm, nstm, buckets, targets)
    assert abs(loss64 - tl) <= 1e-10 * abs(tl)
    np.testing.assert_allclose(out64, tout, rtol=1e-10, atol=1e-12)
    for k in g64:
        np.testing.assert_allclose(g64[k], tg[k], rtol=1e-9, atol=1e-11, err_msg=k)
        assert np.abs(g64[k]).max() > 0, k
    # fp32 oracle agrees with the arbiter to fp32 accuracy
    loss32, g32, _ = oracle32.net_grad(desc, w, stm, nstm, buckets, targets)
    assert abs(loss32 - loss64) <= 1e-5 * abs(loss64)
    for k in g64:
        scale = np.abs(g64[k]).max()
        assert np.abs(g32[k] - g64[k]).max() <= 2e-5 * scale, k


def test_invalid_indices_are_skipped(oracle32):
    # sparse.rs:107-112: out-of-range and negative slots are skipped, later slots still count
    desc = NetDesc(n_inputs=768, nnz=32, ft_out=16, ft_act=ACT_SCRELU)
    rec = synth.records("chess768", 8, seed=2)
    stm, nstm, buckets, targets = oracle32.map_batch("chess768", rec, desc)
    w = synth.init_weights(desc, seed=1, ft_fan_in=8)
    l0, _, _ = oracle32.net_grad(desc, w, stm, nstm, buckets, targets, want_grads=False)
    stm2 = np.concatenate([np.full((8, 1), -1, np.int32), stm[:, :-1]], 1)  # leading terminator
    stm2[:, -1] = 9999                                                         # out of range
    assert (stm[:, -1] == -1).all()
    l1, _, _ = oracle32.net_grad(desc, w, stm2, nstm, buckets, targets, want_grads=False)
    assert l0 == l1


def test_thread_count_does_not_change_results(oracle32):
    c = config(3)
    desc = NetDesc(**{**c.desc.__dict__, "ft_out": 64, "max_batch": 256})
    rec = synth.records(c.game, 256, seed=4)
    batch = oracle32.map_batch(c.game, rec, desc)
    w = synth.init_weights(desc, seed=1)
    os.environ["OMP_NUM_THREADS"] = "8"
    a = oracle32.net_grad(desc, w, *batch)
    oracle32.lib.omp_set_num_threads(1)
    b = oracle32.net_grad(desc, w, *batch)
    oracle32.lib.omp_set_num_threads(oracle32.threads() or 8)
    assert a[0] == b[0]
    for k in a[1]:
        assert np.array_equal(a[1][k], b[1][k]), k


def test_radam_schedule_and_update_against_numpy(oracle32):
    """RAdam's host-side schedule (radam.rs:295-314) and element update (radam.rs:35-52) against the same formulas
    written out in numpy float32; the first five steps use no second-moment division (n_sma <= 5)."""
    from bullet_b200.configs import AdamWParams

    f = np.float32
    b1, b2, thr = f(0.9), f(0.999), f(5.0)
    flags = []
    for step in range(1, 12):
        t = f(step)
        b2t = np.power(b2, t, dtype=np.float32)
        nmax = f(2.0) / (f(1.0) - b2) - f(1.0)
        nsma = nmax - f(2.0) * t * b2t / (f(1.0) - b2t)
        denom = f(1.0) - np.power(b1, t, dtype=np.float32)
        if nsma > thr:
            size = np.sqrt((f(1.0) - b2t) * ((nsma - f(4.0)) / (nmax - f(4.0))) * ((nsma - f(2.0)) / nsma) * (nmax / (nmax - f(2.0)))) / denom
        else:
            size = f(1.0) / denom
        got, flag = oracle32.radam_step(step, 0.9, 0.999)
        assert flag == int(nsma > thr)
        # n_sma is a difference of two numbers near 2000 in f32: one ulp of powf moves it by 1e-3 relative, so the
        # two libraries' powf may only be held together this loosely
        assert abs(got - float(size)) <= 5e-3 * abs(float(size)), (step, got, size)
        flags.append(flag)
    assert flags[:5] == [0] * 5 and flags[5:] == [1] * 6
    hp = AdamWParams(decay=0.01, beta1=0.9, beta2=0.999, min_weight=-0.5, max_weight=0.5)
    for use_denom in (0, 1):
        p, m, v = np.array([0.4, -0.2], np.float32), np.array([0.01, 0.0], np.float32), np.array([1e-4, 0.0], np.float32)
        g = np.array([8.0, -4.0], np.float32)
        rate, adj = f(0.05), f(0.25)
        gg = adj * g
        pe = p * (f(1) - f(0.01) * rate)
        me = f(0.9) * m + (f(1) - f(0.9)) * gg
        ve = f(0.999) * v + (f(1) - f(0.999)) * gg * gg
        val = me / (np.sqrt(ve) + f(1e-8)) if use_denom else me
        pe = np.clip(pe - rate * val, f(-0.5), f(0.5))
        oracle32.radam(p, m, v, g, 0.25, 0.05, use_denom, hp)
        np.testing.assert_allclose(p, pe, rtol=1e-6)
        np.testing.assert_allclose(m, me, rtol=1e-6)
        np.testing.assert_allclose(v, ve, rtol=1e-6)


def test_lookahead_pulls_fast_weights_to_slow_ones(oracle32):
    """ranger.rs:23-43: w = alpha * w + (1 - alpha) * slow, and slow takes the same value."""
    w, slow = np.array([1.0, -2.0, 0.5], np.float32), np.array([0.0, 2.0, 0.5], np.float32)
    oracle32.lookahead(w, slow, 0.25)
    assert np.array_equal(w, np.array([0.25, 1.0, 0.5], np.float32)) and np.array_equal(w, slow)
