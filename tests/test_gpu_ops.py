"""Operator-level GPU tests: the feature-transformer forward on caller-owned device memory,
called through the C ABI with torch tensors supplying the device pointers, against the oracle's
SparseMatmul + bias + activation composition (bit-exact, as the sums run in slot order)."""
import ctypes
import dataclasses

import numpy as np
import pytest

from bullet_b200 import synth
from bullet_b200.configs import ACT_CRELU, ACT_SCRELU, NetDesc

pytestmark = pytest.mark.gpu


def op_inputs(oracle32, desc, game, n, seed):
    """Host-side inputs and the oracle's expected x for `n` positions."""
    from tests.test_gpu_parity import oracle_ft_output, rich_weights

    rec = synth.records(game, n, seed=seed)
    stm, nstm, _, _ = oracle32.map_batch(game, rec, desc)
    w = rich_weights(desc)
    table = w["l0w"].copy()
    if desc.factoriser_rows:
        table = table + np.tile(w["l0f"], desc.n_inputs // desc.factoriser_rows)
    return stm, nstm, w, table, oracle_ft_output(oracle32, desc, w, stm, nstm)


def run_op(entry, desc, table, bias, stm, nstm, n):
    """Calls `entry` (a b200_op_ft_forward-style symbol) on torch-owned device buffers; returns (rc, x, u)."""
    import torch

    from bullet_b200 import _lib
    from bullet_b200.net import pack_indices

    dev = torch.device("cuda", 0)
    t_table = torch.from_numpy(np.ascontiguousarray(table, dtype=np.float32)).to(dev)
    t_bias = torch.from_numpy(np.ascontiguousarray(bias, dtype=np.float32)).to(dev)
    t_stm = torch.from_numpy(pack_indices(stm).view(np.int16)).to(dev)
    t_nstm = torch.from_numpy(pack_indices(nstm).view(np.int16)).to(dev)
    d1 = desc.ft_out if desc.pairwise else 2 * desc.ft_out
    t_x = torch.full((n, d1), float("nan"), device=dev)
    t_u = torch.full((n, 2, desc.ft_out), float("nan"), device=dev) if desc.pairwise else None
    op = _lib.CFtOp(desc.n_inputs, desc.nnz, desc.ft_out, desc.ft_act, int(desc.pairwise), desc.ft_block_rows, n,
                    t_table.data_ptr(), t_bias.data_ptr(), t_stm.data_ptr(), t_nstm.data_ptr(), t_x.data_ptr(),
                    t_u.data_ptr() if t_u is not None else None)
    torch.cuda.synchronize()
    rc = getattr(_lib.load(), entry)(0, None, ctypes.byref(op))
    torch.cuda.synchronize()
    return rc, t_x.cpu().numpy(), None if t_u is None else t_u.cpu().numpy()


CASES = [
    ("pairwise", NetDesc(n_inputs=12288, nnz=32, ft_out=128, ft_act=ACT_CRELU, pairwise=True, factoriser_rows=768,
                         n_out_buckets=8, dense_out=(16, 32, 1), dense_act=(2, 2, 0), ft_block_rows=768), "chess_buckets"),
    ("screlu", NetDesc(n_inputs=768, nnz=32, ft_out=128, ft_act=ACT_SCRELU, ft_block_rows=768), "chess768"),
    ("ataxx", NetDesc(n_inputs=147, nnz=49, ft_out=64, ft_act=ACT_CRELU, ft_block_rows=147), "ataxx147"),
]


@pytest.mark.parametrize("name,desc,game", CASES, ids=[c[0] for c in CASES])
def test_op_ft_forward_bit_exact(oracle32, name, desc, game):
    n = 777
    stm, nstm, w, table, x_ref = op_inputs(oracle32, desc, game, n, seed=61)
    rc, x, u = run_op("b200_op_ft_forward", desc, table, w["l0b"], stm, nstm, n)
    assert rc == 0
    assert np.array_equal(x, x_ref)
    if desc.pairwise:
        h = desc.ft_out // 2
        assert np.array_equal(u[:, 0, :h] * u[:, 0, h:], x[:, :h]) and np.array_equal(u[:, 1, :h] * u[:, 1, h:], x[:, h:])
        assert u.min() >= 0 and u.max() <= 1


def test_op_ft_forward_errors(oracle32):
    from bullet_b200 import _lib

    name, desc, game = CASES[0]
    n = 64
    stm, nstm, w, table, _ = op_inputs(oracle32, desc, game, n, seed=62)
    bad = stm.copy()
    bad[5, 1] = (bad[5, 0] + 768 * 5) % 12288        # a feature from another king bucket
    rc, _, _ = run_op("b200_op_ft_forward", desc, table, w["l0b"], bad, nstm, n)
    assert rc == -4 and b"row block" in _lib.load().b200_last_error()
    rc, _, _ = run_op("b200_op_ft_forward", dataclasses.replace(desc, ft_block_rows=0), table, w["l0b"], stm, nstm, n)
    assert rc == -5
    lib = _lib.load()
    assert lib.b200_op_ft_forward(0, None, None) == -1
