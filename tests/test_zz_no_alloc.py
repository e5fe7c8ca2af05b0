"""The allocation-free feature-transformer forward, collected last on purpose.

`b200_op_ft_forward_noalloc` exists for callers that cannot allocate device memory at call
time: a thread that evaluates positions on a GPU another thread is training on (a cudaMalloc
or cudaFree there would stall the trainer's streams), or a process that gave away all its
device memory up front.  It must return exactly what `b200_op_ft_forward` returns (both run
the same kernel in slot order, so the comparison is bit for bit), also on a second call that
finds the first call's leftovers in the shared scratch, and it must refuse batches beyond its
fixed scratch."""
import numpy as np
import pytest

from tests.test_gpu_ops import CASES, op_inputs, run_op

pytestmark = pytest.mark.gpu


def test_noalloc_matches_allocating_entry_point_twice(oracle32):
    name, desc, game = CASES[0]
    # two calls in a row with different sizes and data: the second one reuses the scratch
    for n, seed in ((3000, 71), (1234, 72)):
        stm, nstm, w, table, x_ref = op_inputs(oracle32, desc, game, n, seed)
        rc_a, x_a, u_a = run_op("b200_op_ft_forward", desc, table, w["l0b"], stm, nstm, n)
        rc_b, x_b, u_b = run_op("b200_op_ft_forward_noalloc", desc, table, w["l0b"], stm, nstm, n)
        assert rc_a == 0 and rc_b == 0
        assert np.array_equal(x_b, x_a) and np.array_equal(u_b, u_a)
        assert np.array_equal(x_b, x_ref)


def test_noalloc_other_activation_after_pairwise(oracle32):
    name, desc, game = CASES[1]
    stm, nstm, w, table, x_ref = op_inputs(oracle32, desc, game, 500, 73)
    rc, x, _ = run_op("b200_op_ft_forward_noalloc", desc, table, w["l0b"], stm, nstm, 500)
    assert rc == 0 and np.array_equal(x, x_ref)


def test_noalloc_refuses_more_than_its_scratch_holds(oracle32):
    from bullet_b200 import _lib

    name, desc, game = CASES[1]
    n = 16384 + 1
    stm, nstm, w, table, _ = op_inputs(oracle32, desc, game, n, 74)
    rc, _, _ = run_op("b200_op_ft_forward_noalloc", desc, table, w["l0b"], stm, nstm, n)
    assert rc == -1 and b"16384" in _lib.load().b200_last_error()
    rc, _, _ = run_op("b200_op_ft_forward_noalloc", desc, table, w["l0b"], stm[:16384], nstm[:16384], 16384)
    assert rc == 0


def test_noalloc_wide_index_lists_and_their_smaller_limit(oracle32):
    """More than 32 index slots per position (ataxx: 49) take twice the list space, so the fixed
    scratch holds half as many positions: 8192 run bit-exactly, 8193 are refused."""
    from bullet_b200 import _lib

    name, desc, game = CASES[2]
    assert desc.nnz == 49
    n = 8192
    stm, nstm, w, table, x_ref = op_inputs(oracle32, desc, game, n + 1, 75)
    rc, x, _ = run_op("b200_op_ft_forward_noalloc", desc, table, w["l0b"], stm[:n], nstm[:n], n)
    assert rc == 0 and np.array_equal(x, x_ref[:n])
    rc, _, _ = run_op("b200_op_ft_forward_noalloc", desc, table, w["l0b"], stm, nstm, n + 1)
    assert rc == -1 and b"8192" in _lib.load().b200_last_error()
    rc, x, _ = run_op("b200_op_ft_forward", desc, table, w["l0b"], stm, nstm, n + 1)   # the allocating entry takes it
    assert rc == 0 and np.array_equal(x, x_ref)
