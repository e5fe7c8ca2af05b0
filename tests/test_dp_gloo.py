"""Data-parallel host logic on CPU: two gloo ranks, the oracle as the compute engine.

Checks that sharding + one sum all-reduce of the flat gradient buffer + AdamW with
grad_factor = 1/global batch reproduces the single-rank result, that the loss rides the same
collective, and that the replicas stay bit-identical."""
import dataclasses
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleEngine:
    """The engine interface of bullet_b200.dp implemented with the CPU oracle (test only)."""

    def __init__(self, desc, weights, hp):
        from oracle import Oracle

        self.orc = Oracle("f32")
        self.desc, self.hp = desc, hp
        self.w = self.orc.to_real(weights)
        self.m, self.v = self.orc.zeros_like(desc), self.orc.zeros_like(desc)
        self.names = list(desc.tensor_shapes())
        self.sizes = [self.w[k].size for k in self.names]
        self.grad = torch.zeros(sum(self.sizes) + 1, dtype=torch.float32)
        self.slots = {}

    def upload(self, slot, *batch):
        self.slots[slot] = batch

    def backward(self, slot):
        loss, g, _ = self.orc.net_grad(self.desc, self.w, *self.slots[slot])
        flat = np.concatenate([g[k] for k in self.names] + [np.array([loss], np.float32)])
        self.grad.copy_(torch.from_numpy(flat))

    def update(self, lr, grad_factor):
        flat = self.grad.numpy()
        g, at = {}, 0
        for k, n in zip(self.names, self.sizes):
            g[k] = np.ascontiguousarray(flat[at:at + n])
            at += n
        self.last_loss = float(flat[-1])
        self.orc.net_update(self.desc, self.w, self.m, self.v, g, grad_factor, lr, self.hp)


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from bullet_b200 import config, synth
    from bullet_b200.configs import AdamWParams
    from bullet_b200.dp import DataParallelStep, shard_batch
    from oracle import Oracle

    c = config(3)
    desc = dataclasses.replace(c.desc, ft_out=64, max_batch=256)
    orc = Oracle("f32")
    weights = synth.init_weights(desc, seed=3)
    eng = OracleEngine(desc, weights, AdamWParams())
    dp = DataParallelStep(eng, global_batch=256)
    losses = []
    for step in range(3):
        full = orc.map_batch(c.game, synth.records(c.game, 256, seed=50 + step), desc)
        eng.upload(0, *shard_batch(full, rank, world))
        dp.step(0, 1e-3)
        losses.append(eng.last_loss)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), losses=np.array(losses), **eng.w)
    dist.destroy_process_group()


def test_two_rank_data_parallel_matches_single_rank(tmp_path):
    from bullet_b200 import config, synth
    from bullet_b200.configs import AdamWParams
    from bullet_b200.dp import shard_bounds
    from oracle import Oracle

    assert shard_bounds(8, 1, 2) == (4, 8)
    with pytest.raises(ValueError):
        shard_bounds(7, 0, 2)
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    c = config(3)
    desc = dataclasses.replace(c.desc, ft_out=64, max_batch=256)
    orc = Oracle("f32")
    batches = [orc.map_batch(c.game, synth.records(c.game, 256, seed=50 + s), desc) for s in range(3)]
    w_ref, _, _, losses_ref = orc.train(desc, synth.init_weights(desc, seed=3), batches, 1e-3, AdamWParams())
    np.testing.assert_allclose(r0["losses"], losses_ref, rtol=1e-5)
    for k in w_ref:
        assert np.array_equal(r0[k], r1[k]), f"replicas differ in {k}"
        err = np.linalg.norm(r0[k].astype(np.float64) - w_ref[k]) / max(np.linalg.norm(w_ref[k]), 1e-30)
        assert err <= 1e-4, (k, err)
