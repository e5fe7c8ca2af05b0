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
    """The engine interface of bullet_b200.dp implemented with the CPU oracle (test only).

    Flat gradient layout as in the library: [loss, padding][all tensors but l0w][l0w]."""

    HEAD = 64

    def __init__(self, desc, weights, hp):
        from oracle import Oracle

        self.orc = Oracle("f32")
        self.desc, self.hp = desc, hp
        self.names = [k for k in desc.tensor_shapes() if k != "l0w"] + ["l0w"]
        self.offsets, at = {}, self.HEAD
        for k in self.names:
            self.offsets[k] = at
            at += weights[k].size
        total = (at + 1023) // 1024 * 1024
        self.flat = {kind: np.zeros(total, np.float32) for kind in ("w", "m", "v")}
        view = lambda kind: {k: self.flat[kind][self.offsets[k]:self.offsets[k] + weights[k].size] for k in self.names}  # noqa: E731
        self.w, self.m, self.v = view("w"), view("m"), view("v")
        for k in self.names:
            self.w[k][:] = weights[k]
        self.grad = torch.zeros(total, dtype=torch.float32)
        self.param = torch.from_numpy(self.flat["w"])
        self.slots = {}

    def state_buffers(self):
        return [torch.from_numpy(self.flat["m"]), torch.from_numpy(self.flat["v"])]

    def upload(self, slot, *batch):
        self.slots[slot] = batch

    # ---- one-piece form
    def backward(self, slot):
        loss, g, _ = self.orc.net_grad(self.desc, self.w, *self.slots[slot])
        flat = self.grad.numpy()
        flat[:] = 0
        flat[0] = loss
        for k in self.names:
            flat[self.offsets[k]:self.offsets[k] + g[k].size] = g[k]

    def update(self, lr, grad_factor):
        self.update_range(lr, grad_factor, 0, self.grad.numel())
        self.update_end()

    # ---- phased form: the oracle computes everything at once, the phases only expose the ranges
    def forward_begin(self, slot):
        self.forward_parts = []

    def forward_ft(self, slot, part, n_parts):
        # a forward slice may only run once the gather of that slice of l0w has landed: remember what it saw
        lo = self.offsets["l0w"] + part * (self.w["l0w"].size // n_parts)
        self.forward_parts.append(self.flat["w"][lo:lo + self.w["l0w"].size // n_parts].copy())

    def tensor_range(self, name):
        return self.offsets[name], self.w[name].size

    def backward_begin(self, slot):
        if getattr(self, "forward_parts", None):  # the weights the forward slices saw are the weights now
            assert np.array_equal(np.concatenate(self.forward_parts), self.w["l0w"])
            self.forward_parts = []
        self.backward(slot)

    def backward_ft(self, slot, part, n_parts):
        pass

    def backward_end(self, slot):
        pass

    def grad_part(self, part, n_parts):
        lo = self.offsets["l0w"]
        if part == n_parts:
            return 0, lo
        per = self.w["l0w"].size // n_parts
        return lo + part * per, per

    def update_range(self, lr, grad_factor, first, count):
        flat = self.grad.numpy()
        self.last_loss = float(flat[0])
        for k in self.names:
            lo, n = self.offsets[k], self.w[k].size
            a, b = max(lo, first), min(lo + n, first + count)
            if a >= b:
                continue
            sl = slice(a - lo, b - lo)
            p, m, v = (np.ascontiguousarray(t[k][sl]) for t in (self.w, self.m, self.v))
            self.orc.adamw(p, m, v, np.ascontiguousarray(flat[a:b]), grad_factor, lr, self.hp)
            self.w[k][sl], self.m[k][sl], self.v[k][sl] = p, m, v

    def update_end(self):
        pass

    # ---- the one-kernel exchange over peer memory, emulated with collectives: what it must compute
    def exchange_export(self):
        return bytes(192)

    def exchange_import(self, rank, world, handles):
        assert len(handles) == 192 * world
        self.xch = (rank, world)

    def update_exchange(self, lr, grad_factor):
        rank, world = self.xch
        per = self.grad.numel() // world
        dist.all_reduce(self.grad)
        self.update_range(lr, grad_factor, rank * per, per)
        dist.all_gather_into_tensor(self.param, self.param[rank * per:(rank + 1) * per].clone())


def _worker(rank, world, port, out_dir, parts, shard, peer=False):
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
    dp = DataParallelStep(eng, global_batch=256, parts=parts, shard_optimiser=shard, peer_exchange=peer)
    losses = []
    for step in range(3):
        full = orc.map_batch(c.game, synth.records(c.game, 256, seed=50 + step), desc)
        eng.upload(0, *shard_batch(full, rank, world))
        dp.step(0, 1e-3)
        losses.append(eng.last_loss)
    dp.gather_state()
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), losses=np.array(losses), m_l0w=eng.m["l0w"], **eng.w)
    dist.destroy_process_group()


@pytest.mark.parametrize("parts,shard,peer,world", [(1, False, False, 2), (4, False, False, 2), (1, True, False, 2),
                                                    (4, True, False, 2), (1, False, True, 2), (4, True, False, 4)])
def test_data_parallel_ranks_match_single_rank(tmp_path, parts, shard, peer, world):
    from bullet_b200 import config, synth
    from bullet_b200.configs import AdamWParams
    from bullet_b200.dp import shard_bounds
    from oracle import Oracle

    assert shard_bounds(8, 1, 2) == (4, 8)
    with pytest.raises(ValueError):
        shard_bounds(7, 0, 2)
    port = 29500 + (os.getpid() + 7 * parts + 3 * shard + 11 * peer + 17 * world) % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path), parts, shard, peer), nprocs=world, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / f"rank{world - 1}.npz")
    c = config(3)
    desc = dataclasses.replace(c.desc, ft_out=64, max_batch=256)
    orc = Oracle("f32")
    batches = [orc.map_batch(c.game, synth.records(c.game, 256, seed=50 + s), desc) for s in range(3)]
    w_ref, m_ref, _, losses_ref = orc.train(desc, synth.init_weights(desc, seed=3), batches, 1e-3, AdamWParams())
    np.testing.assert_allclose(r0["losses"], losses_ref, rtol=1e-5)
    for k in w_ref:
        assert np.array_equal(r0[k], r1[k]), f"replicas differ in {k}"
        err = np.linalg.norm(r0[k].astype(np.float64) - w_ref[k]) / max(np.linalg.norm(w_ref[k]), 1e-30)
        assert err <= 1e-4, (k, err)
    # after gather_state both ranks hold the complete momentum, sharded optimiser or not
    assert np.array_equal(r0["m_l0w"], r1["m_l0w"])
    assert np.linalg.norm(r0["m_l0w"] - m_ref["l0w"]) <= 1e-4 * np.linalg.norm(m_ref["l0w"])
