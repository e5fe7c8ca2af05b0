"""Data-parallel training step over the ranks of one box.

Positions are independent, so a global batch is cut into equal contiguous shards, one per
rank; every rank holds a full replica of the weights and the optimiser state.  The only
exchange is one sum all-reduce of the flat gradient buffer (whose last element carries the
summed loss) between the backward pass and the AdamW update; the update then runs on every
replica with grad_factor = 1 / global batch, which keeps the replicas bit-identical.

The reference has no multi-GPU path (one device chosen by ordinal,
crates/bullet_lib/src/value/builder.rs:97-100); this module is new work on top of its step
loop (crates/trainer/src/run.rs:166-250).  `torch.distributed` supplies the process group:
NCCL over NVLink on GPUs, gloo in the CPU tests.
"""
from __future__ import annotations

import numpy as np


def shard_bounds(n_global: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous shard [begin, end) of rank `rank`; the global batch must divide evenly."""
    if n_global % world:
        raise ValueError(f"global batch {n_global} does not divide over {world} ranks")
    per = n_global // world
    return rank * per, (rank + 1) * per


def shard_batch(batch, rank: int, world: int):
    """Slice (stm, nstm, buckets, targets) to this rank's positions."""
    n = len(batch[3])
    lo, hi = shard_bounds(n, rank, world)
    return tuple(None if a is None else np.ascontiguousarray(a[lo:hi]) for a in batch)


class DataParallelStep:
    """Runs backward -> all-reduce -> update on an engine.

    The engine is anything with the calls of `bullet_b200.net.Net` used here: `backward(slot)`,
    `update(lr, grad_factor)` and a `grad` attribute holding a torch tensor that aliases the
    flat gradient buffer (loss in its last element).
    """

    def __init__(self, engine, global_batch: int, process_group=None):
        import torch.distributed as dist

        self.engine = engine
        self.global_batch = global_batch
        self.group = process_group
        self.dist = dist
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1

    def step(self, slot: int, lr: float) -> None:
        self.engine.backward(slot)
        if self.world > 1:
            self.dist.all_reduce(self.engine.grad, group=self.group)
        self.engine.update(lr, 1.0 / self.global_batch)


def wrap_device_buffer(ptr: int, count: int, device):
    """A float32 torch tensor aliasing `count` floats of device memory at `ptr` (no copy)."""
    import torch

    class _Alias:
        __cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (ptr, False), "version": 2}

    return torch.as_tensor(_Alias(), device=device)


class NetEngine:
    """Adapter giving a `Net` the `grad` tensor the data-parallel step reduces."""

    def __init__(self, net, device):
        self.net = net
        ptr, count = net.grad_buffer()
        self.grad = wrap_device_buffer(ptr, count, device)

    def backward(self, slot: int) -> None:
        self.net.backward(slot)

    def update(self, lr: float, grad_factor: float) -> None:
        self.net.update(lr, grad_factor)
