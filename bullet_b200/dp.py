"""Data-parallel training step over the ranks of one box.

Positions are independent, so a global batch is cut into equal contiguous shards, one per
rank; every rank holds a full replica of the weights and the optimiser state.  The only
exchange is a sum all-reduce of the flat gradient buffer (whose first element carries the
summed loss) between the backward pass and the AdamW update; the update then runs on every
replica with grad_factor = 1 / global batch, which keeps the replicas bit-identical.

With `parts > 1` the exchange is pipelined against the backward pass: the feature-transformer
backward runs one run of table row blocks at a time, and the all-reduce of a finished slice of
the l0w gradient (by far the largest tensor) travels while the next slice and the dense
layers' weight gradients are still being computed; AdamW then runs slice by slice as the
reduced slices arrive.  Every rank issues the same collectives in the same order.

With `shard_optimiser` the all-reduce becomes a reduce-scatter, AdamW on this rank's 1/world of
the buffer and an all-gather of the weights: the same bytes on the wire, 1/world of the
optimiser traffic.  With `peer_exchange` those three steps are ONE kernel of the library over peer memory
(`b200_update_exchange`: peer loads of every rank's gradients, AdamW on this rank's share, peer
stores of the new weights to every rank), fenced by counters the ranks write into each other's memory.
With `peer_overlap` that kernel runs UNDER the feature-transformer backward (`b200_step_exchange`): the
backward announces finished table row blocks to all ranks and the exchange, on a few SMs of its own, takes
them as they arrive, so only the last block and the small tensors are left when the backward ends.
With `shard_optimiser` and `parts > 1` together the three are pipelined
slice by slice of l0w AND across steps: the reduce-scatter of a slice travels under the
backward of the next, and the all-gather of its updated weights is only waited for by the
forward pass of the NEXT step, slice by slice again, so that almost all of the exchange hides
behind kernels (`finish()` waits for what is still in flight).

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
    """Runs backward -> all-reduce -> update on an engine, in one piece or pipelined.

    The engine is anything with the calls of `bullet_b200.net.Net` used here and a `grad`
    attribute holding a torch tensor that aliases the flat gradient buffer.  For `parts == 1`
    it needs `backward(slot)` and `update(lr, grad_factor)`; for `parts > 1` also
    `backward_begin/backward_ft/backward_end`, `grad_part`, `update_range`, `update_end`.
    """

    def __init__(self, engine, global_batch: int, parts: int = 1, shard_optimiser: bool = False, process_group=None,
                 peer_exchange: bool = False, peer_overlap: bool = False):
        import torch.distributed as dist

        self.engine = engine
        self.global_batch = global_batch
        self.group = process_group
        self.dist = dist
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.parts = parts if self.world > 1 else 1
        self.shard = shard_optimiser and self.world > 1
        self.peer = peer_exchange and self.world > 1
        self.peer_error = None
        self.peer_pipelined = False
        self.overlap = False  # the peer exchange runs under the backward pass (b200_step_exchange)
        if peer_overlap and self.world > 1:
            self.peer, parts, self.parts = True, 1, 1
        if self.peer:  # map every rank's gradient and parameter buffers into this process
            try:
                mine = (engine.exchange_export(), engine.grad.numel())
            except Exception as e:  # noqa: BLE001 - any failure means: use the collectives instead, on every rank
                mine, self.peer_error = None, str(e)
            gathered = [None] * self.world
            dist.all_gather_object(gathered, mine, group=process_group)
            if any(g is None for g in gathered):
                self.peer_error = self.peer_error or "another rank could not export its buffers"
            elif any(n != engine.grad.numel() for _, n in gathered):
                raise ValueError("the ranks hold networks of different sizes")
            else:
                try:
                    engine.exchange_import(self.rank, self.world, b"".join(h for h, _ in gathered))
                except Exception as e:  # noqa: BLE001
                    self.peer_error = str(e)
            # all ranks take the same path: one failure sends everybody to the sharded collectives
            outcome = [None] * self.world
            dist.all_gather_object(outcome, self.peer_error, group=process_group)
            failed = [o for o in outcome if o]
            if failed:
                self.peer, self.peer_error = False, failed[0]
                self.shard = True
            else:
                self._token = engine.grad.new_zeros(1)
                self.shard = True  # momentum and velocity live sharded, as with shard_optimiser
                self.peer_pipelined = self.parts > 1
                self.overlap = bool(peer_overlap)
                if self.overlap:
                    engine.set_option("overlap_mode", 1)  # batches are cut for a backward that shares the GPU with the exchange
                if not self.peer_pipelined:
                    self.parts = 1
        self.pipelined = self.shard and self.parts > 1 and not self.peer
        self._gathers = None  # all-gathers of the previous step's weights, one per slice, still to be waited for
        if self.pipelined or self.peer_pipelined:
            self.l0w_first, n_l0w = engine.tensor_range("l0w")
            self.head_split = engine.tensor_range("l1b")[0]  # [0, split): loss, l0b, l0f; [split, l0w): the dense layers
            self.per_part = n_l0w // self.parts
            if n_l0w % self.parts or self.per_part % (4 * self.world):
                raise ValueError("l0w does not split evenly into parts x ranks x 4 floats")
        elif self.shard and engine.grad.numel() % self.world:
            raise ValueError("the flat buffer does not split evenly over the ranks")
        if self.peer_pipelined:
            import torch

            engine.set_option("manual_grad_zero", 1)  # peers read slices of the gradients while the next step runs
            self._side = torch.cuda.Stream(priority=-1)
            self._ev_bwd = [torch.cuda.Event() for _ in range(self.parts)]
            self._ev_done = [torch.cuda.Event() for _ in range(self.parts)]
            self._ev_head_ready, self._ev_head_free = torch.cuda.Event(), torch.cuda.Event()
            self._in_flight = False

    def _sharded_step(self, slot: int, lr: float) -> None:
        """reduce-scatter the gradients, AdamW on this rank's 1/world of the flat buffer only,
        all-gather the weights.  Same bytes on the wire as one all-reduce, 1/world of the
        optimiser traffic per GPU.  Momentum and velocity then live sharded: each rank holds the
        true values for its own range only (`gather_state` collects them, e.g. for a checkpoint).
        The summed loss rides in float 0: reduced onto rank 0, copied into the weight buffer's
        unused first float, gathered with the weights, and copied back on every rank."""
        eng, dist = self.engine, self.dist
        per = eng.grad.numel() // self.world
        mine = slice(self.rank * per, (self.rank + 1) * per)
        eng.backward(slot)
        if dist.get_backend(self.group) == "nccl":
            dist.reduce_scatter_tensor(eng.grad[mine], eng.grad, group=self.group)
        else:  # gloo has no reduce-scatter: reduce everything, use this rank's part
            dist.all_reduce(eng.grad, group=self.group)
        if self.rank == 0:
            eng.param[0:1].copy_(eng.grad[0:1])
        eng.update_range(lr, 1.0 / self.global_batch, self.rank * per, per)
        dist.all_gather_into_tensor(eng.param, eng.param[mine], group=self.group)
        eng.grad[0:1].copy_(eng.param[0:1])
        eng.update_end()

    def _peer_step(self, slot: int, lr: float) -> None:
        """The exchange as one kernel over peer memory: gradients summed with peer loads, AdamW on
        this rank's share, new weights stored to every rank.  The library fences the kernel itself
        (counters exchanged with the peers), so no collective runs in the step at all."""
        eng = self.engine
        eng.backward(slot)
        eng.update_exchange(lr, 1.0 / self.global_batch)
        eng.update_end()

    def _overlap_step(self, slot: int, lr: float) -> bool:
        """The peer exchange hidden under the backward pass: the library announces every finished row block
        of the table gradient to all ranks and a kernel on a few SMs of its own reduces, updates and
        redistributes the blocks while the backward is still at work.  False if this network cannot run it
        (every rank holds the same network, so every rank gets the same answer)."""
        from ._lib import B200Error

        try:
            self.engine.step_exchange(slot, lr, 1.0 / self.global_batch)
        except B200Error as e:
            if e.code != -5:
                raise
            self.overlap = False
            return False
        return True

    def _peer_pipelined_step(self, slot: int, lr: float) -> None:
        """The peer exchange slice by slice of l0w, on a side stream, beside the kernels.

        Compute stream: forward (slice p waits until last step's exchange of slice p is done on
        every rank) -> dense layers, loss, dense gradients -> per slice: clear its gradients,
        backward, mark.  Side stream, per slice, behind its mark: barrier, the exchange kernel on
        this rank's share (peer loads, AdamW, peer stores), barrier.  The small tensors (loss, l0b,
        l0f, dense layers) are complete after the last slice; every rank then sums them over all
        ranks and updates them for itself (no stores to peers), ahead of the last slice's exchange
        on the side stream, because the next forward needs them first."""
        import torch

        eng, dist, P, gf = self.engine, self.dist, self.parts, 1.0 / self.global_batch
        cur, side = torch.cuda.current_stream(), self._side
        share = self.per_part // self.world

        def fenced(first, count, gather):  # on the side stream: barrier, kernel, barrier
            dist.all_reduce(self._token, group=self.group)
            eng.update_exchange_range(lr, gf, first, count, gather, side.cuda_stream)
            dist.all_reduce(self._token, group=self.group)

        eng.forward_begin(slot)
        for p in range(P):
            if self._in_flight:
                cur.wait_event(self._ev_done[p])
            eng.forward_ft(slot, p, P)
        if self._in_flight:
            cur.wait_event(self._ev_head_free)  # every rank has read the small tensors' gradients of the last step
        eng.grad_zero_range(0, self.l0w_first)
        eng.backward_begin(slot)
        for p in range(P):
            whole, mine = self._slice(p)
            eng.grad_zero_range(whole.start, self.per_part)
            eng.backward_ft(slot, p, P)
            if p == P - 1:
                eng.backward_end(slot)  # joins the dense weight gradient: the small tensors are complete
            self._ev_bwd[p].record(cur)
            with torch.cuda.stream(side):
                side.wait_event(self._ev_bwd[p])
                if p == P - 1:  # the small tensors first: complete now, and the next forward starts with them
                    dist.all_reduce(self._token, group=self.group)
                    eng.update_exchange_range(lr, gf, 0, self.l0w_first, False, side.cuda_stream)
                    self._ev_head_ready.record(side)
                fenced(mine.start, share, True)
                if p == P - 1:
                    self._ev_head_free.record(side)  # behind a barrier that follows every rank's read of them
                self._ev_done[p].record(side)
        cur.wait_event(self._ev_head_ready)
        eng.update_end()
        self._in_flight = True

    def _slice(self, part: int):
        """(whole slice, this rank's share of it) of l0w inside the flat buffers, as python slices."""
        first = self.l0w_first + part * self.per_part
        share = self.per_part // self.world
        return slice(first, first + self.per_part), slice(first + self.rank * share, first + (self.rank + 1) * share)

    def _pipelined_sharded_step(self, slot: int, lr: float) -> None:
        """Sharded optimiser, slice by slice of l0w and across steps.

        Order on every rank: forward (slice p waits for last step's gather of slice p) ->
        backward with one reduce-scatter per finished slice -> all-reduce of the small tensors
        (loss, l0b, l0f after the last slice; dense layers after their weight gradients) ->
        per slice: AdamW on this rank's share, all-gather of the slice (left in flight) ->
        AdamW on the small tensors, on every rank alike.  Momentum and velocity of l0w live
        sharded (rank r holds share r of every slice); those of the small tensors are complete
        everywhere."""
        eng, dist, P, gf = self.engine, self.dist, self.parts, 1.0 / self.global_batch
        nccl = dist.get_backend(self.group) == "nccl"
        eng.forward_begin(slot)
        for p in range(P):
            if self._gathers is not None:
                self._gathers[p].wait()  # the compute stream waits; the host does not
            eng.forward_ft(slot, p, P)
        self._gathers = None
        eng.backward_begin(slot)
        scatters = []
        for p in range(P):
            eng.backward_ft(slot, p, P)
            whole, mine = self._slice(p)
            if nccl:
                work = dist.reduce_scatter_tensor(eng.grad[mine], eng.grad[whole], group=self.group, async_op=True)
            else:  # gloo has no reduce-scatter: reduce the slice, use this rank's share
                work = dist.all_reduce(eng.grad[whole], group=self.group, async_op=True)
            scatters.append(work)
        head_a = dist.all_reduce(eng.grad[0:self.head_split], group=self.group, async_op=True)
        eng.backward_end(slot)
        head_b = dist.all_reduce(eng.grad[self.head_split:self.l0w_first], group=self.group, async_op=True)
        gathers = []
        for p in range(P):
            whole, mine = self._slice(p)
            scatters[p].wait()
            eng.update_range(lr, gf, mine.start, mine.stop - mine.start)
            gathers.append(dist.all_gather_into_tensor(eng.param[whole], eng.param[mine], group=self.group, async_op=True))
        head_a.wait()
        head_b.wait()
        eng.update_range(lr, gf, 0, self.l0w_first)
        eng.update_end()
        self._gathers = gathers

    def finish(self) -> None:
        """Waits (on the compute stream) for weight gathers still in flight; call before reading
        weights, saving, or leaving the training loop."""
        if self._gathers is not None:
            for work in self._gathers:
                work.wait()
            self._gathers = None
        if self.peer_pipelined and self._in_flight:
            import torch

            for ev in self._ev_done + [self._ev_head_free]:
                torch.cuda.current_stream().wait_event(ev)
            self._in_flight = False

    def gather_state(self) -> None:
        """After sharded steps: make momentum and velocity complete on every rank."""
        if not self.shard:
            return
        self.finish()
        if getattr(self, "used_overlap", False):
            # rank r holds share r of every row block of l0w and share r of l0f; the small tensors are complete
            first, count = self.engine.tensor_range("l0w")
            block = self.engine.overlap_block_floats()
            ranges = [(first + b * block, block) for b in range(count // block)]
            try:
                ranges.append((self.engine.tensor_range("l0f")[0], block))
            except Exception:  # noqa: BLE001 - no factoriser
                pass
            for buf in self.engine.state_buffers():
                for lo, n in ranges:
                    share = n // self.world
                    mine = buf[lo + self.rank * share: lo + (self.rank + 1) * share].clone()
                    self.dist.all_gather_into_tensor(buf[lo:lo + n], mine, group=self.group)
            return
        if self.pipelined or self.peer_pipelined:
            for buf in self.engine.state_buffers():
                for p in range(self.parts):
                    whole, mine = self._slice(p)
                    self.dist.all_gather_into_tensor(buf[whole], buf[mine].clone(), group=self.group)
            return
        per = self.engine.grad.numel() // self.world
        mine = slice(self.rank * per, (self.rank + 1) * per)
        for buf in self.engine.state_buffers():
            self.dist.all_gather_into_tensor(buf, buf[mine].clone(), group=self.group)

    def step(self, slot: int, lr: float) -> None:
        eng, gf = self.engine, 1.0 / self.global_batch
        if self.peer_pipelined:
            self._peer_pipelined_step(slot, lr)
            return
        if self.overlap and self._overlap_step(slot, lr):
            self.used_overlap = True
            return
        if self.peer:
            self._peer_step(slot, lr)
            return
        if self.pipelined:
            self._pipelined_sharded_step(slot, lr)
            return
        if self.shard:
            self._sharded_step(slot, lr)
            return
        if self.parts == 1:
            eng.backward(slot)
            if self.world > 1:
                self.dist.all_reduce(eng.grad, group=self.group)
            eng.update(lr, gf)
            return
        eng.backward_begin(slot)
        pending = []
        for part in range(self.parts):
            eng.backward_ft(slot, part, self.parts)
            first, count = eng.grad_part(part, self.parts)
            # the collective waits for the kernels enqueued so far and runs beside the next ones
            work = self.dist.all_reduce(eng.grad[first:first + count], group=self.group, async_op=True)
            pending.append((work, first, count))
        eng.backward_end(slot)
        first, count = eng.grad_part(self.parts, self.parts)
        pending.append((self.dist.all_reduce(eng.grad[first:first + count], group=self.group, async_op=True),
                        first, count))
        for work, first, count in pending:
            work.wait()  # orders the compute stream after the collective; the host does not block
            eng.update_range(lr, gf, first, count)
        eng.update_end()


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
        self.param, self._m, self._v = (wrap_device_buffer(*net.flat_buffer(kind), device) for kind in (0, 1, 2))
        self.state_buffers = lambda: [self._m, self._v]
        for name in ("backward", "update", "forward_begin", "forward_ft", "backward_begin", "backward_ft", "backward_end",
                     "grad_part", "update_range", "update_end", "tensor_range", "exchange_export", "exchange_import",
                     "update_exchange", "update_exchange_range", "grad_zero_range", "set_option", "step_exchange"):
            setattr(self, name, getattr(net, name))
        self.overlap_block_floats = lambda: net.desc.ft_block_rows * net.desc.ft_out
