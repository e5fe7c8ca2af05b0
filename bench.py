#!/usr/bin/env python
"""Headline benchmark: training positions/sec of the NNUE step (fwd + bwd + AdamW+clip).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (--config 4, the default): the 768x16 -> 2048 pairwise multi-layer net (8 output buckets, 16 -> 32 -> 1)
at a GLOBAL batch of 131072 seeded synthetic positions per step, sharded evenly over the N ranks (strong
scaling).  For N > 1 the gradient exchange is the library's one kernel over peer memory, run under the
feature-transformer backward.  --config 0..3 give the same line for the four single-GPU configurations.

Prints ONE JSON line on rank 0.  `value` times the step with batches already resident in HBM; `e2e` times the
public call sequence from the raw 32-byte position records a data file holds (copy through pinned staging,
featurising / packing / grouping, step, loss read-back) with the next batch's upload overlapped with the current
step and each step's loss read while the next step runs.  `roofline` covers the dominant feature-transformer
kernel, `cpu_baseline` is the CPU oracle on this box's host cores, `exposed_exchange_ms` (N > 1) is the step
time minus the time of the same kernels with the exchange taken out.  `--impl reference` times the CPU oracle alone.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from bullet_b200 import config, synth  # noqa: E402
from bullet_b200.configs import AdamWParams  # noqa: E402

METRIC = "train positions/sec (fwd+bwd+AdamW)"
UNIT = "positions/s"
GLOBAL_BATCH = 131072  # --global-batch overrides it for profiling runs on a smaller case
CONFIG = 4             # --config: which of the five benchmark configurations (4 = the headline, the default)
WORKLOADS = {
    0: "c0: 768->128 screlu, concat->1 (examples/simple.rs shape), batch {}",
    1: "c1: 768x16(+768 factoriser)->1024 screlu, concat->8 buckets x 1, batch {}",
    2: "c2: ataxx 147->256 crelu, concat->1, nnz 49, batch {}",
    3: "c3: 768x16(+768 factoriser)->2048 crelu pairwise->8 buckets x (16->32->1), batch {}",
    4: "c4: 768x16(+768 factoriser)->2048 crelu pairwise->8 buckets x (16->32->1), global batch {}",
}


def workload():
    return WORKLOADS[CONFIG].format(GLOBAL_BATCH)

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the two tiled feature-transformer kernels of the
# 2048-wide pairwise network, as a two-term model through two ncu captures (16384 and 65536 positions per GPU:
# forward 495.9 and 1817.5 MB, backward 884.6 and 2987.8 MB): what does not grow with the batch (the table, or
# the gradient's write-back) plus a term per position (the activations written or read, 24.6 KB, and for the backward
# the table-gradient lines that L2 writes back and reads again between a row's reductions).
FT_DRAM_MODEL = {  # kernel: (bytes per launch that do not grow with the batch, bytes per position)
    "ft_forward": (55_400_000, 26_888),
    "ft_backward": (183_500_000, 42_790),
}
CPU_REPEATS = 10  # timed repeats of the CPU oracle at most, in the reference arm and in the in-line baseline alike
N_DISTINCT = 3  # distinct host batches cycled through (each far larger than L2 once expanded on device)


def env_int(name, default):
    return int(os.environ.get(name, default))


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_host_batches(cfg, n_local, rank, count):
    """`count` distinct batches of this rank: the raw 32-byte records and the arrays the host mapper makes of them."""
    from bullet_b200.net import featurise

    records, arrays = [], []
    for i in range(count):
        rec = synth.records(cfg.game, n_local, seed=cfg.seed + 1000 * rank + i)
        records.append(rec)
        arrays.append(featurise(cfg.game, rec, cfg.desc))
    return records, arrays


def cpu_reference(cfg, sample, repeats, warmup):
    """The CPU oracle's step on this box's host cores, on a bounded sample of the workload.

    A workload step is fwd+bwd over GLOBAL_BATCH positions plus one AdamW over every parameter.  The
    oracle's fwd+bwd has a part that does not grow with the batch (merging the factoriser into the
    table, clearing and adding the two table-sized gradient buffers) and a part per position; timing
    `sample` and `sample / 2` positions separates the two (t = fixed + per_position * n), so the fixed
    part is counted once per workload step and not once per sample.  AdamW is timed in full.
    Uses every host core whatever OMP_NUM_THREADS the launcher set.  Medians over `repeats`."""
    from oracle import Oracle

    orc = Oracle("f32")
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    orc.lib.omp_set_num_threads(cores)
    sizes = (sample // 2, sample)
    desc = dataclasses.replace(cfg.desc, max_batch=sample)
    rec = synth.records(cfg.game, sample, seed=cfg.seed + 99)
    full = orc.map_batch(cfg.game, rec, desc)
    batches = [tuple(a[:n] for a in full) for n in sizes]
    w = orc.to_real(synth.init_weights(desc, seed=cfg.seed))
    m, v = orc.zeros_like(desc), orc.zeros_like(desc)
    t_fb, t_opt, t_pass = [[], []], [], []
    for i in range(warmup + repeats):
        t_begin = time.perf_counter()
        for k, batch in enumerate(batches):
            t0 = time.perf_counter()
            _, g, _ = orc.net_grad(desc, w, *batch)
            if i >= warmup:
                t_fb[k].append(time.perf_counter() - t0)
        t1 = time.perf_counter()
        orc.net_update(desc, w, m, v, g, 1.0 / GLOBAL_BATCH, cfg.lr, AdamWParams())
        t2 = time.perf_counter()
        if i >= warmup:
            t_opt.append(t2 - t1)
            t_pass.append(t2 - t_begin)
    half, whole, opt = statistics.median(t_fb[0]), statistics.median(t_fb[1]), statistics.median(t_opt)
    per_position = max((whole - half) / (sizes[1] - sizes[0]), 0.0)
    fixed = max(whole - per_position * sizes[1], 0.0)
    step_s = fixed + per_position * GLOBAL_BATCH + opt
    return {
        "value": GLOBAL_BATCH / step_s, "unit": UNIT, "cores": orc.threads(), "kind": "port",
        "sample": (f"CPU oracle (C port of the reference interpreter's arithmetic, OpenMP on {orc.threads()} threads): "
                   f"fwd+bwd timed on {sizes[0]} and on {sizes[1]} of the step's {GLOBAL_BATCH} positions, split into a "
                   f"fixed part ({fixed * 1e3:.1f} ms, counted once per step) and {per_position * 1e6:.2f} us per position; "
                   f"AdamW over all {cfg.desc.n_params()} parameters timed in full ({opt * 1e3:.1f} ms); medians of "
                   f"{repeats} repeats after {warmup} warm-up"),
        "modelled_step_ms": step_s * 1e3, "measured_pass_ms": statistics.median(t_pass) * 1e3,
    }


def run_reference(args, rank, world):
    if rank != 0:
        return
    cfg = config(CONFIG)
    cpu = cpu_reference(cfg, args.cpu_sample, min(max(1, args.steps), CPU_REPEATS), min(max(1, args.warmup), 2))
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        # what one timed repeat really took (two sample passes and one AdamW); the workload step it models
        # (all positions) is cpu_baseline.modelled_step_ms
        "ms_per_step": cpu["measured_pass_ms"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload(), "global_batch": GLOBAL_BATCH, "where": "host CPU cores, no GPU"},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def ft_algorithmic_bytes(desc, batch):
    """Algorithmic bytes of one launch of the FT forward / backward kernel on this batch.

    forward : table rows gathered (one H-float row per active feature of each perspective)
              + the u16 index slots + the activations written (x, and the pairwise crelu outputs
              kept for the backward);
    backward: table-gradient rows updated (one per active feature, read-modify-write counted once)
              + the incoming gradient of both perspectives (2H floats) + the u16 index slots.
    """
    stm, nstm = batch[0], batch[1]
    n = len(batch[3])
    H = desc.ft_out
    rows = int((stm >= 0).sum() + (nstm >= 0).sum())
    idx = 2 * n * desc.nnz * 2
    out_elems = n * desc.dense_in0 + (n * 2 * H if desc.pairwise else 0)
    fwd = rows * H * 4 + idx + out_elems * 4
    bwd = rows * H * 4 + n * 2 * H * 4 + idx
    return fwd, bwd, rows


def run_ours(args, rank, world, local_rank):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: bullet_b200 has no CPU fallback "
                         "(use --impl reference for the CPU oracle)")
    import torch.distributed as dist

    from bullet_b200.dp import DataParallelStep, NetEngine
    from bullet_b200.net import Net

    torch.cuda.set_device(local_rank)
    if world > 1:
        opts = dist.ProcessGroupNCCL.Options()
        opts.is_high_priority_stream = True  # collectives that run beside kernels get their SMs first
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), pg_options=opts)
    cfg = config(CONFIG)
    if GLOBAL_BATCH % world:
        raise SystemExit("the global batch must divide evenly over the ranks")
    n_local = GLOBAL_BATCH // world
    desc = dataclasses.replace(cfg.desc, max_batch=n_local)
    cfg = dataclasses.replace(cfg, desc=desc)
    records, batches = make_host_batches(cfg, n_local, rank, N_DISTINCT)

    stream = torch.cuda.Stream()
    net = Net(desc, device=local_rank, stream=stream.cuda_stream)
    if args.ft_mode:
        net.set_option("ft_mode", args.ft_mode)
    if args.ft_fwd_mode:
        net.set_option("ft_fwd_mode", args.ft_fwd_mode)
    if args.ft_bwd_mode:
        net.set_option("ft_bwd_mode", args.ft_bwd_mode)
    if args.opt:
        for kv in args.opt:
            k, v = kv.split("=")
            net.set_option(k, int(v))
    if args.ft_bwd_wide is not None:
        net.set_option("ft_bwd_wide", args.ft_bwd_wide)
    net.load_weights(synth.init_weights(desc, seed=cfg.seed))
    parts = args.dp_parts if (world > 1 and net.stat("ft_tiled") & 2) else 1
    shard = bool(args.dp_shard) and world > 1
    peer = bool(args.dp_peer) and world > 1
    dp = DataParallelStep(NetEngine(net, torch.device("cuda", local_rank)), GLOBAL_BATCH, parts=parts, shard_optimiser=shard,
                          peer_exchange=peer, peer_overlap=peer and parts == 1 and bool(args.dp_overlap))
    peer, shard, parts = dp.peer, dp.shard, dp.parts  # what is really in use (peer mapping can be refused by the box)
    lr = cfg.lr

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def one_step(slot):
        dp.step(slot, lr)  # backward, all-reduce of the flat gradient buffer when N > 1 (pipelined), AdamW

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with torch.cuda.stream(stream):
        # ---------------------------------------------- device-resident inputs ("value")
        for s in range(N_DISTINCT):
            net.upload(s, *batches[s])
        net.sync()
        for i in range(args.warmup):
            one_step(i % N_DISTINCT)
        barrier()
        try:
            net.timings()  # drop the warm-up steps from the per-kernel averages
        except Exception:
            pass
        launches0 = net.stat("launches")
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for i in range(args.steps):
            one_step(i % N_DISTINCT)
        dp.finish()  # weight gathers still in flight belong to the timed steps
        ev1.record(stream)
        barrier()
        dev_ms = max_over_ranks(ev0.elapsed_time(ev1))
        launches = net.stat("launches") - launches0
        phase = net.timings()
        loss_resident = net.loss() if world == 1 else None

        # ------------------------------------------------ end to end through the public API
        # from the raw position records a data file holds: featurising, packing and grouping are inside the
        # timed region (on the device by default: 32 bytes per position cross PCIe)
        if args.e2e_source == "arrays":
            def upload(slot, k):
                net.upload(slot, *batches[k])
        else:
            def upload(slot, k):
                net.upload_records(slot, cfg.game, records[k], on_device=args.e2e_source == "records")
        upload(0, 0)
        for i in range(max(args.warmup, 1)):
            one_step(i % N_DISTINCT)
            upload((i + 1) % N_DISTINCT, (i + 1) % N_DISTINCT)
            net.loss()
        h2d0 = net.stat("h2d_bytes")
        first = max(args.warmup, 1) % N_DISTINCT
        barrier()
        t0 = time.perf_counter()
        last_loss = None
        for i in range(args.steps):
            slot = (first + i) % N_DISTINCT
            nxt = (slot + 1) % N_DISTINCT
            one_step(slot)                                              # enqueue only
            upload(nxt, nxt)                                             # H2D + preparation of the next batch
            if i:
                last_loss = net.loss(steps_back=1)                       # D2H read of the previous step's loss
        last_loss = net.loss()                                           # ... and of the last step's
        dp.finish()
        barrier()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        h2d_per_step = (net.stat("h2d_bytes") - h2d0) // max(args.steps, 1)
        # N > 1: the same kernels with the exchange taken out (every rank updates its own replica from its own
        # gradients, which is what one GPU does); step time minus this is the exposed part of the exchange
        local_ms = None
        if world > 1:
            net.sync()
            barrier()
            ev2, ev3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev2.record(stream)
            for i in range(args.steps):
                net.backward(i % N_DISTINCT)
                net.update(lr, 1.0 / GLOBAL_BATCH)
            ev3.record(stream)
            barrier()
            local_ms = max_over_ranks(ev2.elapsed_time(ev3)) / args.steps
        clocks = sampler.stop() if rank == 0 else None

    value = GLOBAL_BATCH * args.steps / (dev_ms * 1e-3)
    e2e_value = GLOBAL_BATCH * args.steps / e2e_s
    fwd_b, bwd_b, rows = ft_algorithmic_bytes(desc, batches[0])
    peak, peak_kind = measured_peak_gbs()
    kernels = {
        "ft_forward": {"ms": phase["ft_forward"], "algorithmic_bytes": fwd_b},
        "ft_backward": {"ms": phase["ft_backward"], "algorithmic_bytes": bwd_b},
    }
    for k in kernels.values():
        k["achieved_gbs"] = k["algorithmic_bytes"] / (k["ms"] * 1e-3) / 1e9 if k["ms"] > 0 else None
        k["frac_of_hbm_peak"] = k["achieved_gbs"] / peak if k["achieved_gbs"] else None
    dom = max(kernels, key=lambda n: kernels[n]["ms"])
    # the DRAM model was fitted on the 2048-wide pairwise network only
    traffic = FT_DRAM_MODEL[dom][0] + FT_DRAM_MODEL[dom][1] * n_local if dom in FT_DRAM_MODEL and CONFIG >= 3 else None
    # What bounds the tiled kernels: every active feature's 256-byte row piece passes the SM's
    # shared-memory data pipe (128 bytes per clock per SM) once per 64-column slab, while HBM sees the
    # table once per launch.  The HBM figure is kept beside it: it exceeds 1 because rows are served on chip.
    sm_mhz = ((clocks or {}).get("sm_mhz") or 1965.0) if rank == 0 else 1965.0
    sm_count = torch.cuda.get_device_properties(local_rank).multi_processor_count
    pipe_gbs = sm_count * 128 * sm_mhz * 1e6 / 1e9
    tiled = bool(net.stat("ft_tiled") & (1 if dom == "ft_forward" else 2))
    achieved = kernels[dom]["achieved_gbs"]
    hbm_view = {"achieved": achieved, "peak": peak, "unit": "GB/s", "frac": kernels[dom]["frac_of_hbm_peak"],
                "peak_kind": f"of {peak_kind} (STREAM-style copy)"}
    for k in kernels.values():
        k["frac_of_shared_memory_pipe"] = k["achieved_gbs"] / pipe_gbs if k["achieved_gbs"] else None
    if tiled:
        roofline = {"bound": "shared-memory pipe", "kernel": dom, "achieved": achieved, "peak": pipe_gbs, "unit": "GB/s",
                    "frac": achieved / pipe_gbs if achieved else None, "traffic": traffic,
                    "peak_kind": f"{sm_count} SMs x 128 B/clk x {sm_mhz:.0f} MHz (median SM clock during the run)",
                    "hbm": hbm_view}
    else:
        # the gather kernels read table rows (forward) or add to gradient rows (backward) straight in L2 when the
        # table and its gradient fit there, else in HBM; the L2 rates are measured now, on a 32 MB buffer
        table_bytes = desc.n_inputs * desc.ft_out * 4
        if 2 * table_bytes <= 96 << 20:
            from bullet_b200.net import probe_bandwidth

            kind = "read" if dom == "ft_forward" else "atomic"
            l2_gbs = probe_bandwidth(kind, 32 << 20, 40, local_rank)
            roofline = {"bound": "l2", "kernel": dom, "achieved": achieved, "peak": l2_gbs, "unit": "GB/s",
                        "frac": achieved / l2_gbs if achieved else None, "traffic": traffic,
                        "peak_kind": ("measured now: 16-byte loads of an L2-resident 32 MB buffer" if kind == "read" else
                                      "measured now: 16-byte vector reductions into an L2-resident 32 MB buffer"),
                        "hbm": hbm_view}
        else:
            roofline = dict(hbm_view, bound="hbm", kernel=dom, traffic=traffic)
    roofline.update({"algorithmic_bytes_per_launch": kernels[dom]["algorithmic_bytes"], "launch_ms": kernels[dom]["ms"],
                     "note": "algorithmic bytes count every gathered/updated table row once per active feature; "
                             "traffic is the DRAM side (a two-term model through ncu captures at 16384 and 65536 positions)"})
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_reference(cfg, args.cpu_sample, min(max(1, args.steps), CPU_REPEATS), 2)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload(), "global_batch": GLOBAL_BATCH, "per_gpu_batch": n_local,
                   "parallelism": f"dp{world}",
                   "exchange": ("one kernel over peer memory, run under the feature-transformer backward on SMs of its own: "
                                "finished row blocks are announced to all ranks; peer loads of all gradients, AdamW on 1/N, "
                                "peer stores of the weights" if peer and dp.overlap else
                                "one kernel over peer memory: peer loads of all gradients, AdamW on 1/N, peer stores of the weights"
                                if peer else
                                f"reduce-scatter + sharded AdamW + all-gather in {parts} slices, gathers under the next forward"
                                if shard and parts > 1 else "reduce-scatter + sharded AdamW + all-gather" if shard else
                                f"all-reduce in {parts + 1} pipelined parts" if parts > 1 else "one all-reduce"),
                   "ft_kernels": {"forward": "tiled" if net.stat("ft_tiled") & 1 else "gather",
                                  "backward": "tiled" if net.stat("ft_tiled") & 2 else "gather"},
                   "l2": f"inputs larger than L2: {N_DISTINCT} distinct batches cycled, per-step activations "
                         f"{n_local * (desc.dense_in0 * 2 + 2 * desc.ft_out) * 4 / 1e6:.0f} MB",
                   "active_features_per_position": rows / n_local},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d_per_step) * world,
                "d2h_bytes_per_step": (8 + (4 * (2 * (desc.n_inputs // desc.ft_block_rows + desc.n_out_buckets) + 1)
                                            if args.e2e_source == "records" else 0)) * world,
                "ms_per_step": e2e_s * 1e3 / args.steps,
                "source": {"records": "raw 32-byte records; featuriser, packing and grouping as kernels on the copy stream",
                           "records-host": "raw 32-byte records; featuriser and packing on the host cores",
                           "arrays": "index arrays made by the host mapper before the clock starts"}[args.e2e_source],
                "loss_per_position": None if last_loss is None else last_loss / GLOBAL_BATCH},
        "gpu_launches": int(launches),
        "compute_only_ms_per_step": local_ms,
        "exposed_exchange_ms": None if local_ms is None else dev_ms / args.steps - local_ms,
        "phases_ms": {k: round(v, 4) for k, v in phase.items() if k != "steps"},
        "kernels": kernels, "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks,
        "loss_per_position": None if loss_resident is None else loss_resident / GLOBAL_BATCH,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ft-mode", type=int, default=0, help="0 auto, 1 gather kernels, 2 tiled kernels")
    ap.add_argument("--ft-fwd-mode", type=int, default=0)
    ap.add_argument("--ft-bwd-mode", type=int, default=0)
    ap.add_argument("--opt", action="append", help="library option key=value (b200_net_set_option), repeatable")
    ap.add_argument("--ft-bwd-wide", type=int, default=None, help="tiled backward shape: 1 = 1024 threads, one CTA per SM")
    ap.add_argument("--dp-shard", type=int, default=1,
                    help="N > 1: 1 = reduce-scatter, AdamW on 1/N of the parameters per rank, all-gather; 0 = all-reduce")
    ap.add_argument("--dp-peer", type=int, default=1,
                    help="N > 1: 1 = the exchange as one library kernel over peer memory (reduce + AdamW + gather); "
                         "0, or a box that refuses the peer mapping = NCCL collectives (--dp-shard)")
    ap.add_argument("--dp-overlap", type=int, default=0,
                    help="N > 1 with --dp-peer 1: 1 = the exchange kernel runs under the backward pass (b200_step_exchange); "
                         "measured slower than the exchange behind the backward on 2 GPUs, hence off")
    ap.add_argument("--dp-parts", type=int, default=1,
                    help="N > 1: slices of l0w exchanged while the backward (and, with --dp-shard 1, the next forward) still runs")
    ap.add_argument("--e2e-source", default="records", choices=["records", "records-host", "arrays"],
                    help="what the end-to-end loop uploads every step: raw records prepared on the device (default), raw "
                         "records prepared on the host, or ready-made index arrays")
    ap.add_argument("--cpu-sample", type=int, default=16384,
                    help="positions of the larger of the two timed CPU-oracle passes (the other takes half)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--config", type=int, default=4, choices=[0, 1, 2, 3, 4],
                    help="benchmark configuration: 4 (default) is the headline; 0-3 give the roofline lines of the other networks")
    ap.add_argument("--global-batch", type=int, default=None,
                    help="positions per step over all ranks (default: the configuration's own, 131072 for the headline)")
    args = ap.parse_args()
    globals()["CONFIG"] = args.config
    globals()["GLOBAL_BATCH"] = args.global_batch or config(args.config).batch
    rank, world, local_rank = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
