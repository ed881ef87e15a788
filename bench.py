#!/usr/bin/env python
"""Benchmark of the infinitely-connected-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload cfg0|cfg2|cfg4]

One "step" is one forward pass of the Crystalformer model (4 layers, model_dim 128, 8 heads, 64 radial-basis bins for
cfg0/cfg4; 7 layers without the value encoding for cfg2) over one batch of seeded synthetic crystals.  Per GPU the batch
has the configuration's crystal count; with N GPUs a batch of N times that many crystals is drawn, split over the ranks
by the reference's greedy rule on n^2 (crystalformer_b200.sharding.lpt_assign) and only the per-crystal outputs are
gathered on every rank, by stores into the peers' memory (crystalformer_b200.sharding.PeerGather; weak scaling).
Rank 0 prints ONE JSON line:

  value            crystals / s over all ranks, inputs already resident in HBM.  K steps are issued back to back (no host
                   synchronisation in between); every step has its own CUDA-event pair and a 256 MB write flushes the L2
                   between the pairs.  The time of a round of K steps is the device wall clock from the first step's
                   start to the last step's end minus the K - 1 flushes in between (their duration is measured
                   separately), so device idle time caused by a slow host counts; the round is repeated until about one
                   second of device time has been timed and the rounds are averaged; max over ranks.
  e2e              the same through crystalformer_b200.serving.PipelinedPredictor with HOST inputs: pinned host -> device
                   copies of the step's inputs and the device -> host copy of the outputs are inside the timed region,
                   which is HOST wall clock from the first submit to the last result (no L2 flush in this loop)
  parity           (N = 1) the outputs of the timed model against the CPU reference's outputs for the same batch and
                   state_dict; the run fails above the tolerance
  roofline         the dominant kernel (the attention call of every layer), timed live with CUDA events on the launch
                   stream during the timed steps.  `executed`: the work the kernel really does, from its own counters
                   (chunks of eight list entries swept, 16-bin tiles evaluated), against the SFU and FP32 issue rates;
                   `algorithmic`: the reference's enumeration (125 translations per edge) divided by the same time
  lattice_sum_microbench   the 2,000,000 (i,j,head) lattice-sum kernel benchmark (phi + 64-bin psi, forward)
  workloads        (N = 1) the other configurations: cfg2 and cfg4 forward, cfg3 training step, a few timed steps each,
                   each beside the CPU reference on a sample of its crystals
  strong           (N > 1) the fixed 256-crystal cfg2 and 64-crystal cfg4 batches split over the N ranks
  cpu_baseline     (N = 1) the reference's kernels compiled for the CPU driving the same model on the host cores

--impl reference times the reference's CPU implementation of the path (its own kernel sources compiled for the CPU
when oracle/_ref exists, else the C restatement) on the host cores, on the same batch and seed-0 weights.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

WORKLOADS = {
    "cfg0": dict(config="cfg0", layers=4, K=64, crystals=128),
    "cfg2": dict(config="cfg2", layers=7, K=0, crystals=256),
    "cfg4": dict(config="cfg4", layers=4, K=64, crystals=64),
}
FIXED_BOX_TERMS = 125  # (2 R + 1)^3 with the default lattice_range R = 2
PARITY_TOL = 1e-4
SM_FP32_LANES, SM_SFU_LANES = 128, 16  # FP32 and MUFU lane-instructions per clock and SM


def fp32_instr_per_term(K, H=8):
    """FP32-pipe instructions per (edge, translation) term of the reference's enumeration, basis shared by the heads:
    geometry and minimum pass 25, two per bin, (2 + K) per head."""
    return 25 + 2 * K + H * (2 + K)


def sfu_per_term(K, H=8):
    return (1 if K > 0 else 0) + K + H


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons while the timed region runs."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.path = tempfile.NamedTemporaryFile(prefix="clocks_", suffix=".csv", delete=False).name
        self.proc = None
        self.gpu = gpu_index
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples taken between the two wall-clock times (all samples if none fall inside)."""
        import datetime
        if self.proc is None:
            return None
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = []
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                stamp = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((stamp, float(f[1]), float(f[2]), float(f[3]), f[5:9]))
            except ValueError:
                continue
        os.unlink(self.path)
        if not rows:
            return None
        inside = [r for r in rows if t_begin is not None and t_begin <= r[0] <= t_end]
        used = inside if inside else rows
        reasons = set()
        for r in used:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median([r[1] for r in used])), "sm_max_mhz": float(max(r[2] for r in used)),
                "power_w_max": float(max(r[3] for r in used)), "samples": len(used),
                "window": "timed region" if inside else "whole run (timed region shorter than the sampling period)",
                "reasons": sorted(reasons)}


def make_model(layers, K, seed=0):
    import torch
    from crystalformer_b200.model import Latticeformer, default_params
    torch.manual_seed(seed)
    params = default_params(num_layers=layers, value_pe_dist_real=K)
    return Latticeformer(params), params


def fix_gauss_scale(model, data):
    """One training-mode forward stores the batch statistics of alpha in gauss_scale (as the reference's first training
    step does, models/indexed_lattice_multi_head_attention_cuda.py:669-673); afterwards the model is shard-invariant."""
    import torch
    model.train()
    with torch.no_grad():
        model(data)
    model.eval()


def to_device_batch(cb, device, pinned=False):
    import torch
    import types
    host = dict(x=torch.from_numpy(cb.x), pos=torch.from_numpy(cb.pos), trans_vec=torch.from_numpy(cb.trans_vec),
                sizes=torch.from_numpy(cb.sizes))
    if pinned:
        return types.SimpleNamespace(**{k: v.pin_memory() for k, v in host.items()})
    return types.SimpleNamespace(**{k: v.to(device) for k, v in host.items()})


def metric_name(layers):
    return "crystals/sec (4-layer, fwd)" if layers == 4 else f"crystals/sec ({layers}-layer, fwd)"


class StepTimer:
    """Device timing of a loop of steps on one rank (see the module docstring): rounds of `steps` steps, each step in its
    own event pair, the L2 flush between the pairs."""

    def __init__(self, device, world, flush_bytes=256 * 1024 * 1024, share=None):
        import torch
        self.torch, self.device, self.world = torch, device, world
        if share is not None:  # another timer's flush buffer and its measured duration
            self.flush, self.flush_ms = share.flush, share.flush_ms
        else:
            self.flush = torch.empty(flush_bytes, dtype=torch.uint8, device=device)  # > 126 MB L2
            self.flush_ms = self._flush_time()

    def barrier(self):
        import torch.distributed as dist
        self.torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
        self.torch.cuda.synchronize()

    def _flush_time(self):
        torch = self.torch
        for _ in range(3):
            self.flush.zero_()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(10):
            self.flush.zero_()
        e.record()
        e.synchronize()
        return s.elapsed_time(e) / 10

    def max_over_ranks(self, value):
        import torch.distributed as dist
        t = self.torch.tensor([value], device=self.device, dtype=self.torch.float64)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def one_round(self, step, steps, drain=None, finish=None):
        """finish: called after the last step, before the round's end is recorded (work the steps left on other streams
        is made to count)."""
        torch = self.torch
        spans = []
        host_t0 = time.perf_counter()
        for _ in range(steps):
            self.flush.zero_()  # L2 flush between timed iterations
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            step()
            e.record()
            spans.append((s, e))
        host_issue = time.perf_counter() - host_t0  # the host is done issuing; the device may still be busy
        if finish:
            finish()
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        if drain:
            drain()
        self.barrier()
        span = sum(s.elapsed_time(e) for s, e in spans)
        wall = spans[0][0].elapsed_time(end) - (steps - 1) * self.flush_ms
        return {"span_ms": span, "wall_ms": max(wall, span), "host_issue_ms": host_issue * 1e3}

    def run(self, step, steps, warmup, drain=None, target_ms=1000.0, max_rounds=200, finish=None):
        """Returns (ms per step, max over ranks; this rank's diagnostics)."""
        for _ in range(warmup):
            step()
        if drain:
            drain()
        self.barrier()
        first = self.one_round(step, steps, drain, finish)
        first_max = self.max_over_ranks(first["wall_ms"])
        rounds = int(min(max_rounds, max(1, math.ceil(target_ms / max(first_max, 1e-3)))))
        done, total_max = [first], first_max
        for _ in range(rounds - 1):
            r = self.one_round(step, steps, drain, finish)
            done.append(r)
            total_max += self.max_over_ranks(r["wall_ms"])
        n = len(done) * steps
        diag = {"rounds": len(done), "timed_steps": n,
                "span_ms_per_step": sum(r["span_ms"] for r in done) / n,
                "device_wall_ms_per_step": sum(r["wall_ms"] for r in done) / n,
                "host_issue_ms_per_step": sum(r["host_issue_ms"] for r in done) / n,
                "l2_flush_ms": self.flush_ms}
        diag["host_bound"] = diag["host_issue_ms_per_step"] > diag["span_ms_per_step"]
        return total_max / n, diag


def count_kernel_launches(fn):
    """Kernels launched by one call of fn, counted from the CUDA activity records of torch.profiler (None if the
    profiler is not available)."""
    import torch
    try:
        from torch.profiler import ProfilerActivity, profile
        fn()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            fn()
            torch.cuda.synchronize()
        names = [ev.name for ev in prof.events() if ev.device_type == torch.autograd.DeviceType.CUDA
                 and "memcpy" not in ev.name.lower() and "memset" not in ev.name.lower()]
        import re
        short = lambda n: (re.findall(r"(\w+)\s*(?:<[^()]*>)?\s*\(", n) or [n])[-1] if "(" in n else n.split("<")[0].split("::")[-1]
        return len(names), sorted(set(short(n) for n in names))
    except Exception:  # noqa: BLE001 - any profiler failure only loses the diagnostic
        return None, None


def run_b200(args):
    import torch
    import torch.distributed as dist
    from crystalformer_b200 import ops
    from crystalformer_b200.sharding import PeerGather, crystal_cost, gather_outputs, lpt_assign, shard_balance
    from crystalformer_b200.synthetic import make_config

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False

    wl = WORKLOADS[args.workload]
    # weak scaling = the work per GPU does not change with N: the global batch of N ranks is N copies of the workload's
    # batch (an independent draw of N x 128 crystals would give every rank a different amount of work than the N = 1
    # run has: the 128 crystals of cfg0 are 17 % lighter in lattice-sum terms than the mean of the distribution), which
    # the greedy split below deals out one copy per rank.  Sharding of heterogeneous fixed batches is what `strong`
    # measures.
    import numpy as np
    one = make_config(wl["config"], num_crystals=wl["crystals"])
    global_batch = one if world == 1 else one.select(np.tile(np.arange(one.num_crystals), world))
    # the reference's greedy split, with the row scheduler's cost (n^2 x the terms per edge, which depend on the cell
    # volume) in place of n^2 as the weight: shards of equal n^2 differ by several percent in lattice-sum terms
    cost = crystal_cost(global_batch.sizes, global_batch.trans_vec)
    shards = lpt_assign(global_batch.sizes, world, weights=cost)
    mine = global_batch.select(shards[rank])
    n_atoms, n_edges, max_atoms = mine.num_atoms, mine.num_edges, int(mine.sizes.max())

    model, params = make_model(wl["layers"], wl["K"])
    model = model.to(device)
    # gauss_scale from the statistics of rank 0's shard, shared by every rank (broadcast once, outside the timed region)
    resident = to_device_batch(mine, device)
    fix_gauss_scale(model, resident)
    if world > 1:
        for layer in model.encoder.layers:
            dist.broadcast(layer.self_attn.gauss_scale.data, src=0)

    native_log = []  # the library records an event pair around every layer's attention call
    timer = StepTimer(device, world)

    # N > 1: the pooling + head kernel of every rank stores its outputs into every rank's gather buffer over NVLink
    # and a small kernel waits for all ranks (sharding.PeerGather); no collective library on the data path.
    # (overlap: a step's collect, where a rank waits for the others, runs on its own stream beside the next steps)
    peers = PeerGather(shards, model.mlp[-1].out_features, device, slots=20, overlap=True) if world > 1 else None
    extra = {} if peers is None else {"gather": peers}

    ready = torch.cuda.Event()
    ready.record()  # the resident inputs have been valid since here: a step's preparation need not wait for the step before it

    def step_resident():
        with torch.no_grad():
            return model(resident, counts=(n_atoms, n_edges, max_atoms), inputs_ready=ready, **extra)

    pinned = to_device_batch(mine, device, pinned=True)
    h2d_bytes = sum(t.numel() * t.element_size() for t in vars(pinned).values())
    d2h_bytes = (global_batch.num_crystals if world > 1 else mine.num_crystals) * 4

    from crystalformer_b200.serving import PipelinedPredictor
    # ten batches in flight alternating between six compute streams (the kernels of independent batches fill each
    # other's idle issue slots: measured 0.255 / 0.216 / 0.210 / 0.209 ms per batch with 2 / 4 / 6 / 8 streams); every
    # submit is one call of the library (cf_serve_submit)
    e2e_depth, e2e_streams = 10, 6
    runner = PipelinedPredictor(model, depth=e2e_depth, device=device, gather=peers, streams=e2e_streams)
    pending = []

    def step_e2e():
        """One batch through the public serving API: pinned host inputs -> device -> forward -> outputs in pinned host
        memory.  Several batches are in flight; the host blocks only when it collects the oldest result."""
        pending.append(runner.submit(pinned))
        if len(pending) == runner.depth:
            runner.result(pending.pop(0))

    def drain():
        while pending:
            runner.result(pending.pop(0))

    # ---- value: device-resident inputs
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        time.sleep(0.3)  # let nvidia-smi start sampling
    t_begin = time.time()
    finish = None if peers is None else peers.wait_ready  # the last step's collect belongs to the round
    ms_step, diag_resident = timer.run(step_resident, args.steps, args.warmup, finish=finish)
    t_end = time.time()
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    if peers is not None:
        peers.check()  # raises if a collect gave up waiting for a rank
    # the attention calls are timed in a round of their own, with the same flushes: the event pairs the library records
    # around them sit between the kernels of a step and cost the step a few tens of microseconds
    model.encoder.attention_event_log = native_log
    timer.one_round(step_resident, args.steps, finish=finish)
    model.encoder.attention_event_log = None
    op_ms = sum(s.elapsed_time(e) for s, e in native_log)
    op_calls = len(native_log)

    # ---- e2e: host wall clock around the serving pipeline, no flush: one uninterrupted stream of batches, a multiple of
    #      `steps` long enough for about a second (a first round of `steps` batches sets the length), from the first
    #      submit to the last result
    for _ in range(args.warmup):
        step_e2e()
    drain()
    timer.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_e2e()
    drain()
    torch.cuda.synchronize()
    first_round = timer.max_over_ranks(time.perf_counter() - t0)  # (the same on every rank: all run the same length)
    e2e_steps = args.steps * int(max(1, min(200, math.ceil(1.0 / max(first_round, 1e-6)))))
    timer.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_e2e()
    t1 = time.perf_counter()
    drain()
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    e2e_wall = timer.max_over_ranks(t2 - t0)
    e2e_issue = t1 - t0
    ms_e2e = e2e_wall * 1e3 / e2e_steps
    if peers is not None:
        peers.check()
    # one more batch through the serving pipeline, compared with the forward of the device-resident copy: the timed
    # loop delivered the outputs of the model, not of a shortened path
    y_served = runner.result(runner.submit(pinned)).clone()
    with torch.no_grad():
        y_direct = model(resident, counts=(n_atoms, n_edges, max_atoms), **({} if peers is None else {"gather": peers}))
    if peers is not None:
        peers.wait_ready()
    e2e_equal = bool(torch.equal(y_served, y_direct.cpu()))
    # ---- the same stream with the species as indices (z: the position of the 1 in every one-hot row of x), the
    #      predictor's compact input: 8 bytes per atom go to the device instead of 4 x 98; a shorter run, reported beside
    #      the figure above, which uses the reference's input format
    import types as _types
    pinned_z = _types.SimpleNamespace(z=pinned.x.argmax(1).contiguous().pin_memory(), pos=pinned.pos,
                                      trans_vec=pinned.trans_vec, sizes=pinned.sizes)
    z_equal = bool(torch.equal(runner.result(runner.submit(pinned_z)), y_served))
    z_steps = max(args.steps, e2e_steps // 4)
    timer.barrier()
    t0 = time.perf_counter()
    for _ in range(z_steps):
        pending.append(runner.submit(pinned_z))
        if len(pending) == runner.depth:
            runner.result(pending.pop(0))
    drain()
    torch.cuda.synchronize()
    z_wall = timer.max_over_ranks(time.perf_counter() - t0)
    if peers is not None:
        peers.check()
    e2e_z = {"value": global_batch.num_crystals * z_steps / z_wall, "unit": "crystals/s", "ms_per_step": z_wall * 1e3 / z_steps,
             "h2d_bytes_per_step": h2d_bytes - pinned.x.numel() * 4 + pinned_z.z.numel() * 8, "timed_steps": z_steps,
             "outputs_equal_one_hot_input": z_equal,
             "input": "species indices z (N) int64 instead of the one-hot rows x (N,98); otherwise as e2e"}

    total_crystals = global_batch.num_crystals
    value = total_crystals / (ms_step * 1e-3)
    e2e_value = total_crystals / (ms_e2e * 1e-3)

    # ---- N > 1: the peer-gathered outputs against the library all-gather of the same step
    gather_check = None
    if world > 1:
        with torch.no_grad():
            y_local = model(resident, counts=(n_atoms, n_edges, max_atoms))
            y_peer = model(resident, counts=(n_atoms, n_edges, max_atoms), gather=peers)
        peers.wait_ready()
        y_nccl = gather_outputs(y_local, shards)
        peers.check()
        gather_check = "ok" if torch.equal(y_peer, y_nccl) else "MISMATCH"

    strong = None
    if world > 1 and not args.no_strong:
        strong = {name: strong_scaling_case(name, rank, world, device, timer) for name in ("cfg2", "cfg4")}

    every = [diag_resident]
    if world > 1:
        every = [None] * world
        dist.all_gather_object(every, diag_resident)

    result = None
    if rank == 0:
        K = wl["K"]
        sm_mhz = clocks["sm_max_mhz"] if clocks else 1965.0
        roofline = attention_roofline(ops, device, model, step_resident, wl, n_atoms, n_edges, max_atoms, op_ms, op_calls,
                                      ms_step, sm_mhz * 1e6)
        micro = lattice_microbench(ops, device, roofline["peaks"])
        cpu = parity = None
        if world == 1 and not args.no_cpu_baseline:
            with torch.no_grad():
                y_gpu = model(resident, counts=(n_atoms, n_edges, max_atoms)).cpu().numpy()
            cpu, y_cpu = cpu_baseline(model, params, mine)
            parity = {"max_rel": float(np.abs(y_gpu - y_cpu).max() / np.abs(y_cpu).max()), "tol": PARITY_TOL,
                      "crystals": int(mine.num_crystals), "against": cpu["kind"] + " CPU forward, same batch and state_dict"}
            parity["ok"] = parity["max_rel"] <= PARITY_TOL
        workloads = None
        if world == 1 and not args.no_workloads and args.workload == "cfg0":
            workloads = {"cfg2": extra_workload("cfg2", device, timer, not args.no_cpu_baseline),
                         "cfg4": extra_workload("cfg4", device, timer, not args.no_cpu_baseline),
                         "cfg3_train": train_step_case(ops, device, 256)}
        # the kernels of one forward, counted from the profiler's CUDA activity records: last of all, because the
        # profiler's instrumentation stays attached to the process and slows later launches on the host side
        launches, kernel_names = count_kernel_launches(step_resident)
        result = {
            "metric": metric_name(wl["layers"]),
            "value": value, "unit": "crystals/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {wl['layers']}-layer Crystalformer forward, K={K}, "
                                   f"{wl['crystals']} crystals per GPU per step", "global_batch": total_crystals,
                       "atoms_this_rank": n_atoms, "edges_this_rank": n_edges, "cutoff": "adaptive -3.5 sigma, minimum box R=2",
                       "l2": "flushed between timed steps (256 MB write between the per-step event pairs)",
                       "timing": "rounds of `steps` steps issued back to back; device wall clock of a round minus the "
                                 "flushes inside it; rounds repeated until about 1 s of device time, averaged; max over ranks",
                       "parallelism": f"dp{world} (greedy LPT split on the row-cost weight, outputs gathered by peer stores)",
                       "global_batch_is": "the workload's batch" if world == 1 else
                                          f"{world} copies of the workload's batch (work per GPU = the one-GPU run's)",
                       "shard_balance": shard_balance(global_batch.sizes, shards, cost)},
            "per_rank": {"resident": every},
            "e2e": {"value": e2e_value, "unit": "crystals/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes, "timed_steps": e2e_steps,
                    "host_issue_ms_per_step": e2e_issue * 1e3 / e2e_steps,
                    "clock": "host wall clock (perf_counter) from the first submit to the last result of one uninterrupted "
                             "stream of timed_steps batches (pipeline fill and drain inside the clock), max over ranks",
                    "outputs_equal_direct_forward": e2e_equal,
                    "api": f"crystalformer_b200.serving.PipelinedPredictor, {e2e_depth} batches in flight on {e2e_streams} compute stream(s)"},
            "e2e_species_indices": e2e_z,
            "gpu_launches": None if launches is None else launches * args.steps,
            "gpu_launches_per_step": launches, "kernels_per_step": kernel_names,
            "parity": parity, "roofline": roofline, "lattice_sum_microbench": micro, "cpu_baseline": cpu,
            "workloads": workloads, "strong": strong, "gather_check": gather_check, "clocks": clocks,
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result


def measure_pipe_peaks(ops, device):
    """FFMA and MUFU.EX2 issue rates of this GPU (lane-instructions / s), measured with cf_pipe_probe."""
    import torch
    sink = torch.zeros(4, device=device)
    peaks = {}
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    for kind, name in ((0, "fp32"), (1, "sfu")):
        blocks, threads, iters = sms * 8, 256, 1 << 13
        best = 1e30
        for _ in range(5):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(); ops.pipe_probe(kind, blocks, threads, iters, sink); e.record(); e.synchronize()
            best = min(best, s.elapsed_time(e))
        peaks[name] = blocks * threads * iters * 8 / (best * 1e-3)
    return peaks, sms


def attention_roofline(ops, device, model, step, wl, n_atoms, n_edges, max_atoms, op_ms, op_calls, ms_step, clock_hz):
    """Roofline object of one attention call (all kernels between the library's event pair of a layer).  clock_hz: the
    GPU's maximum SM clock (the nominal pipe rates are lanes x SMs x this clock)."""
    import torch
    K, layers = wl["K"], wl["layers"]
    peaks, sms = measure_pipe_peaks(ops, device)
    nominal = {"fp32": sms * SM_FP32_LANES * clock_hz, "sfu": sms * SM_SFU_LANES * clock_hz}
    t_call = op_ms * 1e-3 / max(op_calls, 1)
    terms = n_edges * FIXED_BOX_TERMS  # lower bound: the adaptive rule never shrinks the minimum box
    algorithmic = {"terms_per_call": terms, "fp32_lane_instr": terms * fp32_instr_per_term(K),
                   "sfu_lane_ops": terms * sfu_per_term(K),
                   "fp32_rate_over_peak": terms * fp32_instr_per_term(K) / t_call / nominal["fp32"],
                   "sfu_rate_over_peak": terms * sfu_per_term(K) / t_call / nominal["sfu"],
                   "note": "work of the reference's enumeration of every (edge, translation) term divided by this "
                           "kernel's time: a speed-up over that algorithm, not a utilisation (the kernel reads "
                           "precomputed lists and skips terms below the weight floor)"}
    sorted_path = K == 64 and max_atoms <= 32
    executed = None
    traffic = None
    if sorted_path:
        # counters of the sorted row kernel over one extra, untimed forward
        words = torch.zeros(4, dtype=torch.int64, device=device)
        ops.set_row_stats(words)
        try:
            step()
            torch.cuda.synchronize()
        finally:
            ops.set_row_stats(None)
        chunks, tiles, rows = (int(v) / layers for v in words[:3].tolist())
        # per lane and chunk: 2 ex2 (weights) + 2 rsqrt; per (chunk, tile): 4 ex2 (basis values).  FP32-pipe: about 18
        # per chunk (exponents, basis coordinates, operand splits) and 20 per (chunk, tile).
        sfu_ops = 32 * (4 * chunks + 4 * tiles)
        fp32_ops = 32 * (18 * chunks + 20 * tiles)
        t_sfu, t_fp32 = sfu_ops / nominal["sfu"], fp32_ops / nominal["fp32"]
        executed = {"chunks_per_call": chunks, "bin_tiles_per_call": tiles, "rows_per_call": rows,
                    "entries_per_call": 8 * chunks, "sfu_lane_ops": sfu_ops, "fp32_lane_instr": fp32_ops,
                    "mma_m16n8k8_per_call": 4 * chunks + 3 * tiles,
                    "sfu_frac": t_sfu / t_call, "fp32_frac": t_fp32 / t_call,
                    "sfu_frac_of_probe": sfu_ops / peaks["sfu"] / t_call}
        # bytes the call has to move at least: the list entries it sweeps, the row directory and per-edge minima, and
        # q, k, v, a in / out, lse out once per atom
        traffic = 64 * chunks + 32 * n_atoms + 4 * n_edges + n_atoms * 4 * (3 * 128 + 8 + 128 + 8)
    frac = executed["sfu_frac"] if executed else None
    return {
        "kernel": ("infinite_attn_sorted_rows_kernel (+ the launch for left-over rows): one attention call"
                   if sorted_path else "phi_from_list_kernel + infinite_attn_rows_kernel: one attention call"),
        "bound": "sfu", "unit": "G MUFU lane-ops/s",
        "achieved": None if executed is None else executed["sfu_lane_ops"] / t_call / 1e9,
        "peak": nominal["sfu"] / 1e9, "frac": frac,
        "peak_source": f"{sms} SMs x {SM_SFU_LANES} MUFU lanes x {clock_hz / 1e9:.3f} GHz (nominal); cf_pipe_probe measured "
                       f"{peaks['sfu'] / 1e9:.0f} G MUFU/s and {peaks['fp32'] / 1e9:.0f} G FFMA/s in this run "
                       "(MEASURED_PEAKS.json holds HBM and bf16 figures only)",
        "executed": executed, "algorithmic": algorithmic, "launches": op_calls, "avg_launch_us": t_call * 1e6,
        "share_of_step": t_call * 1e3 * layers / ms_step,
        "traffic": traffic, "traffic_unit": "bytes per call, from the run's own sizes and counters (see profiles/ for the "
                                            "ncu dram__bytes figure of the same kernel)",
        "hbm_frac_if_streamed": None if traffic is None else traffic / t_call / 6558.7e9,
        "peaks": peaks,
    }


def extra_workload(name, device, timer, with_cpu):
    """A few timed steps of another configuration (single GPU), beside the CPU reference on a sample of its crystals."""
    import torch
    from crystalformer_b200.synthetic import make_config
    wl = WORKLOADS[name]
    cb = make_config(wl["config"])
    model, params = make_model(wl["layers"], wl["K"])
    model = model.to(device)
    batch = to_device_batch(cb, device)
    fix_gauss_scale(model, batch)
    counts = (cb.num_atoms, cb.num_edges, int(cb.sizes.max()))
    log = []

    def step():
        with torch.no_grad():
            return model(batch, counts=counts)

    ms, diag = timer.run(step, 10, 3, target_ms=150.0, max_rounds=10)
    model.encoder.attention_event_log = log  # (the attention calls are timed in a round of their own)
    timer.one_round(step, 10)
    model.encoder.attention_event_log = None
    out = {"metric": metric_name(wl["layers"]), "crystals": cb.num_crystals, "atoms": cb.num_atoms, "edges": cb.num_edges,
           "layers": wl["layers"], "K": wl["K"], "ms_per_step": ms, "crystals_per_s": cb.num_crystals / (ms * 1e-3),
           "attention_us_per_call": 1e3 * sum(s.elapsed_time(e) for s, e in log) / max(len(log), 1),
           "timed_steps": diag["timed_steps"], "host_issue_ms_per_step": diag["host_issue_ms_per_step"]}
    if with_cpu:
        import oracle as _oracle
        from oracle.model_cpu import forward_cpu
        sample = cb.select(range({"cfg2": 64, "cfg4": 2}.get(name, 8)))
        state = {k: v.detach().cpu() for k, v in model.state_dict().items()}
        use_ref = _oracle.have_ref()
        t0 = time.time()
        y_cpu = forward_cpu(state, params, sample, use_ref=use_ref)
        dt = time.time() - t0
        with torch.no_grad():
            y_gpu = model(to_device_batch(sample, device)).cpu().numpy()
        out["cpu_reference"] = {"value": sample.num_crystals / dt, "unit": "crystals/s", "cores": os.cpu_count(),
                                "kind": "reference" if use_ref else "port",
                                "sample": f"first {sample.num_crystals} crystals, one forward pass, {dt:.1f} s"}
        out["parity"] = {"max_rel": float(np.abs(y_gpu - y_cpu).max() / np.abs(y_cpu).max()), "tol": PARITY_TOL,
                         "crystals": sample.num_crystals}
    return out


def strong_scaling_case(name, rank, world, device, timer):
    """The configuration's fixed batch split over the ranks by lpt_assign (the reference's rule,
    models/latticeformer.py:243-252), outputs gathered by peer stores; rank 0 also times the unsplit batch alone."""
    import torch
    import torch.distributed as dist
    from crystalformer_b200.sharding import PeerGather, crystal_cost, lpt_assign, shard_balance
    from crystalformer_b200.synthetic import make_config
    wl = WORKLOADS[name]
    cb = make_config(wl["config"])
    model, _ = make_model(wl["layers"], wl["K"])
    model = model.to(device)
    whole = to_device_batch(cb, device)
    fix_gauss_scale(model, whole)  # (every rank computes the same statistics from the same whole batch)
    cost = crystal_cost(cb.sizes, cb.trans_vec)
    shards = lpt_assign(cb.sizes, world, weights=cost)
    mine = cb.select(shards[rank])
    part = to_device_batch(mine, device)
    counts = (mine.num_atoms, mine.num_edges, int(mine.sizes.max()) if mine.num_crystals else 1)
    peers = PeerGather(shards, model.mlp[-1].out_features, device, slots=8, overlap=True)

    def step():
        with torch.no_grad():
            return model(part, counts=counts, gather=peers)

    ms, _ = timer.run(step, 10, 3, target_ms=150.0, max_rounds=10, finish=peers.wait_ready)
    peers.check()
    with torch.no_grad():
        y_all = model(part, counts=counts, gather=peers)
    peers.wait_ready()
    peers.check()
    # the unsplit batch on one GPU (rank 0 alone; the others wait)
    single = torch.zeros(1, dtype=torch.float64, device=device)
    ok = True
    if rank == 0:
        wcounts = (cb.num_atoms, cb.num_edges, int(cb.sizes.max()))
        alone = StepTimer(device, 1, share=timer)

        def whole_step():
            with torch.no_grad():
                return model(whole, counts=wcounts)

        ms1, _ = alone.run(whole_step, 10, 3, target_ms=150.0, max_rounds=10)
        single[0] = ms1
        y_one = whole_step()
        ok = bool((y_all - y_one).abs().max() <= 1e-5 * y_one.abs().max())
    dist.all_reduce(single, op=dist.ReduceOp.MAX)
    dist.barrier()
    peers.close()
    edges = [int((cb.sizes[s] ** 2).sum()) for s in shards]
    return {"crystals": cb.num_crystals, "ms_per_step": ms, "crystals_per_s": cb.num_crystals / (ms * 1e-3),
            "ms_per_step_n1": float(single.item()), "speedup_vs_n1": float(single.item()) / ms,
            "edges_max_over_mean": shard_balance(cb.sizes, shards)["edges_max_over_mean"],
            "cost_max_over_mean": shard_balance(cb.sizes, shards, cost)["cost_max_over_mean"],
            "largest_crystal_edges_over_mean_shard": float(int(cb.sizes.max()) ** 2 / (sum(edges) / world)),
            "sharded_equals_unsharded": ok}


def run_kernel_case(args):
    """--only microbench : the lattice-sum kernels on --pairs pairs (3 warm-up + 10 timed launches).
    --only attention  : the fused attention forward on the workload's crystals (3 warm-up + 10 timed calls).
    --only train      : one training step (forward + backward, L1 loss against N(0,1) targets, autograd path) of the
                        4-layer K=64 model on the 256-crystal training batch (1-40 atoms), 5 warm-up + 20 timed steps."""
    import torch
    from crystalformer_b200 import ops
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if args.only == "microbench":
        return lattice_microbench(ops, device, None, pairs=args.pairs)
    from crystalformer_b200.encoder import BatchGeometry
    from crystalformer_b200.synthetic import make_config
    if args.only == "train":
        return train_step_case(ops, device, args.crystals)
    wl = WORKLOADS[args.workload]
    cb = make_config(wl["config"], num_crystals=args.crystals or wl["crystals"])
    d = lambda x: torch.as_tensor(np.ascontiguousarray(x)).to(device)
    g = BatchGeometry(d(cb.pos), d(cb.trans_vec), d(cb.sizes), cb.num_atoms, cb.num_edges, int(cb.sizes.max()))
    gen = torch.Generator(device=device).manual_seed(0)
    N, K = cb.num_atoms, wl["K"]
    q = torch.randn((N, 8, 16), device=device, generator=gen) * 0.3
    k, v = (torch.randn((N, 8, 16), device=device, generator=gen) for _ in range(2))
    a = -0.5 / (1.4 * (1 + 0.1 * torch.randn((N, 8), device=device, generator=gen)).clamp(0.75, 1.4)) ** 2
    W = torch.randn((8, 16, 64), device=device, generator=gen) * 0.1 if K else None
    tvecs = d(cb.trans_vec)
    geo = (g.pos_ij, tvecs, g.rvlen, g.batch, g.edges, g.row_start, g.max_atoms)
    run = lambda: ops.infinite_attn_fwd(q, k, v, a, *geo, K, 14.0, 1.0, W, -3.5, 2, 2, row_order=g.row_order)

    def graph_ms(fn, reps=20):
        """Device time per call with the host out of the way: `reps` calls captured in one CUDA graph."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(reps):
                    fn()
            graph.replay()
            torch.cuda.synchronize()
            best = 1e30
            for _ in range(5):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record(); graph.replay(); e.record(); e.synchronize()
                best = min(best, s.elapsed_time(e) / reps)
        torch.cuda.current_stream().wait_stream(side)
        return best

    # the same call reading the batch's term lists / row lists (built once per batch, shared by the layers)
    a_widest = -0.5 * 0.5 / 1.4 ** 2
    build = lambda: ops.term_list_build(*geo, -3.5, 2, 2, a_widest, row_order=g.row_order)
    lists = build()
    run_listed = lambda: ops.infinite_attn_fwd(q, k, v, a, *geo, K, 14.0, 1.0, W, -3.5, 2, 2, row_order=g.row_order,
                                               term_lists=lists)
    out = {"case": "attention", "workload": args.workload, "crystals": cb.num_crystals, "atoms": N, "edges": cb.num_edges,
           "K": K, "device_ms_per_call_graph": graph_ms(run), "device_ms_per_call_listed_graph": graph_ms(run_listed),
           "device_ms_list_build_graph": graph_ms(build),
           "listed_vs_enumerated_rel_diff": float((run_listed()[0] - run()[0]).abs().max() / run()[0].abs().max())}
    if K == 64 and g.max_atoms <= 32:
        build_rows = lambda: ops.row_list_build(*geo, -3.5, 2, 2, a_widest, row_order=g.row_order)
        rows = build_rows()
        run_sorted = lambda: ops.infinite_attn_fwd_sorted(q, k, v, a, *geo, K, 14.0, 1.0, W, -3.5, 2, 2, rows)
        out["device_ms_per_call_sorted_graph"] = graph_ms(run_sorted)
        out["device_ms_row_list_build_graph"] = graph_ms(build_rows)
        out["sorted_vs_enumerated_rel_diff"] = float((run_sorted()[0] - run()[0]).abs().max() / run()[0].abs().max())
    return out


def train_step_case(ops, device, crystals=None):
    """Device time of a training step and of the fused attention operators inside it (forward and backward)."""
    import torch
    from crystalformer_b200.synthetic import make_config
    cb = make_config("cfg3", num_crystals=crystals)
    model, _ = make_model(4, 64)
    model = model.to(device)
    batch = to_device_batch(cb, device)
    fix_gauss_scale(model, batch)
    model.train()
    counts = (cb.num_atoms, cb.num_edges, int(cb.sizes.max()))
    target = torch.randn((cb.num_crystals, 1), device=device, generator=torch.Generator(device=device).manual_seed(3))
    events = {"fwd": [], "bwd": []}
    on = {"v": False}

    def wrap(fn, key):
        def inner(*a, **k):
            if not on["v"]:
                return fn(*a, **k)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(); r = fn(*a, **k); e.record()
            events[key].append((s, e))
            return r
        return inner

    raw = ops.infinite_attn_fwd, ops.infinite_attn_bwd
    ops.infinite_attn_fwd, ops.infinite_attn_bwd = wrap(raw[0], "fwd"), wrap(raw[1], "bwd")

    weights = [w for w in model.parameters() if w.requires_grad]

    def step():
        for w in weights:  # (what zero_grad(set_to_none=True) does, without walking the module tree every step)
            w.grad = None
        loss = (model(batch, counts=counts) - target).abs().mean()
        loss.backward()
        return loss

    try:
        for _ in range(5):
            step()
        torch.cuda.synchronize()
        reps = 20
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        s.record()
        for _ in range(reps):
            loss = step()
        e.record()
        host = time.perf_counter() - t0
        torch.cuda.synchronize()
        # the attention operators are timed in three more steps: their event pairs cost the host time that the timed
        # steps, which the host's issue rate bounds, should not pay
        on["v"] = True
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    finally:
        ops.infinite_attn_fwd, ops.infinite_attn_bwd = raw
    ms = s.elapsed_time(e) / reps
    per = {k: sum(a.elapsed_time(b) for a, b in v) / max(len(v), 1) for k, v in events.items()}
    return {"case": "train", "workload": "cfg3", "metric": "training step (fwd + bwd, L1 loss)", "crystals": cb.num_crystals,
            "atoms": cb.num_atoms, "edges": cb.num_edges,
            "ms_per_step": ms, "crystals_per_s": cb.num_crystals / (ms * 1e-3), "host_issue_ms": host * 1e3 / reps,
            "attention_fwd_us": per["fwd"] * 1e3, "attention_bwd_us": per["bwd"] * 1e3,
            "attention_calls_per_step": len(events["fwd"]) // 3, "loss": float(loss.item()),
            "timing": "20 steps back to back between one CUDA-event pair (no L2 flush: the step's working set of "
                      "activations exceeds what survives between uses anyway)",
            "note": "term lists built once per step inside the first forward call; the rest of the step is torch autograd"}


def lattice_microbench(ops, device, peaks, pairs=250000):
    """2,000,000 (i,j,head) items = 250,000 pairs x 8 heads from 4096 crystals, one width per item, phi + 64-bin psi."""
    import torch
    from crystalformer_b200.synthetic import microbench_edges
    cb, edges, pos_ij, a = microbench_edges(num_pairs=pairs)
    d = lambda x: torch.as_tensor(np.ascontiguousarray(x)).to(device)
    sizes = d(cb.sizes)
    atom_start, edge_start = ops.crystal_offsets(sizes)
    geo = ops.batch_prepare(d(cb.pos), d(cb.trans_vec), sizes, atom_start, edge_start, cb.num_atoms, 0, want_edges=False,
                            want_pos_ij=False)
    A, P, T, Bt, Ed = d(a), d(pos_ij), d(cb.trans_vec), d(cb.batch), d(edges)
    box = ops.lattice_box(A, Bt, Ed, geo["rvlen"], -3.5, 2, 2, a_per_edge=True).max(dim=1).values.long()
    terms = int(((2 * box[:, 0] + 1) * (2 * box[:, 1] + 1) * (2 * box[:, 2] + 1)).sum())
    E = edges.shape[1]
    z = torch.empty((E, 8), device=device)
    v = torch.empty((E, 8, 64), device=device)
    run = lambda: ops.lattice_sum_fwd(A, P, T, Bt, Ed, 64, 14.0, 1.0, rvlen=geo["rvlen"], cutoff_radius=-3.5,
                                      lattice_range=2, minimum_range=2, a_per_edge=True, z=z, v=v)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    times = []
    for _ in range(10):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); run(); e.record(); e.synchronize()
        times.append(s.elapsed_time(e) * 1e-3)
    t = float(np.median(times))
    work = terms * fp32_instr_per_term(64)
    out_bytes = E * 8 * 65 * 4
    if peaks is None:
        return {"case": "microbench", "items": E * 8, "edges": E, "terms": terms, "ms": t * 1e3}
    return {"items": E * 8, "edges": E, "terms": terms, "ms": t * 1e3, "items_per_s": E * 8 / t,
            "algorithmic_fp32_rate_over_probe": work / t / peaks["fp32"],
            "algorithmic_sfu_rate_over_probe": terms * sfu_per_term(64) / t / peaks["sfu"],
            "note": "algorithmic = every (edge, translation) term of the boxes x the reference's per-term instruction "
                    "count, divided by the time: the kernels skip terms below the weight floor, so this is a speed-up "
                    "over the enumeration, not a pipe utilisation (ncu: XU 37 %, ALU 43 %, FMA 22 % of peak, "
                    "profiles/ncu_full_lattice_psi_microbench80k.md)",
            "hbm_gbs": out_bytes / t / 1e9, "hbm_frac": out_bytes / t / 6558.7e9,
            "kernels": "lattice_phi_kernel + lattice_psi_kernel", "l2": "output 520 MB per launch exceeds L2"}


def cpu_baseline(model, params, cb, seconds_budget=10.0):
    """The CPU reference's model forward on the WHOLE batch (its outputs are the parity reference of the run), repeated
    until about `seconds_budget` seconds of CPU work have been timed.  Returns (record, outputs)."""
    from oracle.model_cpu import forward_cpu
    import oracle as _oracle
    state = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    use_ref = _oracle.have_ref() and params.value_pe_dist_real in (0, 64)
    t0 = time.time()
    y = forward_cpu(state, params, cb, use_ref=use_ref)
    dt = time.time() - t0
    passes = 1
    while dt < seconds_budget and passes < 8:
        t1 = time.time()
        forward_cpu(state, params, cb, use_ref=use_ref)
        dt += time.time() - t1
        passes += 1
    rec = {"value": cb.num_crystals * passes / dt, "unit": "crystals/s", "cores": os.cpu_count(),
           "kind": "reference" if use_ref else "port",
           "what": ("the reference's CUDA kernel sources (real_enc_proj_fwd, fused_dpa_fwd_v3) compiled for the CPU with "
                    "OpenMP over edges / atoms, dense layers by torch CPU" if use_ref else
                    "the C restatement of the reference kernels, dense layers by torch CPU"),
           "sample": f"all {cb.num_crystals} crystals of the batch, {passes} forward pass(es), {dt:.1f} s, all host cores"}
    return rec, y


def run_reference(args):
    """The reference arm: the reference's CPU implementation of the path on the host cores, rank 0 only, on the same
    workload: the same seeded batch and the same seed-0 model weights as the other arm (the Gaussian-width statistics
    are taken from the batch inside the forward, which is what the other arm's calibration pass stores)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    import torch
    import oracle as _oracle
    from oracle.model_cpu import forward_cpu
    from crystalformer_b200.synthetic import make_config
    torch.set_num_threads(os.cpu_count())
    wl = WORKLOADS[args.workload]
    world = args.gpus
    cb = make_config(wl["config"], num_crystals=wl["crystals"])  # (the other arm's global batch is N copies of it)
    model, params = make_model(wl["layers"], wl["K"])  # CPU module: a container of the seed-0 weights, never run
    state = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    use_ref = _oracle.have_ref()
    # a step = the batch of one GPU of the other arm
    sample = cb
    t0 = time.time()
    forward_cpu(state, params, sample.select(range(min(8, sample.num_crystals))), use_ref=use_ref)  # warm-up (page-in, OpenMP pool)
    t0 = time.time()
    forward_cpu(state, params, sample, use_ref=use_ref)
    first = time.time() - t0
    steps = int(max(1, min(args.steps, math.floor(150.0 / max(first, 1e-3)))))
    dt = first
    for _ in range(steps - 1):
        t1 = time.time()
        forward_cpu(state, params, sample, use_ref=use_ref)
        dt += time.time() - t1
    value = sample.num_crystals * steps / dt
    kind = "reference" if use_ref else "port"
    return {
        "impl": "reference", "metric": metric_name(wl["layers"]),
        "value": value, "unit": "crystals/s", "n_gpus": world, "steps": steps, "warmup": 1,
        "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {wl['layers']}-layer Crystalformer forward, K={wl['K']}, "
                               f"{wl['crystals']} crystals per GPU per step",
                   "weights": "seed 0, the same construction as the other arm",
                   "arm": ("the reference's own CUDA kernel sources compiled for the CPU (oracle/_ref), OpenMP over all host "
                           "cores; not its PyTorch path, which is several times slower" if use_ref else
                           "C restatement of the reference kernels (oracle/), OpenMP over all host cores"),
                   "steps_requested": args.steps,
                   "steps_note": "as many of the requested steps as fit in about 150 s of CPU time"},
        "cpu_baseline": {"value": value, "unit": "crystals/s", "cores": os.cpu_count(), "kind": kind,
                         "sample": f"{sample.num_crystals} crystals per step ({'the whole batch' if world == 1 else 'one rank share of the global batch'})"},
        "e2e": {"value": value, "unit": "crystals/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg0", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="skip the cfg2 / cfg4 / cfg3-train section")
    ap.add_argument("--no-strong", action="store_true", help="N > 1: skip the fixed-batch cfg2 / cfg4 section")
    ap.add_argument("--only", default=None, choices=["microbench", "attention", "train"],
                    help="run one kernel case a few times and exit (small, fixed work: meant for profiler captures)")
    ap.add_argument("--pairs", type=int, default=250000, help="(i,j) pairs of the lattice-sum microbenchmark")
    ap.add_argument("--crystals", type=int, default=None, help="crystals of the --only attention / train case")
    args = ap.parse_args()
    if args.only:
        print(json.dumps(run_kernel_case(args)))
        return
    if args.impl == "reference":
        result = run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        result = run_b200(args)
    if result is not None:
        print(json.dumps(result))
        parity = result.get("parity")
        if parity is not None and not parity["ok"]:
            raise SystemExit(f"parity check failed: {parity}")


if __name__ == "__main__":
    main()
