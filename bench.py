#!/usr/bin/env python
"""Benchmark of the infinitely-connected-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload cfg0|cfg2|cfg4]

One "step" is one forward pass of the Crystalformer model (4 layers, model_dim 128, 8 heads, 64 radial-basis bins for
cfg0/cfg4; 7 layers without the value encoding for cfg2) over one batch of seeded synthetic crystals.  Per GPU the batch
has the configuration's crystal count; with N GPUs a batch of N times that many crystals is drawn, split over the ranks
by the reference's greedy rule on n^2 (crystalformer_b200.sharding.lpt_assign) and only the per-crystal outputs are
gathered on every rank, by stores into the peers' memory (crystalformer_b200.sharding.PeerGather; weak scaling).
Rank 0 prints ONE JSON line:

  value            crystals / s over all ranks, inputs already resident in HBM, device-timed (CUDA events), max over ranks;
                   the steps are issued back to back (no host synchronisation in between), each inside its own event
                   pair, the L2 flush between the pairs
  e2e              the same through crystalformer_b200.serving.PipelinedPredictor with HOST inputs: pinned host -> device
                   copies of the step's inputs and the device -> host copy of the outputs are inside the timed region
  roofline         the dominant operator (the phi and row kernels of every layer's fused attention), timed live with
                   CUDA events on the launch stream during the timed steps; work = (edge, translation) terms of the
                   batch x FP32-pipe instructions per term; peak = FP32 FMA issue rate measured by cf_pipe_probe
  lattice_sum_microbench   the 2,000,000 (i,j,head) lattice-sum kernel benchmark (phi + 64-bin psi, forward), same units
  cpu_baseline     (N = 1) the CPU oracle's model forward on a bounded sample of the same batch, on the host cores

--impl reference times the reference's CPU implementation of the path (its own kernel sources compiled for the CPU
when oracle/_ref exists, else the C restatement) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
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


def fp32_instr_per_term(K, H=8):
    """FP32-pipe instructions per (edge, translation) term with the basis shared by the heads: geometry and minimum
    pass 25, two per bin, (2 + K) per head."""
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


def run_b200(args):
    import torch
    import torch.distributed as dist
    import types
    from crystalformer_b200 import ops
    from crystalformer_b200.encoder import BatchGeometry
    from crystalformer_b200.sharding import PeerGather, lpt_assign, shard_balance
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
    global_batch = make_config(wl["config"], num_crystals=wl["crystals"] * world)
    shards = lpt_assign(global_batch.sizes, world)
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

    # instrument the fused operator: CUDA events around every call, on the launching stream
    op_events = []
    raw_fwd = ops.infinite_attn_fwd
    record = {"on": False}

    def timed_fwd(*a, **kw):
        if not record["on"]:
            return raw_fwd(*a, **kw)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        r = raw_fwd(*a, **kw)
        e.record()
        op_events.append((s, e))
        return r

    ops.infinite_attn_fwd = timed_fwd          # torch-operator path
    native_log = []                            # one-call path: the library records the events itself
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)  # > 126 MB L2

    # N > 1: the pooling + head kernel of every rank stores its outputs into every rank's gather buffer over NVLink
    # and a small kernel waits for all ranks (sharding.PeerGather); no collective library on the data path.
    peers = PeerGather(shards, model.mlp[-1].out_features, device) if world > 1 else None
    extra = {} if peers is None else {"gather": peers}

    def step_resident():
        with torch.no_grad():
            return model(resident, counts=(n_atoms, n_edges, max_atoms), **extra)

    pinned = to_device_batch(mine, device, pinned=True)
    h2d_bytes = sum(t.numel() * t.element_size() for t in vars(pinned).values())
    d2h_bytes = (global_batch.num_crystals if world > 1 else mine.num_crystals) * 4

    from crystalformer_b200.serving import PipelinedPredictor
    runner = PipelinedPredictor(model, depth=3, device=device, gather=peers)
    pending = []

    def step_e2e():
        """One batch through the public serving API: pinned host inputs -> device -> forward -> outputs in pinned host
        memory.  Up to three batches are in flight; the host blocks only when it collects the oldest result."""
        pending.append(runner.submit(pinned))
        if len(pending) == runner.depth:
            runner.result(pending.pop(0))

    def drain():
        while pending:
            runner.result(pending.pop(0))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step, steps, warmup, instrument=False):
        """Device time of `steps` steps, max over ranks.  The steps are issued back to back, as a job that streams
        batches does: the host is not synchronised in between, so it can run ahead of the device.  Every step is
        bracketed by its own event pair on the compute stream and the L2 flush sits between the pairs, outside them."""
        for _ in range(warmup):
            step()
        drain()
        barrier()
        spans = []
        host_t0 = time.perf_counter()
        record["on"] = instrument
        model.encoder.attention_event_log = native_log if instrument else None
        for _ in range(steps):
            flush.zero_()  # L2 flush between timed iterations
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            step()
            e.record()
            spans.append((s, e))
        host_issue = time.perf_counter() - host_t0  # the host is done issuing; the device may still be busy
        drain()
        record["on"] = False
        model.encoder.attention_event_log = None
        barrier()
        total = sum(s.elapsed_time(e) for s, e in spans)
        if peers is not None:
            peers.check()  # raises if a collect gave up waiting for a rank
        t = torch.tensor([total], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        # where the time went on this rank: its own spans, the device wall clock from the first step's start to the
        # last step's end (flushes and any idle gaps included) and the host time spent issuing the steps
        mine_diag = {"rank": rank, "span_ms_per_step": total / steps,
                     "device_wall_ms_per_step": spans[0][0].elapsed_time(spans[-1][1]) / steps,
                     "host_issue_ms_per_step": host_issue * 1e3 / steps}
        every = [mine_diag]
        if world > 1:
            every = [None] * world
            dist.all_gather_object(every, mine_diag)
        diag.append(every)
        return float(t.item())  # ms for all steps, max over ranks

    diag = []
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        time.sleep(0.3)  # let nvidia-smi start sampling
    t_begin = time.time()
    ms_total = timed(step_resident, args.steps, args.warmup, instrument=True)
    t_end = time.time()
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    op_events += native_log
    op_ms = sum(s.elapsed_time(e) for s, e in op_events)
    op_calls = len(op_events)
    ms_e2e = timed(step_e2e, args.steps, args.warmup)

    total_crystals = global_batch.num_crystals
    value = total_crystals * args.steps / (ms_total * 1e-3)
    e2e_value = total_crystals * args.steps / (ms_e2e * 1e-3)

    result = None
    if rank == 0:
        # ---- roofline of the dominant operator
        K = wl["K"]
        sink = torch.zeros(4, device=device)
        peaks = {}
        for kind, name in ((0, "fp32"), (1, "sfu")):
            blocks, threads, iters = ops_sm_count(device) * 8, 256, 1 << 13
            best = 1e30
            for _ in range(5):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record(); ops.pipe_probe(kind, blocks, threads, iters, sink); e.record(); e.synchronize()
                best = min(best, s.elapsed_time(e))
            peaks[name] = blocks * threads * iters * 8 / (best * 1e-3)  # lane-instructions / s
        terms_per_call = n_edges * FIXED_BOX_TERMS  # lower bound: the adaptive rule never shrinks the minimum box
        t_call = op_ms * 1e-3 / max(op_calls, 1)
        achieved = terms_per_call * fp32_instr_per_term(K) / t_call
        achieved_sfu = terms_per_call * sfu_per_term(K) / t_call
        # crystals of up to 32 atoms with a value encoding: the row kernel sums phi from the term lists itself
        phi_in_row = K > 0 and max_atoms <= 32 and os.environ.get("CF_PHI_IN_ROW", "1") != "0"
        roofline = {
            "kernel": ("infinite_attn_rows_kernel, phi summed from the term lists inside (one fused-attention call)"
                       if phi_in_row else "phi_from_list_kernel + infinite_attn_rows_kernel (one fused-attention call)"),
            "bound": "fp32_simt", "achieved": achieved / 1e9, "peak": peaks["fp32"] / 1e9, "unit": "G lane-instr/s",
            "frac": achieved / peaks["fp32"], "peak_source": "cf_pipe_probe FFMA, measured in this run",
            "sfu": {"achieved": achieved_sfu / 1e9, "peak": peaks["sfu"] / 1e9, "frac": achieved_sfu / peaks["sfu"]},
            "terms_per_launch": terms_per_call, "launches": op_calls, "avg_launch_us": t_call * 1e6,
            "share_of_step": op_ms / ms_total,
            # dram__bytes_read.sum + dram__bytes_write.sum per fused-attention call from the ncu capture of this workload
            # (row kernel with phi inside: 11.95 MB at cfg0, caches cold under ncu, of which 8 MB are the term lists; the
            # two-kernel form read 8.33 + 13.09 MB); not re-measured per run, and only known for cfg0
            "traffic": (11.95e6 if phi_in_row else 21.4e6) if args.workload == "cfg0" else None,
            "traffic_unit": "bytes per call (ncu, cfg0, cold caches)",
            "note": "work counted for EVERY (edge, translation) term; terms whose weights fall below 2^-30 are skipped "
                    "by the kernel, so frac may exceed the executed-instruction utilisation",
        }
        micro = lattice_microbench(ops, device, peaks)
        cpu = cpu_baseline(model, params, mine) if (world == 1 and not args.no_cpu_baseline) else None
        # own kernels per forward: geometry (offsets, cells, atoms, edges, row order; the offsets are a launch of their own
        # above 1024 crystals), term lists; L + 1 dense blocks; per layer rows (and phi, unless the row kernel computes
        # it); pooling + head (N > 1: + the collect of the peer gather)
        geometry = 1 if mine.num_crystals <= 1024 else 2
        per_step_launches = (geometry + 1 + (wl["layers"] + 1) + (1 if phi_in_row else 2) * wl["layers"] + 1
                             + (1 if world > 1 else 0))
        result = {
            "metric": "crystals/sec (4-layer, fwd)" if wl["layers"] == 4 else f"crystals/sec ({wl['layers']}-layer, fwd)",
            "value": value, "unit": "crystals/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {wl['layers']}-layer Crystalformer forward, K={K}, "
                                   f"{wl['crystals']} crystals per GPU per step", "global_batch": total_crystals,
                       "atoms_this_rank": n_atoms, "edges_this_rank": n_edges, "cutoff": "adaptive -3.5 sigma, minimum box R=2",
                       "l2": "flushed between timed steps (256 MB write between the per-step event pairs)",
                       "timing": "steps issued back to back without host synchronisation; sum of per-step event spans",
                       "parallelism": f"dp{world} (LPT on n^2, outputs gathered by peer stores)",
                       "shard_balance": shard_balance(global_batch.sizes, shards)},
            "per_rank": {"resident": diag[0], "e2e": diag[1]},
            "e2e": {"value": e2e_value, "unit": "crystals/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                    "api": "crystalformer_b200.serving.PipelinedPredictor, 3 batches in flight"},
            "gpu_launches": per_step_launches * args.steps,
            "roofline": roofline, "lattice_sum_microbench": micro, "cpu_baseline": cpu, "clocks": clocks,
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result


def ops_sm_count(device):
    import torch
    return torch.cuda.get_device_properties(device).multi_processor_count


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
        return train_step_case(ops, device, args)
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
    run = lambda: ops.infinite_attn_fwd(q, k, v, a, g.pos_ij, tvecs, g.rvlen, g.batch, g.edges, g.row_start,
                                        g.max_atoms, K, 14.0, 1.0, W, -3.5, 2, 2, row_order=g.row_order)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    times = []
    for _ in range(10):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); run(); e.record(); e.synchronize()
        times.append(s.elapsed_time(e))
    phi_only = lambda: ops.lattice_sum_fwd(a, g.pos_ij, tvecs, g.batch, g.edges, 0, 14.0, 1.0, rvlen=g.rvlen,
                                           cutoff_radius=-3.5)
    for _ in range(3):
        phi_only()
    torch.cuda.synchronize()
    phi_times = []
    for _ in range(10):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); phi_only(); e.record(); e.synchronize()
        phi_times.append(s.elapsed_time(e))
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

    # the same call reading the batch's term lists (built once per batch, shared by the layers)
    a_widest = -0.5 * 0.5 / 1.4 ** 2
    build = lambda: ops.term_list_build(g.pos_ij, tvecs, g.rvlen, g.batch, g.edges, g.row_start, g.max_atoms, -3.5, 2, 2,
                                        a_widest, row_order=g.row_order)
    lists = build()
    run_listed = lambda: ops.infinite_attn_fwd(q, k, v, a, g.pos_ij, tvecs, g.rvlen, g.batch, g.edges, g.row_start,
                                               g.max_atoms, K, 14.0, 1.0, W, -3.5, 2, 2, row_order=g.row_order,
                                               term_lists=lists)
    diff = float((run_listed()[0] - run()[0]).abs().max() / run()[0].abs().max())
    return {"case": "attention", "workload": args.workload, "crystals": cb.num_crystals, "atoms": N, "edges": cb.num_edges,
            "K": K, "ms_median": float(np.median(times)), "ms_min": float(min(times)),
            "phi_kernel_alone_ms": float(np.median(phi_times)),
            "device_ms_per_call_graph": graph_ms(run), "device_ms_phi_graph": graph_ms(phi_only),
            "device_ms_per_call_listed_graph": graph_ms(run_listed), "device_ms_list_build_graph": graph_ms(build),
            "listed_vs_enumerated_rel_diff": diff}


def train_step_case(ops, device, args):
    """Device time of a training step and of the fused attention operators inside it (forward and backward)."""
    import torch
    from crystalformer_b200.synthetic import make_config
    cb = make_config("cfg3", num_crystals=args.crystals)
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

    def step():
        model.zero_grad(set_to_none=True)
        loss = (model(batch, counts=counts) - target).abs().mean()
        loss.backward()
        return loss

    try:
        for _ in range(5):
            step()
        torch.cuda.synchronize()
        on["v"] = True
        reps = 20
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        s.record()
        for _ in range(reps):
            loss = step()
        e.record()
        host = time.perf_counter() - t0
        torch.cuda.synchronize()
    finally:
        ops.infinite_attn_fwd, ops.infinite_attn_bwd = raw
    ms = s.elapsed_time(e) / reps
    per = {k: sum(a.elapsed_time(b) for a, b in v) / max(len(v), 1) for k, v in events.items()}
    return {"case": "train", "workload": "cfg3", "crystals": cb.num_crystals, "atoms": cb.num_atoms, "edges": cb.num_edges,
            "ms_per_step": ms, "crystals_per_s": cb.num_crystals / (ms * 1e-3), "host_issue_ms_per_step": host * 1e3 / reps,
            "attention_fwd_ms_per_call": per["fwd"], "attention_bwd_ms_per_call": per["bwd"],
            "attention_calls_per_step": len(events["fwd"]) // reps, "loss": float(loss.item()),
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
            "fp32_frac": work / t / peaks["fp32"], "sfu_frac": terms * sfu_per_term(64) / t / peaks["sfu"],
            "hbm_gbs": out_bytes / t / 1e9, "kernels": "lattice_phi_kernel + lattice_psi_kernel",
            "l2": "output 520 MB per launch exceeds L2"}


def cpu_baseline(model, params, cb, seconds_budget=20.0):
    """The CPU oracle's model forward on the first crystals of the batch (about 10-30 s of CPU work)."""
    from oracle.model_cpu import forward_cpu
    import oracle as _oracle
    state = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    use_ref = _oracle.have_ref() and params.value_pe_dist_real in (0, 64)
    sample = min(8, cb.num_crystals)
    t0 = time.time(); forward_cpu(state, params, cb.select(range(sample)), use_ref=use_ref); dt = time.time() - t0
    rate = sample / dt
    sample2 = int(min(cb.num_crystals, max(sample, rate * seconds_budget)))
    if sample2 > sample:
        t0 = time.time(); forward_cpu(state, params, cb.select(range(sample2)), use_ref=use_ref); dt = time.time() - t0
        sample = sample2
    passes = 1
    if dt < 10.0:  # a whole batch takes only a few seconds: repeat it, so that about 10 s of CPU work are timed
        passes = int(min(8, max(2, round(10.0 / max(dt, 1e-3)))))
        t0 = time.time()
        for _ in range(passes):
            forward_cpu(state, params, cb.select(range(sample)), use_ref=use_ref)
        dt = time.time() - t0
    return {"value": sample * passes / dt, "unit": "crystals/s", "cores": os.cpu_count(),
            "kind": "reference" if use_ref else "port",
            "sample": f"first {sample} crystals of the batch, {passes} forward pass(es), {dt:.1f} s, OpenMP over all host cores"}


def run_reference(args):
    """The reference arm: the reference's CPU implementation of the path on the host cores, rank 0 only."""
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
    cb = make_config(wl["config"], num_crystals=wl["crystals"] * world)
    # a CPU-only model with the same architecture and random init; no kernels of this repository are involved
    params, state = reference_state(wl["layers"], wl["K"])
    use_ref = _oracle.have_ref()
    sample = cb.select(range(min(cb.num_crystals, args.reference_sample)))
    for _ in range(min(args.warmup, 1)):
        forward_cpu(state, params, sample.select(range(min(2, sample.num_crystals))), use_ref=use_ref)
    t0 = time.time()
    for _ in range(args.steps):
        forward_cpu(state, params, sample, use_ref=use_ref)
    dt = time.time() - t0
    value = sample.num_crystals * args.steps / dt
    return {
        "impl": "reference", "metric": "crystals/sec (4-layer, fwd)" if wl["layers"] == 4 else f"crystals/sec ({wl['layers']}-layer, fwd)",
        "value": value, "unit": "crystals/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {wl['layers']}-layer Crystalformer forward, K={wl['K']}, "
                               f"{wl['crystals']} crystals per GPU per step"},
        "cpu_baseline": {"value": value, "unit": "crystals/s", "cores": os.cpu_count(),
                         "kind": "reference" if use_ref else "port",
                         "sample": f"first {sample.num_crystals} crystals of the batch per step"},
        "e2e": {"value": value, "unit": "crystals/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def reference_state(layers, K, seed=0):
    """Random-init weights with the model's shapes, drawn on the CPU without constructing any CUDA-backed module."""
    import torch
    import types
    from crystalformer_b200.params import DEFAULT_MODEL_PARAMS
    p = dict(DEFAULT_MODEL_PARAMS); p.update(num_layers=layers, value_pe_dist_real=K)
    params = types.SimpleNamespace(**p)
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=0.05: torch.randn(*s, generator=g) * std
    st = {"input_embeddings.weight": r(128, 98)}
    for l in range(layers):
        pre = f"encoder.layers.{l}.self_attn."
        for n in "qkv":
            st[pre + f"{n}_proj_weight"] = r(128, 128, std=0.1)
        st[pre + "in_proj_bias"] = torch.zeros(384)
        st[pre + "lattice_pos_weights"] = r(128, std=0.25)
        st[pre + "gauss_scale"] = torch.tensor([20.0, 0.0])
        if K > 0:
            st[pre + "pe_dist_proj"] = r(1, 8, 16, K, std=0.1)
        st[pre + "out_proj.weight"] = r(128, 128, std=0.1)
        st[pre + "out_proj.bias"] = torch.zeros(128)
        st[f"encoder.layers.{l}.linear1.weight"] = r(512, 128); st[f"encoder.layers.{l}.linear1.bias"] = torch.zeros(512)
        st[f"encoder.layers.{l}.linear2.weight"] = r(128, 512); st[f"encoder.layers.{l}.linear2.bias"] = torch.zeros(128)
    st["mlp.0.weight"] = r(128, 128); st["mlp.0.bias"] = torch.zeros(128)
    st["mlp.3.weight"] = r(1, 128); st["mlp.3.bias"] = torch.zeros(1)
    return params, st


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg0", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--reference-sample", type=int, default=24, help="crystals per step of the reference arm")
    ap.add_argument("--only", default=None, choices=["microbench", "attention", "train"],
                    help="run one kernel case a few times and exit (small, fixed work: meant for profiler captures)")
    ap.add_argument("--pairs", type=int, default=250000, help="(i,j) pairs of the lattice-sum microbenchmark")
    ap.add_argument("--crystals", type=int, default=None, help="crystals of the --only attention case")
    args = ap.parse_args()
    if args.only:
        print(json.dumps(run_kernel_case(args)))
        return
    if args.impl == "reference":
        args.steps = min(args.steps, 5)
        result = run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        result = run_b200(args)
    if result is not None:
        print(json.dumps(result))


if __name__ == "__main__":
    main()
