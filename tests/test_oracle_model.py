"""The CPU restatement of the model forward (oracle/model_cpu.py) against the reference model's own outputs, and the
sharding helpers on CPU ranks (gloo).  No GPU."""
import json
import os
import sys
import types

import numpy as np
import pytest
import torch

import oracle
from conftest import rel_err
from crystalformer_b200.sharding import crystal_cost, gather_outputs, lpt_assign, shard_balance
from crystalformer_b200.synthetic import CrystalBatch, make_config, make_crystals, uniform_atoms

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def golden_batch(g):
    z = g["in_x"].argmax(1) + 1
    return CrystalBatch(x=g["in_x"], pos=g["in_pos"], trans_vec=g["in_trans"], sizes=g["in_sizes"], batch=g["in_batch"], z=z)


@pytest.mark.parametrize("use_ref", [False, True])
def test_cpu_model_matches_reference_model(golden_model, use_ref):
    if use_ref and not oracle.have_ref():
        pytest.skip("reference kernels were not compiled for the CPU here")
    from oracle.model_cpu import forward_cpu
    g = golden_model
    P = types.SimpleNamespace(**json.loads(bytes(g["in_params_json"]).decode()))
    state = {k[len("state:"):]: v for k, v in g.items() if k.startswith("state:")}
    y = forward_cpu(state, P, golden_batch(g), use_ref=use_ref)
    assert rel_err(y, g["y_f64"]) < 1e-4


def test_lpt_assignment_follows_the_reference_rule():
    sizes = [5, 30, 1, 17, 17, 2, 29, 8]
    shards = lpt_assign(sizes, 3)
    assert sorted(sum(shards, [])) == list(range(8))
    # descending n^2: 30, 29, 17, 17, 8, 5, 2, 1 ; totals start at (1, 0, 0)
    assert shards == [[3, 4, 7, 0, 5, 2], [1], [6]]
    e = [sum(sizes[i] ** 2 for i in s) for s in shards]
    assert max(e) - min(e) <= max(s * s for s in sizes)
    cb = make_config("cfg0", num_crystals=1024)
    for n in (2, 4, 8):
        bal = shard_balance(cb.sizes, lpt_assign(cb.sizes, n))
        assert bal["edges_max_over_mean"] < 1.01
        # the same greedy rule on a weight that also knows the cell volumes: every crystal placed once, weights balanced
        cost = crystal_cost(cb.sizes, cb.trans_vec)
        by_cost = lpt_assign(cb.sizes, n, weights=cost)
        assert sorted(sum(by_cost, [])) == list(range(cb.num_crystals))
        assert shard_balance(cb.sizes, by_cost, cost)["cost_max_over_mean"] < 1.01
    assert lpt_assign(sizes, 3, weights=[s * s for s in sizes]) == shards


def test_empty_and_single_shard_gather():
    out = gather_outputs(torch.arange(6.0).reshape(3, 2), [[2, 0, 1]])
    assert out.tolist() == [[2.0, 3.0], [4.0, 5.0], [0.0, 1.0]]


WORKER = r"""
import os, sys, json
sys.path.insert(0, {repo!r})
import numpy as np, torch, torch.distributed as dist
from crystalformer_b200.sharding import lpt_assign, gather_outputs
dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
rank, world = dist.get_rank(), dist.get_world_size()
sizes = [5, 30, 1, 17, 17, 2, 29, 8, 3]
shards = lpt_assign(sizes, world)
if os.environ.get("FAIL_RANK") == str(rank):
    raise SystemExit(3)  # a rank that leaves before the collective
local = torch.tensor([[float(c), float(sizes[c])] for c in shards[rank]]).reshape(-1, 2)
out = gather_outputs(local, shards)
assert out[:, 0].tolist() == [float(c) for c in range(len(sizes))], out
assert out[:, 1].tolist() == [float(s) for s in sizes]
if rank == 0:
    print("GATHER_OK")
dist.destroy_process_group()
"""


def run_ranks(tmp_path, world, extra_env=None, timeout=120):
    import subprocess
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(repo=REPO))
    port = 29500 + (os.getpid() % 400)
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   GLOO_SOCKET_IFNAME="lo", **(extra_env or {}))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        try:
            o, e = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            o, e = p.communicate()
        outs.append((p.returncode, o, e))
    return outs


@pytest.mark.parametrize("world", [2, 3])
def test_gather_across_cpu_ranks(tmp_path, world):
    outs = run_ranks(tmp_path, world)
    assert all(rc == 0 for rc, _, _ in outs), outs
    assert "GATHER_OK" in outs[0][1]


def test_a_rank_that_leaves_makes_the_others_fail_not_hang(tmp_path):
    """Failure is injected on the host: rank 1 exits before the gather; rank 0's collective ends with an error."""
    outs = run_ranks(tmp_path, 2, extra_env={"FAIL_RANK": "1"}, timeout=90)
    assert outs[1][0] == 3
    assert outs[0][0] != 0 and "GATHER_OK" not in outs[0][1]


def test_elu_width_function_equals_the_recorded_operations():
    """The one-node width pipeline of the attention module (training, default parameters) against the same arithmetic
    recorded operation by operation: equal values, equal gradients (float64, CPU)."""
    import torch
    import torch.nn.functional as F
    from crystalformer_b200.attention import EluWidthFunction
    torch.manual_seed(0)
    N, H, D = 37, 8, 16
    q = torch.randn(N, H, D, dtype=torch.float64, requires_grad=True)
    w = torch.randn(1, H, D, dtype=torch.float64, requires_grad=True)
    scale, shift = torch.tensor(0.7, dtype=torch.float64), torch.tensor(-0.2, dtype=torch.float64)
    beta, lb, c = 0.1, 0.5, -0.5 / 1.4 ** 2
    a = EluWidthFunction.apply(q, w, scale, shift, beta, lb, c)
    ga = torch.randn(N, H, dtype=torch.float64)
    gq, gw = torch.autograd.grad(a, (q, w), ga)
    alpha = ((q * w).sum(-1) + shift) * scale
    ref = ((1.0 - lb) * F.elu(alpha * (beta / (1.0 - lb))) + 1.0) * c
    rq, rw = torch.autograd.grad(ref, (q, w), ga)
    assert torch.equal(a, ref)
    assert torch.allclose(gq, rq, rtol=1e-12, atol=1e-14) and torch.allclose(gw, rw, rtol=1e-12, atol=1e-14)


def test_copies_of_a_batch_are_dealt_one_per_rank():
    """The weak-scaling batch of the benchmark: N copies of the one-GPU batch.  The greedy split on the row cost (which
    differs from crystal to crystal) gives every rank exactly one copy of every crystal; on n^2, where different crystals
    tie, every rank still gets the same multiset of sizes.  Either way the work per rank is the one-GPU work."""
    import numpy as np
    from crystalformer_b200.sharding import crystal_cost, lpt_assign
    from crystalformer_b200.synthetic import make_config
    one = make_config("cfg0", num_crystals=32)
    for world in (2, 4, 8):
        tiled = one.select(np.tile(np.arange(one.num_crystals), world))
        for weights in (None, crystal_cost(tiled.sizes, tiled.trans_vec)):
            shards = lpt_assign(tiled.sizes, world, weights=weights)
            assert sorted(i for s in shards for i in s) == list(range(tiled.num_crystals))
            for s in shards:
                if weights is None:
                    assert sorted(tiled.sizes[list(s)].tolist()) == sorted(one.sizes.tolist())
                else:
                    assert sorted(int(i) % one.num_crystals for i in s) == list(range(one.num_crystals))
