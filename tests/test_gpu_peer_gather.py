"""Peer gather (cf_peer_gather_store / cf_peer_gather_collect / the gather stage of cf_model_forward): every rank's
per-crystal outputs stored into every rank's buffer, against the index arithmetic of sharding.gather_outputs.

One GPU: the ranks are emulated in ONE process and ONE stream - all stores are complete before the first collect
starts, so no kernel ever waits for a kernel that has not run.  Two or more GPUs: real ranks as child processes with
the buffers mapped between them; the result must equal the library all-gather's."""
import ctypes
import json
import os
import subprocess
import sys
import types

import numpy as np
import pytest
import torch

from conftest import REPO

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


def test_emulated_ranks_store_then_collect():
    from crystalformer_b200 import _lib
    from crystalformer_b200.sharding import _gather_index, lpt_assign, peer_descriptor
    rng = np.random.default_rng(5)
    sizes = rng.integers(1, 30, size=37)
    world, targets = 3, 2
    shards = lpt_assign(sizes, world)
    longest = max(len(s) for s in shards)
    truth = torch.as_tensor(rng.standard_normal((len(sizes), targets)).astype(np.float32)).cuda()
    cells = [torch.zeros(world * longest * targets, dtype=torch.int64, device="cuda") for _ in range(world)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    index = _gather_index(shards, longest, torch.device("cuda"))
    for step in (1, 2, 0xFFFFFFFF):  # (the last one: a step with the top bit set)
        for r in range(world):
            local = (truth[torch.as_tensor(shards[r]).cuda()] * (step % 7 + 1)).contiguous()
            d = peer_descriptor(world, r, longest, step, [t.data_ptr() for t in cells])
            _lib.call("cf_peer_gather_store", local.data_ptr(), local.shape[0], targets, ctypes.byref(d), _stream())
        for r in range(world):
            out = torch.empty((len(sizes), targets), device="cuda")
            _lib.call("cf_peer_gather_collect", cells[r].data_ptr(), step, index.data_ptr(), len(sizes), targets,
                      longest, out.data_ptr(), status.data_ptr(), 5.0, _stream())
            assert torch.equal(out, truth * (step % 7 + 1))
        assert int(status.item()) == 0


def test_collect_gives_up_on_rows_that_nothing_stores():
    """Bounded wait: rank 1's cells never carry the step, so the collect returns after its time limit with status
    1 + 1, NaN for rank 1's rows and the values of rank 0's; the context stays usable."""
    from crystalformer_b200 import _lib
    world, rows, targets = 2, 4, 1
    one = int(np.float32(1.0).view(np.uint32)) | (1 << 32)  # { 1.0f, step 1 }
    cells = torch.tensor([one] * rows + [0] * rows, dtype=torch.int64, device="cuda")
    index = torch.arange(world * rows, device="cuda")
    out = torch.zeros((world * rows, targets), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _lib.call("cf_peer_gather_collect", cells.data_ptr(), 1, index.data_ptr(), world * rows, targets, rows,
              out.data_ptr(), status.data_ptr(), 0.2, _stream())
    torch.cuda.synchronize()
    assert int(status.item()) == 2
    assert bool((out[:rows] == 1.0).all()) and bool(torch.isnan(out[rows:]).all())
    assert float((out[:rows] + 1).sum().item()) == 2.0 * rows  # the device still answers


@pytest.mark.parametrize("overlap", [False, True])
def test_model_forward_with_a_gather_of_one_rank(golden_model, overlap):
    """world = 1 through the public classes: the pooling + head kernel stores into the (own) gather buffer and the
    collect puts the rows into the order of the unsharded batch; also with the collects on a stream of their own."""
    from test_gpu_model import batch_of, build
    from crystalformer_b200.sharding import PeerGather
    model = build(golden_model).eval()
    batch = batch_of(golden_model)
    B = batch.sizes.shape[0]
    order = list(np.random.default_rng(0).permutation(B))  # local crystal c is crystal order[c] of the "unsharded" batch
    gather = PeerGather([[int(g) for g in order]], model.mlp[-1].out_features, torch.device("cuda"), overlap=overlap)
    with torch.no_grad():
        y = model(batch)
        for _ in range(7):  # several steps: slots are reused
            y_all = model(batch, gather=gather)
            gather.wait_ready()
            gather.check()
            expect = torch.empty_like(y)
            expect[torch.as_tensor(order).cuda()] = y
            assert torch.equal(y_all, expect)
    gather.close()


@pytest.mark.parametrize("overlap,streams", [(False, 1), (True, 3)])
def test_predictor_with_a_gather_of_one_rank(golden_model, overlap, streams):
    """Host batches through PipelinedPredictor with a peer gather (world = 1): each submit is one library call that
    copies the inputs, runs the forward, collects the gathered rows and copies them and the status word to the host."""
    import types
    from test_gpu_model import build
    from crystalformer_b200.serving import PipelinedPredictor
    from crystalformer_b200.sharding import PeerGather
    from crystalformer_b200.synthetic import make_crystals, uniform_atoms
    model = build(golden_model).eval()
    B = 9
    batches = [make_crystals(70 + s, B, uniform_atoms(1, 8), length_range=(3.0, 10.0)) for s in range(11)]
    host = [types.SimpleNamespace(x=torch.from_numpy(b.x).pin_memory(), pos=torch.from_numpy(b.pos).pin_memory(),
                                  trans_vec=torch.from_numpy(b.trans_vec).pin_memory(),
                                  sizes=torch.from_numpy(b.sizes).pin_memory()) for b in batches]
    order = [int(g) for g in np.random.default_rng(1).permutation(B)]
    with torch.no_grad():
        direct = [model(types.SimpleNamespace(**{k: v.cuda() for k, v in vars(h).items()})).cpu() for h in host]
    gather = PeerGather([order], model.mlp[-1].out_features, torch.device("cuda"), slots=8, overlap=overlap)
    runner = PipelinedPredictor(model, depth=4, streams=streams, gather=gather)
    got, tickets = [], []
    for h in host:
        if runner.pending() == runner.depth:
            got.append(runner.result(tickets.pop(0)).clone())
        tickets.append(runner.submit(h))
    while tickets:
        got.append(runner.result(tickets.pop(0)).clone())
    assert runner._native[0] is not None  # the one-call path was taken
    for y_all, y in zip(got, direct):
        expect = torch.empty_like(y)
        expect[torch.as_tensor(order)] = y
        assert torch.equal(y_all, expect)
    gather.check()
    gather.close()


_CHILD = r"""
import json, os, sys, types
sys.path.insert(0, os.environ["CF_REPO"])
sys.path.insert(0, os.path.join(os.environ["CF_REPO"], "tests"))
import numpy as np, torch, torch.distributed as dist
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
from crystalformer_b200.sharding import PeerGather, gather_outputs, lpt_assign
from crystalformer_b200.synthetic import make_crystals, uniform_atoms
from crystalformer_b200.model import Latticeformer, default_params
torch.manual_seed(0)
model = Latticeformer(default_params(num_layers=2, value_pe_dist_real=64)).to(dev).eval()
cb = make_crystals(3, 24 * world, uniform_atoms(1, 12))
shards = lpt_assign(cb.sizes, world)
mine = cb.select(shards[rank])
t = lambda a: torch.from_numpy(a).to(dev)
batch = types.SimpleNamespace(x=t(mine.x), pos=t(mine.pos), trans_vec=t(mine.trans_vec), sizes=t(mine.sizes))
# one training-mode forward fixes the Gaussian-width statistics (rank 0's, sent to all), so that the model runs its
# one-call inference path and is the same on every rank
model.train()
with torch.no_grad():
    model(batch)
model.eval()
for name, buf in model.named_buffers():
    if name.endswith("gauss_scale"):
        dist.broadcast(buf, src=0)
ok = True
for overlap in (False, True):
    gather = PeerGather(shards, model.mlp[-1].out_features, dev, timeout_s=10.0, slots=8 if overlap else 4, overlap=overlap)
    with torch.no_grad():
        y = model(batch)
        want = gather_outputs(y, shards)
        outs = []
        for step in range(12 if overlap else 4):
            got = model(batch, gather=gather)
            if overlap:
                outs.append(got)  # compared after the loop: the rank runs ahead of its collects
            else:
                ok = ok and bool(torch.equal(got, want))
            if step == 1:  # outputs that exist already
                gather.store(y)
                got2 = gather.collect()
                gather.wait_ready()
                ok = ok and bool(torch.equal(got2, want))
        gather.wait_ready()
        torch.cuda.synchronize()
        ok = ok and all(bool(torch.equal(o, want)) for o in outs)
    gather.check()
    gather.close()
# host batches through the pipelined predictor: one library call per batch does copies, forward, collect and read-back
from crystalformer_b200.serving import PipelinedPredictor
pin = lambda a: torch.from_numpy(a).pin_memory()
hostb = types.SimpleNamespace(x=pin(mine.x), pos=pin(mine.pos), trans_vec=pin(mine.trans_vec), sizes=pin(mine.sizes))
gather = PeerGather(shards, model.mlp[-1].out_features, dev, timeout_s=10.0, slots=8, overlap=True)
runner = PipelinedPredictor(model, depth=4, streams=3, gather=gather, dense_tile_rows=0)
tickets, outs = [], []
for step in range(13):
    if runner.pending() == runner.depth:
        outs.append(runner.result(tickets.pop(0)).clone())
    tickets.append(runner.submit(hostb))
while tickets:
    outs.append(runner.result(tickets.pop(0)).clone())
one_call = runner._native[0] is not None
served = len(outs) == 13 and all(bool(torch.equal(o, want.cpu())) for o in outs)
if not served:
    print("rank", rank, "served outputs differ:", [float((o - want.cpu()).abs().max()) for o in outs], file=sys.stderr)
gather.check()
gather.close()
flag = torch.tensor([int(ok), int(one_call), int(served)], device=dev)
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0:
    print(json.dumps(dict(zip(("model", "one_call", "served"), flag.tolist()))))
dist.destroy_process_group()
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_on_two_gpus(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    env = dict(os.environ, CF_REPO=REPO, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29641", str(script)]
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    assert json.loads(proc.stdout.strip().splitlines()[-1]) == {"model": 1, "one_call": 1, "served": 1}
