"""Model-level parity on the GPU: the drop-in attention module, encoder and model shell against outputs and
gradients of the reference's own PyTorch model (tests/golden/golden_model.npz, made by tests/golden/make_golden.py)."""
import json
import types

import numpy as np
import pytest
import torch

from conftest import rel_err
from crystalformer_b200.synthetic import make_crystals, uniform_atoms

pytestmark = pytest.mark.gpu
TOL = 1e-4


def build(golden_model, fused=True):
    from crystalformer_b200.model import Latticeformer
    P = json.loads(bytes(golden_model["in_params_json"]).decode())
    model = Latticeformer(types.SimpleNamespace(**P))
    state = {k[len("state:"):]: torch.tensor(v) for k, v in golden_model.items() if k.startswith("state:")}
    model.load_state_dict(state)
    for layer in model.encoder.layers:
        layer.self_attn.fused = fused
    return model.cuda()


def batch_of(g):
    t = lambda x: torch.as_tensor(x).cuda()
    return types.SimpleNamespace(x=t(g["in_x"]), pos=t(g["in_pos"]), batch=t(g["in_batch"]), trans_vec=t(g["in_trans"]),
                                 sizes=t(g["in_sizes"]))


@pytest.mark.parametrize("fused", [True, False])
def test_forward_matches_reference_model(golden_model, fused):
    """The golden run used the fixed (2R+1)^3 box of the PyTorch path; with the default adaptive rule and the
    minimum box of the same size the kernels enumerate at least those translations, so the outputs agree to the
    tolerance unless a cell has a d-spacing below 2.46 Angstrom; the golden crystals have none."""
    model = build(golden_model, fused).eval()
    with torch.no_grad():
        y = model(batch_of(golden_model))
    assert rel_err(y.cpu().numpy(), golden_model["y_f64"]) < TOL
    assert rel_err(y.cpu().numpy(), golden_model["y_f32"]) < TOL


@pytest.mark.parametrize("fused", [True, False])
def test_training_step_gradients_match_reference_model(golden_model, fused):
    model = build(golden_model, fused).train()
    y = model(batch_of(golden_model))
    loss = (y - torch.as_tensor(golden_model["in_targets"]).cuda()).abs().mean()
    loss.backward()
    assert rel_err(loss.item(), golden_model["loss_f64"]) < TOL
    grads = dict(model.named_parameters())
    checked = 0
    for key, ref in golden_model.items():
        if key.startswith("grad_f64:"):
            name = key[len("grad_f64:"):]
            got = grads[name].grad
            assert got is not None, name
            assert rel_err(got.cpu().numpy(), ref) < 2e-4, name  # tiny-norm gradients at init; float64 arbiter
            checked += 1
    assert checked >= 8


def test_one_call_encoder_forward_equals_the_operator_by_operator_path(golden_model):
    """Inference takes the single-call path (cf_encoder_forward); it must agree with the torch-operator path that
    training uses, and with the reference's output."""
    model = build(golden_model).eval()
    model.native = False  # keep the model shell in torch so that the encoder-level call is the one exercised
    data = batch_of(golden_model)
    calls = []
    enc = model.encoder
    original = enc._forward_native
    enc._forward_native = lambda *a, **k: (calls.append(1), original(*a, **k))[1]
    with torch.no_grad():
        y_native = model(data)
        enc.native = False
        y_ops = model(data)
    assert len(calls) == 1
    assert rel_err(y_native.cpu().numpy(), y_ops.cpu().numpy()) < 1e-5
    assert rel_err(y_native.cpu().numpy(), golden_model["y_f64"]) < TOL
    enc.native = True
    y_grad = model(data)  # gradients enabled: must not take the inference path
    assert len(calls) == 1 and y_grad.requires_grad


def test_one_call_model_forward_equals_the_torch_shell(golden_model):
    """cf_model_forward (embedding, geometry, encoder, pooling and head in one library call) against the same model
    evaluated through torch modules around the encoder, with and without host-side counts."""
    model = build(golden_model).eval()
    data = batch_of(golden_model)
    calls = []
    original = model._forward_native
    model._forward_native = lambda *a, **k: (calls.append(1), original(*a, **k))[1]
    sizes = golden_model["in_sizes"]
    counts = (int(sizes.sum()), int((sizes ** 2).sum()), int(sizes.max()))
    with torch.no_grad():
        y_native = model(data)
        y_counts = model(data, counts=counts)
        model.native = False
        y_shell = model(data)
    assert len(calls) == 2
    assert torch.equal(y_native, y_counts)
    assert rel_err(y_native.cpu().numpy(), y_shell.cpu().numpy()) < 1e-5
    assert rel_err(y_native.cpu().numpy(), golden_model["y_f64"]) < TOL
    model.native = True
    assert model(data).requires_grad and len(calls) == 2  # gradients enabled: the autograd path


def test_one_call_model_forward_on_more_than_1024_crystals(golden_model):
    """Above 1024 crystals the offsets come from their own launch instead of the geometry launch: same outputs as the
    torch shell, and the first crystals' outputs equal those of a batch that holds only them (below the limit)."""
    from crystalformer_b200.model import Latticeformer, default_params
    torch.manual_seed(5)
    model = Latticeformer(default_params(num_layers=2)).cuda()
    cb = make_crystals(77, 1100, uniform_atoms(1, 3), length_range=(4.0, 9.0))
    t = lambda x: torch.as_tensor(x).cuda()
    of = lambda c: types.SimpleNamespace(x=t(c.x), pos=t(c.pos), batch=t(c.batch), trans_vec=t(c.trans_vec), sizes=t(c.sizes))
    data, head = of(cb), of(cb.select(range(300)))
    model.train()
    with torch.no_grad():
        model(head)  # fixes gauss_scale
    model.eval()
    with torch.no_grad():
        y = model(data)
        y_head = model(head)
        model.native = False
        y_shell = model(data)
    assert rel_err(y.cpu().numpy(), y_shell.cpu().numpy()) < 1e-5
    assert rel_err(y[:300].cpu().numpy(), y_head.cpu().numpy()) < 1e-5


@pytest.mark.parametrize("atoms", [(1, 7), (20, 45)])
def test_fused_dense_block_equals_the_sgemm_path(golden_model, atoms):
    """The tensor-core dense block (TF32 product + bfloat16 correction product) against the same forward with cuBLAS SGEMMs: fp32-level
    agreement, on a batch smaller than one 16-row tile wave and on one with several tiles per block row range."""
    from crystalformer_b200.model import Latticeformer, default_params
    torch.manual_seed(3)
    model = Latticeformer(default_params(num_layers=3)).cuda()
    cb = make_crystals(60, 9, uniform_atoms(*atoms), length_range=(4.0, 10.0))
    t = lambda x: torch.as_tensor(x).cuda()
    data = types.SimpleNamespace(x=t(cb.x), pos=t(cb.pos), batch=t(cb.batch), trans_vec=t(cb.trans_vec), sizes=t(cb.sizes))
    model.train()
    with torch.no_grad():
        model(data)  # stores gauss_scale
    model.eval()
    with torch.no_grad():
        model.encoder.dense_fused = True
        y_fused = model(data)
        model.encoder.dense_fused = False
        y_sgemm = model(data)
        model.native = False
        model.encoder.native = False
        y_torch = model(data)
    assert rel_err(y_fused.cpu().numpy(), y_sgemm.cpu().numpy()) < 1e-5
    assert rel_err(y_fused.cpu().numpy(), y_torch.cpu().numpy()) < 1e-5


def test_state_dict_keys_are_the_reference_keys(golden_model):
    model = build(golden_model)
    ref_keys = sorted(k[len("state:"):] for k in golden_model if k.startswith("state:"))
    assert sorted(model.state_dict().keys()) == ref_keys


def test_sharded_batches_give_identical_outputs(golden_model):
    """Crystals are independent: evaluating them in two groups gives the same per-crystal outputs (the reference
    prints the same check as `parallel mismatch`, models/latticeformer.py:288-289).  The dense projections run in
    cuBLAS, whose tiling depends on the number of atoms, so the comparison is to 1e-5 rather than bitwise."""
    model = build(golden_model).eval()
    cb = make_crystals(12, 6, uniform_atoms(1, 7), length_range=(3.0, 10.0))
    t = lambda x: torch.as_tensor(x).cuda()
    to_data = lambda b: types.SimpleNamespace(x=t(b.x), pos=t(b.pos), batch=t(b.batch), trans_vec=t(b.trans_vec), sizes=t(b.sizes))
    with torch.no_grad():
        full = model(to_data(cb))
        a, b = model(to_data(cb.select([4, 0, 2]))), model(to_data(cb.select([1, 5, 3])))
    assert rel_err(a.cpu().numpy(), full[[4, 0, 2]].cpu().numpy()) < 1e-5
    assert rel_err(b.cpu().numpy(), full[[1, 5, 3]].cpu().numpy()) < 1e-5


@pytest.mark.parametrize("depth,streams,count,one_call", [(2, 1, 5, True), (4, 3, 14, True), (3, 2, 7, False)])
def test_pipelined_predictor_equals_direct_calls(golden_model, depth, streams, count, one_call):
    """Batches streamed through PipelinedPredictor (copies on a second stream, several batches in flight - on one compute
    stream or alternating between three -, early preparation beside the previous batches, results in pinned ring
    buffers) give exactly what model(batch) gives, in submission order."""
    from crystalformer_b200.serving import PipelinedPredictor
    model = build(golden_model).eval()
    batches = [make_crystals(40 + s, 5 + (3 * s) % 7, uniform_atoms(1, 8), length_range=(3.0, 10.0)) for s in range(count)]
    host = [types.SimpleNamespace(x=torch.from_numpy(b.x).pin_memory(), pos=torch.from_numpy(b.pos).pin_memory(),
                                  trans_vec=torch.from_numpy(b.trans_vec).pin_memory(),
                                  sizes=torch.from_numpy(b.sizes).pin_memory()) for b in batches]
    with torch.no_grad():
        direct = [model(types.SimpleNamespace(**{k: v.cuda() for k, v in vars(h).items()})).cpu() for h in host]
    # one_call: each submit is one call of cf_serve_submit (copies, forward and events issued by the library); otherwise
    # the same steps are issued through torch (the path taken with a post-processing callable or a peer gather)
    runner = PipelinedPredictor(model, depth=depth, streams=streams, post=None if one_call else (lambda y: y))
    got, tickets = [], []
    for h in host:
        if runner.pending() == runner.depth:
            got.append(runner.result(tickets.pop(0)).clone())
        tickets.append(runner.submit(h))
    while tickets:
        got.append(runner.result(tickets.pop(0)).clone())
    assert len(got) == len(direct)
    for y, ref in zip(got, direct):
        assert torch.equal(y, ref)
    assert (runner._native[0] is not None) == one_call
    if one_call:  # the same batches with species indices instead of one-hot rows: the same bits
        for h, ref in zip(host[:depth], direct):
            assert bool(((h.x.sum(1) == 1) & (h.x.max(1).values == 1)).all())  # (the synthetic rows are one-hot)
            hz = types.SimpleNamespace(z=h.x.argmax(1).contiguous().pin_memory(), pos=h.pos, trans_vec=h.trans_vec, sizes=h.sizes)
            assert torch.equal(runner.result(runner.submit(hz)), ref)
    with pytest.raises(RuntimeError):
        runner.result(123)
    if one_call:  # a batch larger than the slot's buffers is refused by the library, not written past their end
        from crystalformer_b200 import _lib
        import ctypes
        st, h = runner._native[0], host[0]
        st["c"].max_atoms_total = 1
        with pytest.raises(_lib.CrystalformerB200Error) as e:
            _lib.call("cf_serve_submit", ctypes.byref(runner._plan["desc"]), ctypes.byref(st["c"]), h.x.data_ptr(),
                      h.pos.data_ptr(), h.trans_vec.data_ptr(), h.sizes.data_ptr(), int(h.x.shape[0]), int(h.sizes.shape[0]),
                      int((h.sizes ** 2).sum()), int(h.sizes.max()), 1, None, None)
        assert "exceeds the slot's buffers" in str(e.value)
