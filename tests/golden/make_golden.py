"""Generates the golden vectors under tests/golden/ by running the REFERENCE project's own PyTorch implementation.

Run in a container where the reference tree is mounted (default /root/reference; override with CF_REFERENCE_ROOT):

    python tests/golden/make_golden.py

The reference cannot travel to the GPU machines, so its outputs are committed here as small .npz files together with
this script.  Three files are written (name them on the command line to regenerate only some):

* golden_ops.npz   - operator level: phi, psi, W psi, the edge-indexed attention and all their gradients for a small
                     ragged batch, from LogSumExpXYFunc / AverageGaussiansBySoftmaxXYFunc_ /
                     _scaled_dot_product_attention (models/indexed_lattice_multi_head_attention.py:309,741,140), in
                     float32 and float64.  The PyTorch path enumerates the fixed (2R+1)^3 translation box.
* golden_reci.npz  - the reciprocal-space lattice sum (compute_reci_domain_attn,
                     models/indexed_lattice_multi_head_attention.py:925-950, on the cos_kr / k2 tables of
                     compute_lattice_distances(output_rec=True), models/indexed_latticeformer_encoder.py:140-162) and
                     its autograd gradient, float32 and float64.
* golden_model.npz - model level: a 2-layer Latticeformer (models/latticeformer.py) with random-init weights, its
                     state_dict, inputs, per-crystal outputs and a few parameter gradients of an L1 training step.
"""
import contextlib
import io
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("CF_REFERENCE_ROOT", "/root/reference")
sys.dont_write_bytecode = True
sys.path.insert(0, REF)
sys.path.insert(0, REPO)

from crystalformer_b200.synthetic import make_crystals, uniform_atoms  # noqa: E402

from models.indexed_latticeformer_encoder import compute_lattice_distances  # noqa: E402
from models.indexed_lattice_multi_head_attention import (  # noqa: E402
    AverageGaussiansBySoftmaxXYFunc_, LogSumExpXYFunc, _scaled_dot_product_attention, compute_reci_domain_attn)
from models.latticeformer import Latticeformer  # noqa: E402

H, D, K = 8, 16, 64
DIST_MAX, WSCALE, LATTICE_RANGE = 14.0, 1.0, 2


def ops_case(dtype):
    cb = make_crystals(11, 7, uniform_atoms(1, 6), length_range=(3.0, 9.0))
    # one crystal twice as large as the attention kernel's 64-wide summation block is not needed here; n <= 6
    rng = np.random.default_rng(5)
    N = cb.num_atoms
    sigma = 1.4 * (0.6 + 0.9 * rng.random((N, H)))
    inp = dict(
        sizes=cb.sizes, pos=cb.pos, trans=cb.trans_vec, batch=cb.batch,
        a=(-0.5 / sigma ** 2).astype(np.float32),
        W=(rng.standard_normal((1, H, D, K)) * 0.2).astype(np.float32),
        q=(rng.standard_normal((N, H, D)) * 0.7).astype(np.float32),
        k=rng.standard_normal((N, H, D)).astype(np.float32),
        v=rng.standard_normal((N, H, D)).astype(np.float32),
        go=rng.standard_normal((N, H, D)).astype(np.float32),
    )
    t = {n: torch.tensor(x).to(dtype) if x.dtype.kind == "f" else torch.tensor(x) for n, x in inp.items()}
    dist, _, _, _, _, edges, _ = compute_lattice_distances(t["pos"], t["batch"], t["trans"], t["sizes"], LATTICE_RANGE)
    dist2 = dist * dist
    a = t["a"].clone().requires_grad_(True)
    W = t["W"].clone().requires_grad_(True)
    q = t["q"].clone().requires_grad_(True)
    k = t["k"].clone().requires_grad_(True)
    v = t["v"].clone().requires_grad_(True)
    phi = LogSumExpXYFunc.apply(dist2.unsqueeze(1), a.unsqueeze(2)[edges[0]], -1)
    phi.retain_grad()
    psiW = AverageGaussiansBySoftmaxXYFunc_.apply(DIST_MAX, K, dist2[:, None, :, None], a[:, :, None, None][edges[0]],
                                                  -2, W, WSCALE)
    psiW.retain_grad()
    with torch.no_grad():
        psi = AverageGaussiansBySoftmaxXYFunc_.apply(DIST_MAX, K, dist2[:, None, :, None],
                                                     a[:, :, None, None][edges[0]], -2, None, WSCALE)
    out, prob, _ = _scaled_dot_product_attention(q, k, v, t["batch"], t["batch"], edges, phi, psiW, 0.0, 0)
    (out * t["go"]).sum().backward()
    res = dict(edges=edges, phi=phi, psi=psi, psiW=psiW, out=out, prob=prob, g_phi=phi.grad, g_psiW=psiW.grad,
               g_a=a.grad, g_W=W.grad, g_q=q.grad, g_k=k.grad, g_v=v.grad)
    return inp, {n: x.detach().numpy() for n, x in res.items()}


def reci_case(dtype):
    cb = make_crystals(13, 7, uniform_atoms(1, 6), length_range=(3.0, 9.0))
    rng = np.random.default_rng(6)
    N = cb.num_atoms
    # a = -0.5 s^2 with s in 2.5 .. 4.5 Angstrom: the R = 2 sum has converged for these cells, so it stays positive and
    # well away from its 1e-6 clamp (log and 1/S would otherwise amplify float rounding beyond any fixed tolerance)
    inp = dict(sizes=cb.sizes, pos=cb.pos, trans=cb.trans_vec, batch=cb.batch,
               a=(-0.5 * (2.5 + 2.0 * rng.random((N, H))) ** 2).astype(np.float32))
    t = {n: torch.tensor(x).to(dtype) if x.dtype.kind == "f" else torch.tensor(x) for n, x in inp.items()}
    _, cos_kr, k2, vcell, _, edges, _ = compute_lattice_distances(t["pos"], t["batch"], t["trans"], t["sizes"],
                                                                  LATTICE_RANGE, output_dis=False, output_rec=True)
    a = t["a"].clone().requires_grad_(True)
    phi = compute_reci_domain_attn(a, cos_kr, k2, vcell, edges[0], t["batch"])
    gz = torch.tensor(rng.standard_normal((edges.shape[1], H))).to(dtype)
    (phi * gz).sum().backward()
    inp["gz"] = gz.numpy().astype(np.float32)
    res = dict(edges=edges, phi=phi, g_a=a.grad, vcell=vcell)
    return inp, {n: x.detach().numpy() for n, x in res.items()}


def model_case():
    P = json.load(open(os.path.join(REF, "params/latticeformer/default.json")))
    P.update(num_layers=2, ff_dim=128, embedding_dim=[64])
    cb = make_crystals(12, 6, uniform_atoms(1, 7), length_range=(3.0, 10.0))
    data = types.SimpleNamespace(
        x=torch.tensor(cb.x), pos=torch.tensor(cb.pos), batch=torch.tensor(cb.batch),
        trans_vec=torch.tensor(cb.trans_vec), sizes=torch.tensor(cb.sizes))
    torch.manual_seed(12)
    with contextlib.redirect_stdout(io.StringIO()):
        model = Latticeformer(types.SimpleNamespace(**P))
        model.train()
        model(data)  # the first training-mode forward fixes gauss_scale (…attention.py:1311-1327)
    state = {n: x.detach().clone().numpy() for n, x in model.state_dict().items()}
    targets = torch.tensor(np.random.default_rng(3).standard_normal((cb.num_crystals, 1)).astype(np.float32))
    out = {}
    for tag, dt in (("f32", torch.float32), ("f64", torch.float64)):
        m = model.double() if dt == torch.float64 else model
        d = types.SimpleNamespace(**{n: (x.to(dt) if x.is_floating_point() else x) for n, x in vars(data).items()})
        m.zero_grad()
        y = m(d)
        loss = (y - targets.to(dt)).abs().mean()
        loss.backward()
        out[f"y_{tag}"] = y.detach().numpy()
        out[f"loss_{tag}"] = loss.detach().numpy()
        for n, p in m.named_parameters():
            if p.grad is not None and (".0.self_attn." in n or n == "input_embeddings.weight"):
                out[f"grad_{tag}:{n}"] = p.grad.detach().numpy()
    inp = dict(sizes=cb.sizes, pos=cb.pos, trans=cb.trans_vec, batch=cb.batch, x=cb.x, targets=targets.numpy(),
               params_json=np.frombuffer(json.dumps(P).encode(), dtype=np.uint8))
    return inp, state, out


def main():
    which = set(sys.argv[1:]) or {"golden_ops.npz", "golden_reci.npz", "golden_model.npz"}
    if "golden_ops.npz" in which:
        inp, r32 = ops_case(torch.float32)
        _, r64 = ops_case(torch.float64)
        blob = {f"in_{n}": x for n, x in inp.items()}
        blob.update({f"f32_{n}": x for n, x in r32.items()})
        blob.update({f"f64_{n}": x for n, x in r64.items()})
        np.savez_compressed(os.path.join(HERE, "golden_ops.npz"), **blob)
    if "golden_reci.npz" in which:
        inp, r32 = reci_case(torch.float32)
        _, r64 = reci_case(torch.float64)
        blob = {f"in_{n}": x for n, x in inp.items()}
        blob.update({f"f32_{n}": x for n, x in r32.items()})
        blob.update({f"f64_{n}": x for n, x in r64.items()})
        np.savez_compressed(os.path.join(HERE, "golden_reci.npz"), **blob)
    if "golden_model.npz" in which:
        inp, state, out = model_case()
        blob = {f"in_{n}": x for n, x in inp.items()}
        blob.update({f"state:{n}": x for n, x in state.items()})
        blob.update(out)
        np.savez_compressed(os.path.join(HERE, "golden_model.npz"), **blob)
    for f in sorted(which):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
