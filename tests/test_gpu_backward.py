"""GPU parity of the backward kernels: per-edge lattice-sum backward and the fused attention backward, against the
float64 oracle and the gradients autograd produced through the reference's PyTorch implementation (golden vectors)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import rel_err
from crystalformer_b200.synthetic import make_crystals, uniform_atoms

pytestmark = pytest.mark.gpu

H, D, K = 8, 16, 64
DIST_MAX, WSCALE = 14.0, 1.0
TOL = 1e-4


@pytest.fixture(scope="module")
def ops():
    from crystalformer_b200 import ops as _ops
    return _ops


def dev(x):
    return None if x is None else torch.as_tensor(np.ascontiguousarray(x)).cuda()


def random_case(seed, crystals, nmax, lengths=(2.5, 8.0), nmin=1):
    cb = make_crystals(seed, crystals, uniform_atoms(nmin, nmax), length_range=lengths)
    edges = oracle.edge_index(cb.sizes)
    pos_ij, _, _, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    rng = np.random.default_rng(seed)
    N = cb.num_atoms
    sig = 1.4 * (0.6 + 0.9 * rng.random((N, H)))
    a = (-0.5 / sig ** 2).astype(np.float32)
    W = (rng.standard_normal((1, H, D, K)) * 0.1).astype(np.float32)
    return cb, edges, pos_ij, rvlen, a, W, rng


def test_lattice_sum_backward_against_golden(ops, golden_ops):
    g = golden_ops
    edges = g["f32_edges"]
    N = g["in_a"].shape[0]
    pos_ij, _, _, _ = oracle.geometry(g["in_pos"], g["in_trans"], edges)
    row_start = dev(oracle.row_starts(edges, N))
    base = (dev(g["in_a"]), dev(pos_ij), dev(g["in_trans"]), dev(g["in_batch"]), dev(edges))
    z, _ = ops.lattice_sum_fwd(*base, K, DIST_MAX, WSCALE, W=dev(g["in_W"]))
    ga, gW = ops.lattice_sum_bwd(*base, row_start, z, dev(g["f32_g_phi"]), dev(g["f32_g_psiW"]), K, DIST_MAX, WSCALE,
                                 W=dev(g["in_W"]))
    assert rel_err(ga.cpu().numpy(), g["f64_g_a"]) < TOL
    assert gW.shape == g["in_W"].shape and rel_err(gW.cpu().numpy(), g["f64_g_W"]) < TOL


@pytest.mark.parametrize("cutoff,minimum,Kbins,proj", [(-3.5, 2, 64, True), (-3.5, 0, 64, False), (7.5, 2, 64, True),
                                                       (0.0, 2, 64, False), (-3.5, 2, 0, False)])
def test_lattice_sum_backward_against_oracle(ops, cutoff, minimum, Kbins, proj):
    cb, edges, pos_ij, rvlen, a, W, rng = random_case(71, 8, 7)
    N, E = cb.num_atoms, edges.shape[1]
    Wn = W if proj else None
    common = dict(rvlen=rvlen, cutoff_radius=cutoff, lattice_range=2, minimum_range=minimum)
    z64, v64 = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, Kbins, DIST_MAX, WSCALE, W=Wn,
                                      precision="f64", **common)
    gz = rng.standard_normal((E, H)).astype(np.float32)
    gv = rng.standard_normal(v64.shape).astype(np.float32) if Kbins else None
    ga64, gW64 = oracle.lattice_sum_bwd(a, pos_ij, cb.trans_vec, cb.batch, edges, z64, gz, gv, Kbins, DIST_MAX, WSCALE,
                                        W=Wn, precision="f64", **common)
    base = (dev(a), dev(pos_ij), dev(cb.trans_vec), dev(cb.batch), dev(edges))
    dcommon = dict(rvlen=dev(rvlen), cutoff_radius=cutoff, lattice_range=2, minimum_range=minimum)
    z, _ = ops.lattice_sum_fwd(*base, Kbins, DIST_MAX, WSCALE, W=dev(Wn), **dcommon)
    row_start = dev(oracle.row_starts(edges, N))
    ga, gW = ops.lattice_sum_bwd(*base, row_start, z, dev(gz), dev(gv), Kbins, DIST_MAX, WSCALE, W=dev(Wn), **dcommon)
    assert rel_err(ga.cpu().numpy(), ga64) < TOL
    if proj:
        assert rel_err(gW.cpu().numpy(), gW64) < TOL
    again, _ = ops.lattice_sum_bwd(*base, row_start, z, dev(gz), dev(gv), Kbins, DIST_MAX, WSCALE, W=dev(Wn), **dcommon)
    assert torch.equal(ga, again)


def fused_grads(ops, cb, edges, pos_ij, rvlen, q, k, v, a, W, go, Kbins, cutoff, minimum):
    N = cb.num_atoms
    row_start = dev(oracle.row_starts(edges, N))
    W3 = None if W is None else dev(W[0])
    args = (dev(q), dev(k), dev(v), dev(a), dev(pos_ij), dev(cb.trans_vec), dev(rvlen), dev(cb.batch), dev(edges),
            row_start, int(cb.sizes.max()), Kbins, DIST_MAX, WSCALE, W3, cutoff, 2, minimum)
    out, logit, lse, psi_row = ops.infinite_attn_fwd(*args, want_psi_row=True)
    gq, gk, gv, ga = ops.infinite_attn_bwd(*args, logit, lse, out, dev(go))
    gW = torch.einsum("nhd,nhk->hdk", dev(go), psi_row) if Kbins else None
    return out, gq, gk, gv, ga, gW


def test_fused_backward_against_golden(ops, golden_ops):
    g = golden_ops
    cb = make_crystals(11, 7, uniform_atoms(1, 6), length_range=(3.0, 9.0))
    edges = g["f32_edges"]
    pos_ij, _, _, rvlen = oracle.geometry(g["in_pos"], g["in_trans"], edges)
    qs = g["in_q"] / np.float32(np.sqrt(D))
    out, gq, gk, gv, ga, gW = fused_grads(ops, cb, edges, pos_ij, rvlen, qs, g["in_k"], g["in_v"], g["in_a"], g["in_W"],
                                          g["in_go"], K, 0.0, 2)
    assert rel_err(out.cpu().numpy(), g["f64_out"]) < TOL
    assert rel_err(gq.cpu().numpy() / np.sqrt(D), g["f64_g_q"]) < TOL
    assert rel_err(gk.cpu().numpy(), g["f64_g_k"]) < TOL
    assert rel_err(gv.cpu().numpy(), g["f64_g_v"]) < TOL
    assert rel_err(ga.cpu().numpy(), g["f64_g_a"]) < TOL
    assert rel_err(gW.cpu().numpy(), g["f64_g_W"][0]) < TOL


@pytest.mark.parametrize("cutoff,minimum,nmax,Kbins", [(-3.5, 2, 7, 64), (-3.5, 0, 7, 64), (7.5, 2, 5, 64),
                                                       (0.0, 2, 40, 64), (-3.5, 2, 7, 0)])
def test_fused_backward_against_oracle_chain(ops, cutoff, minimum, nmax, Kbins):
    cb, edges, pos_ij, rvlen, a, W, rng = random_case(72, 8, nmax, nmin=max(1, nmax // 3))
    N, E = cb.num_atoms, edges.shape[1]
    q = (rng.standard_normal((N, H, D)) * 0.5).astype(np.float32)
    k, v, go = (rng.standard_normal((N, H, D)).astype(np.float32) for _ in range(3))
    Wn = W if Kbins else None
    common = dict(rvlen=rvlen, cutoff_radius=cutoff, lattice_range=2, minimum_range=minimum, precision="f64")
    z, psiW = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, Kbins, DIST_MAX, WSCALE, W=Wn, **common)
    prob, ref_out = oracle.fused_attn_fwd(q, k, v, z, psiW, edges, precision="f64")
    rq, rk, rv, r_phi, r_psiW = oracle.fused_attn_bwd(q, k, v, psiW, edges, prob, ref_out, go, precision="f64")
    ra, rW = oracle.lattice_sum_bwd(a, pos_ij, cb.trans_vec, cb.batch, edges, z, r_phi, r_psiW, Kbins, DIST_MAX, WSCALE,
                                    W=Wn, **common)
    out, gq, gk, gv, ga, gW = fused_grads(ops, cb, edges, pos_ij, rvlen, q, k, v, a, Wn, go, Kbins, cutoff, minimum)
    assert rel_err(out.cpu().numpy(), ref_out) < TOL
    assert rel_err(gq.cpu().numpy(), rq) < TOL and rel_err(gk.cpu().numpy(), rk) < TOL
    assert rel_err(gv.cpu().numpy(), rv) < TOL and rel_err(ga.cpu().numpy(), ra) < TOL
    if Kbins:
        assert rel_err(gW.cpu().numpy(), rW[0]) < TOL
    again = fused_grads(ops, cb, edges, pos_ij, rvlen, q, k, v, a, Wn, go, Kbins, cutoff, minimum)
    assert torch.equal(ga, again[4]) and torch.equal(gq, again[1]) and torch.equal(gk, again[2])
