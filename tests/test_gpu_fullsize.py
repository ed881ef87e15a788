"""Parity properties at the full sizes of the benchmark configurations, where the CPU oracle would take too long:
size-independent invariants of the path, plus spot checks of randomly drawn rows against the float64 oracle."""
import numpy as np
import pytest
import torch

import oracle
from conftest import rel_err
from crystalformer_b200.synthetic import all_pairs_edges, make_config, microbench_edges

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


def prepared(ops, cb):
    sizes = dev(cb.sizes)
    atom_start, edge_start = ops.crystal_offsets(sizes)
    return ops.batch_prepare(dev(cb.pos), dev(cb.trans_vec), sizes, atom_start, edge_start, cb.num_atoms, cb.num_edges)


def random_inputs(N, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((N, H, D), device="cuda", generator=g) * 0.3
    k, v = (torch.randn((N, H, D), device="cuda", generator=g) for _ in range(2))
    a = -0.5 / (1.4 * (0.55 + 0.9 * torch.rand((N, H), device="cuda", generator=g))) ** 2
    W = torch.randn((H, D, K), device="cuda", generator=g) * 0.1
    return q, k, v, a, W


@pytest.mark.parametrize("cfg", ["cfg0", "cfg3"])
def test_edge_list_of_full_batches_is_bit_exact(ops, cfg):
    cb = make_config(cfg)
    prep = prepared(ops, cb)
    assert np.array_equal(prep["edges"].cpu().numpy(), all_pairs_edges(cb.sizes))
    assert prep["edges"].shape[1] == int((cb.sizes ** 2).sum())


@pytest.mark.parametrize("cfg", ["cfg0", "cfg3", "cfg4"])
def test_fused_attention_invariants_at_full_size(ops, cfg):
    cb = make_config(cfg, num_crystals=16 if cfg == "cfg4" else None)
    prep = prepared(ops, cb)
    N, E = cb.num_atoms, cb.num_edges
    q, k, v, a, W = random_inputs(N, 7)
    tv = dev(cb.trans_vec)
    args = (q, k, v, a, prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"], prep["row_start"],
            int(cb.sizes.max()), K, DIST_MAX, WSCALE)
    out, logit, lse, psi_row = ops.infinite_attn_fwd(*args, W, -3.5, 2, 2, want_psi_row=True)
    assert torch.isfinite(out).all() and torch.isfinite(logit).all()
    # (1) attention weights of every (atom, head) sum to one
    p = torch.exp(logit - lse[prep["edges"][0]])
    row_sum = torch.zeros((N, H), device="cuda").index_add_(0, prep["edges"][0], p)
    assert float((row_sum - 1).abs().max()) < 1e-5
    # (2) the radial-basis histogram is non-negative and its mass is bounded by the attention mass
    assert float(psi_row.min()) >= 0.0
    # (3) linearity in the projection: out(W1 + W2) - out(0) = (out(W1) - out(0)) + (out(W2) - out(0))
    zero = torch.zeros_like(W)
    o0 = ops.infinite_attn_fwd(*args, zero, -3.5, 2, 2)[0]
    W2 = torch.flip(W, dims=(2,)) * 0.5
    o1, o2 = ops.infinite_attn_fwd(*args, W, -3.5, 2, 2)[0], ops.infinite_attn_fwd(*args, W2, -3.5, 2, 2)[0]
    o12 = ops.infinite_attn_fwd(*args, W + W2, -3.5, 2, 2)[0]
    assert rel_err((o12 - o0).cpu().numpy(), ((o1 - o0) + (o2 - o0)).cpu().numpy()) < 1e-5
    # (4) the fused operator equals the operator split (phi, W psi per edge, then edge-indexed attention)
    z, psiW = ops.lattice_sum_fwd(a, prep["pos_ij"], tv, prep["batch"], prep["edges"], K, DIST_MAX, WSCALE, W=W,
                                  rvlen=prep["rvlen"], cutoff_radius=-3.5)
    _, out_split = ops.fused_attn_fwd(q, k, v, z, psiW, prep["edges"], prep["row_start"])
    assert rel_err(out.cpu().numpy(), out_split.cpu().numpy()) < TOL
    # (5) spot check: every row of a few crystals against the float64 oracle
    rng = np.random.default_rng(1)
    pick = rng.choice(cb.num_crystals, size=min(3, cb.num_crystals), replace=False)
    pick = [int(c) for c in pick if cb.sizes[c] <= 64][:2] or [int(np.argmin(cb.sizes))]
    sub = cb.select(pick)
    starts = np.concatenate([[0], np.cumsum(cb.sizes)])
    rows = np.concatenate([np.arange(starts[c], starts[c + 1]) for c in pick])
    e_sub = oracle.edge_index(sub.sizes)
    pij, _, _, rvl = oracle.geometry(sub.pos, sub.trans_vec, e_sub)
    qn, kn, vn, an = (t[rows].cpu().numpy() for t in (q, k, v, a))
    zr, pw = oracle.lattice_sum_fwd(an, pij, sub.trans_vec, sub.batch, e_sub, K, DIST_MAX, WSCALE, W=W.cpu().numpy()[None],
                                    rvlen=rvl, cutoff_radius=-3.5, precision="f64")
    _, ref = oracle.fused_attn_fwd(qn, kn, vn, zr, pw, e_sub, precision="f64")
    assert rel_err(out[rows].cpu().numpy(), ref) < TOL


def test_microbenchmark_kernel_properties_at_full_size(ops):
    """2,000,000 (i,j,head) items: phi agrees between the K = 0 and K = 64 launches bit for bit; psi is a
    non-negative histogram whose mass is at most 1 (weights sum to one, every basis value is at most one); a sample of
    edges matches the float64 oracle."""
    cb, edges, pos_ij, a = microbench_edges()
    _, _, _, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges[:, :1])
    A, P, T, B, Ed, RV = dev(a), dev(pos_ij), dev(cb.trans_vec), dev(cb.batch), dev(edges), dev(rvlen)
    kw = dict(rvlen=RV, cutoff_radius=-3.5, lattice_range=2, minimum_range=2, a_per_edge=True)
    z64, psi = ops.lattice_sum_fwd(A, P, T, B, Ed, K, DIST_MAX, WSCALE, **kw)
    z0, _ = ops.lattice_sum_fwd(A, P, T, B, Ed, 0, DIST_MAX, WSCALE, **kw)
    assert torch.equal(z64, z0)
    assert float(psi.min()) >= 0.0
    # neighbouring bins overlap (width = spacing), so the mass of a unit weight is at most sum_k exp(-(k-x)^2/2) < 2.51
    assert float(psi.sum(dim=2).max()) < 2.51
    rng = np.random.default_rng(2)
    pick = np.sort(rng.choice(edges.shape[1], size=300, replace=False))
    zr, pr = oracle.lattice_sum_fwd(a[pick], pos_ij[pick], cb.trans_vec, cb.batch, edges[:, pick], K, DIST_MAX, WSCALE,
                                    rvlen=rvlen, cutoff_radius=-3.5, a_per_edge=True, precision="f64")
    assert rel_err(z64[pick].cpu().numpy(), zr) < TOL and rel_err(psi[pick].cpu().numpy(), pr) < TOL
    box = ops.lattice_box(A, B, Ed, RV, -3.5, 2, 2, a_per_edge=True).cpu().numpy()[pick]
    _, _, ref_box = oracle.lattice_sum_fwd(a[pick], pos_ij[pick], cb.trans_vec, cb.batch, edges[:, pick], 0, DIST_MAX,
                                           WSCALE, rvlen=rvlen, cutoff_radius=-3.5, a_per_edge=True, return_box=True)
    assert np.array_equal(box, ref_box)


def test_training_step_at_cfg3_size_is_finite_and_repeatable(ops):
    """Forward + backward of the fused operator on the 256-crystal training batch: finite, run-to-run identical, and
    the gradient of a agrees with the operator-split backward."""
    cb = make_config("cfg3")
    prep = prepared(ops, cb)
    N = cb.num_atoms
    q, k, v, a, W = random_inputs(N, 9)
    go = torch.randn((N, H, D), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))
    tv = dev(cb.trans_vec)
    args = (q, k, v, a, prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"], prep["row_start"],
            int(cb.sizes.max()), K, DIST_MAX, WSCALE, W, -3.5, 2, 2)
    out, logit, lse, psi_row = ops.infinite_attn_fwd(*args, want_psi_row=True)
    g1 = ops.infinite_attn_bwd(*args, logit, lse, out, go)
    g2 = ops.infinite_attn_bwd(*args, logit, lse, out, go)
    assert all(torch.isfinite(t).all() for t in g1)
    assert all(torch.equal(x, y) for x, y in zip(g1, g2))
    # operator split: attention backward gives the gradients of phi and W psi, the lattice-sum backward turns them into ga
    z, psiW = ops.lattice_sum_fwd(a, prep["pos_ij"], tv, prep["batch"], prep["edges"], K, DIST_MAX, WSCALE, W=W,
                                  rvlen=prep["rvlen"], cutoff_radius=-3.5)
    prob, out_split = ops.fused_attn_fwd(q, k, v, z, psiW, prep["edges"], prep["row_start"])
    gq, gk, gv, gphi, gpsiW = ops.fused_attn_bwd(q, k, v, psiW, prep["edges"], prep["row_start"], prob, out_split, go)
    ga, gW = ops.lattice_sum_bwd(a, prep["pos_ij"], tv, prep["batch"], prep["edges"], prep["row_start"], z, gphi, gpsiW,
                                 K, DIST_MAX, WSCALE, W=W, rvlen=prep["rvlen"], cutoff_radius=-3.5)
    assert rel_err(g1[3].cpu().numpy(), ga.cpu().numpy()) < TOL
    assert rel_err(g1[0].cpu().numpy(), gq.cpu().numpy()) < TOL
    assert rel_err(g1[1].cpu().numpy(), gk.cpu().numpy()) < TOL
    assert rel_err(g1[2].cpu().numpy(), gv.cpu().numpy()) < TOL
    assert rel_err(torch.einsum("nhd,nhk->hdk", go, psi_row).cpu().numpy(), gW.cpu().numpy()) < TOL
