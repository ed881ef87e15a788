"""GPU parity of the fully fused attention (phi and psi recomputed inside the kernels) against the operator-level
oracle chain lattice sum -> edge-indexed attention, and against the reference-made golden vectors."""
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
    return torch.as_tensor(np.ascontiguousarray(x)).cuda()


def prepare(ops, cb):
    sizes = dev(cb.sizes)
    atom_start, edge_start = ops.crystal_offsets(sizes)
    o = ops.batch_prepare(dev(cb.pos), dev(cb.trans_vec), sizes, atom_start, edge_start, cb.num_atoms, cb.num_edges)
    o["atom_start"] = atom_start
    return o


def fused(ops, cb, prep, q, k, v, a, W, Kbins, cutoff, minimum, want_psi=False):
    # geometry alternately as relative positions per edge and as absolute positions per atom
    geo = dict(pos_ij=prep["pos_ij"]) if (Kbins + int(cutoff)) % 2 == 0 else dict(pos_ij=None, pos=dev(cb.pos))
    return ops.infinite_attn_fwd(dev(q), dev(k), dev(v), dev(a), geo.pop("pos_ij"), dev(cb.trans_vec), prep["rvlen"],
                                 prep["batch"], prep["edges"], prep["row_start"], int(cb.sizes.max()), Kbins, DIST_MAX,
                                 WSCALE, None if W is None else dev(W), cutoff, 2, minimum, want_psi_row=want_psi, **geo)


def test_fused_forward_against_golden(ops, golden_ops):
    g = golden_ops
    cb = make_crystals(11, 7, uniform_atoms(1, 6), length_range=(3.0, 9.0))  # the crystals of the golden file
    assert np.array_equal(cb.pos, g["in_pos"])
    prep = prepare(ops, cb)
    qs = g["in_q"] / np.float32(np.sqrt(D))
    out, logit, lse, _ = fused(ops, cb, prep, qs, g["in_k"], g["in_v"], g["in_a"], g["in_W"][0], K, 0.0, 2)
    assert rel_err(out.cpu().numpy(), g["f64_out"]) < TOL
    p = torch.exp(logit - lse[prep["edges"][0]])
    assert rel_err(p.cpu().numpy(), g["f64_prob"]) < TOL


@pytest.mark.parametrize("cutoff,minimum,nmax,Kbins", [(-3.5, 2, 7, 64), (-3.5, 0, 7, 64), (7.5, 2, 5, 64),
                                                       (0.0, 2, 40, 64), (-3.5, 2, 7, 0), (-3.5, 2, 150, 64)])
def test_fused_forward_against_oracle_chain(ops, cutoff, minimum, nmax, Kbins):
    crystals = 3 if nmax > 100 else 10
    cb = make_crystals(61, crystals, uniform_atoms(max(1, nmax // 3), nmax), length_range=(2.5, 9.0) if nmax < 100 else (8.0, 16.0))
    prep = prepare(ops, cb)
    N = cb.num_atoms
    rng = np.random.default_rng(61)
    sig = 1.4 * (0.6 + 0.9 * rng.random((N, H)))
    a = (-0.5 / sig ** 2).astype(np.float32)
    W = (rng.standard_normal((H, D, K)) * 0.1).astype(np.float32)
    q = (rng.standard_normal((N, H, D)) * 0.5).astype(np.float32)
    k, v = (rng.standard_normal((N, H, D)).astype(np.float32) for _ in range(2))
    edges = oracle.edge_index(cb.sizes)
    pos_ij, _, _, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    precision = "f64" if nmax < 100 else "f32"
    z, psiW = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, Kbins, DIST_MAX, WSCALE,
                                     W=W[None] if Kbins else None, rvlen=rvlen, cutoff_radius=cutoff, minimum_range=minimum,
                                     precision=precision)
    prob, ref = oracle.fused_attn_fwd(q, k, v, z, psiW, edges, precision=precision)
    out, logit, lse, psi_row = fused(ops, cb, prep, q, k, v, a, W if Kbins else None, Kbins, cutoff, minimum, want_psi=True)
    assert rel_err(out.cpu().numpy(), ref) < TOL
    p = torch.exp(logit - lse[prep["edges"][0]])
    assert rel_err(p.cpu().numpy(), prob) < TOL
    if Kbins:
        _, psi = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, Kbins, DIST_MAX, WSCALE, rvlen=rvlen,
                                        cutoff_radius=cutoff, minimum_range=minimum, precision=precision)
        row = np.zeros((N, H, K))
        np.add.at(row, edges[0], prob[:, :, None] * psi)
        assert rel_err(psi_row.cpu().numpy(), row) < TOL
    again = fused(ops, cb, prep, q, k, v, a, W if Kbins else None, Kbins, cutoff, minimum)
    assert torch.equal(out, again[0]) and torch.equal(logit, again[1])  # no atomics: bitwise repeatable


@pytest.mark.parametrize("cutoff,minimum,nmax,Kbins,floor", [(-3.5, 2, 7, 64, -30.0), (-3.5, 0, 7, 64, -30.0),
                                                             (7.5, 2, 5, 64, -30.0), (0.0, 2, 40, 64, -30.0),
                                                             (-3.5, 2, 7, 0, -30.0), (-3.5, 2, 150, 64, -30.0),
                                                             (-3.5, 2, 24, 64, -30.0), (-3.5, 0, 30, 64, -30.0),
                                                             (-3.5, 2, 7, 64, -1000.0)])
def test_term_lists_give_the_enumerated_result(ops, cutoff, minimum, nmax, Kbins, floor):
    """The same attention fed from the batch's term lists (found once, for the widest admissible Gaussian) instead of
    enumerating every head's box: against the float64 oracle chain and against the enumerating kernels.  The widths
    here span a factor of 2.5, so heads have different boxes and the listed terms are masked per head.  With the
    weight floor switched off the lists would hold whole boxes; they then do not fit their pool and every row falls
    back to enumeration, which the last case exercises.  Crystals of up to 12 atoms take one warp per row, up to 32
    atoms four warps per row with phi summed inside the row kernel, larger ones the separate phi kernel."""
    crystals = 3 if nmax > 100 else 10
    cb = make_crystals(61, crystals, uniform_atoms(max(1, nmax // 3), nmax), length_range=(2.5, 9.0) if nmax < 100 else (8.0, 16.0))
    prep = prepare(ops, cb)
    N = cb.num_atoms
    rng = np.random.default_rng(61)
    sig = 1.4 * (0.6 + 0.9 * rng.random((N, H)))
    a = (-0.5 / sig ** 2).astype(np.float32)
    a_widest = float(-0.5 / (1.4 * 1.5) ** 2)  # no sigma above 1.4 x 1.5
    W = (rng.standard_normal((H, D, K)) * 0.1).astype(np.float32)
    q = (rng.standard_normal((N, H, D)) * 0.5).astype(np.float32)
    k, v = (rng.standard_normal((N, H, D)).astype(np.float32) for _ in range(2))
    tv, max_atoms = dev(cb.trans_vec), int(cb.sizes.max())
    args = (dev(q), dev(k), dev(v), dev(a), prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"],
            prep["row_start"], max_atoms, Kbins, DIST_MAX, WSCALE, dev(W) if Kbins else None, cutoff, 2, minimum)
    ops.set_weight_floor_log2(floor)
    try:
        lists = ops.term_list_build(prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"], prep["row_start"],
                                    max_atoms, cutoff, 2, minimum, a_widest)
        listed = ops.infinite_attn_fwd(*args, term_lists=lists)
        plain = ops.infinite_attn_fwd(*args)
        again = ops.infinite_attn_fwd(*args, term_lists=lists)
    finally:
        ops.set_weight_floor_log2(-30.0)
    assert torch.equal(listed[0], again[0]) and torch.equal(listed[1], again[1])  # bitwise repeatable
    assert rel_err(listed[0].cpu().numpy(), plain[0].cpu().numpy()) < 2e-6
    assert rel_err(listed[1].cpu().numpy(), plain[1].cpu().numpy()) < 2e-6
    edges = oracle.edge_index(cb.sizes)
    pos_ij, _, _, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    precision = "f64" if nmax < 100 else "f32"
    z, psiW = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, Kbins, DIST_MAX, WSCALE,
                                     W=W[None] if Kbins else None, rvlen=rvlen, cutoff_radius=cutoff, minimum_range=minimum,
                                     precision=precision)
    _, ref = oracle.fused_attn_fwd(q, k, v, z, psiW, edges, precision=precision)
    assert rel_err(listed[0].cpu().numpy(), ref) < TOL
    # backward over the same lists: against the enumerating backward (both from the enumerated forward's logits, so
    # that only the backward differs) and bitwise repeatable; a warp owns whole keys, whatever the list sizes
    go = dev(rng.standard_normal((N, H, D)).astype(np.float32))
    ops.set_weight_floor_log2(floor)
    try:
        g_plain = ops.infinite_attn_bwd(*args, plain[1], plain[2], plain[0], go)
        g_listed = ops.infinite_attn_bwd(*args, plain[1], plain[2], plain[0], go, term_lists=lists)
        g_again = ops.infinite_attn_bwd(*args, plain[1], plain[2], plain[0], go, term_lists=lists)
    finally:
        ops.set_weight_floor_log2(-30.0)
    for got, want, twice in zip(g_listed, g_plain, g_again):
        assert torch.equal(got, twice)
        assert rel_err(got.cpu().numpy(), want.cpu().numpy()) < 5e-6


def test_fused_forward_flags_understated_max_atoms(ops):
    cb = make_crystals(62, 4, uniform_atoms(5, 9))
    prep = prepare(ops, cb)
    N = cb.num_atoms
    z = lambda *s: torch.zeros(s, device="cuda")
    out, _, _, _ = ops.infinite_attn_fwd(z(N, H, D), z(N, H, D), z(N, H, D), -torch.ones((N, H), device="cuda"),
                                         prep["pos_ij"], dev(cb.trans_vec), prep["rvlen"], prep["batch"], prep["edges"],
                                         prep["row_start"], 2, 0, DIST_MAX, WSCALE, None, -3.5, 2, 2)
    assert torch.isnan(out).all()
