"""Pins the CPU oracle: the C restatement (oracle/cf_oracle.c) against vectors from the reference's own PyTorch
implementation (tests/golden/golden_ops.npz) and, where built, against the reference's kernel sources compiled for
the CPU (oracle/_ref).  No GPU."""
import numpy as np
import pytest

import oracle
from conftest import rel_err
from crystalformer_b200.synthetic import all_pairs_edges, make_crystals, uniform_atoms

H, D, K = 8, 16, 64
DIST_MAX, WSCALE = 14.0, 1.0
TOL = 1e-4  # fp32 parity bound: max|x-ref| <= 1e-4 max|ref| per tensor


def _geom(g):
    edges = oracle.edge_index(g["in_sizes"])
    pos_ij, rvecs, vcell, rvlen = oracle.geometry(g["in_pos"], g["in_trans"], edges)
    return edges, pos_ij, rvlen


def test_edge_list_is_bit_exact(golden_ops):
    edges = oracle.edge_index(golden_ops["in_sizes"])
    assert edges.dtype == np.int64
    assert np.array_equal(edges, golden_ops["f32_edges"])
    assert np.array_equal(edges, all_pairs_edges(golden_ops["in_sizes"]))


@pytest.mark.parametrize("precision,tol", [("f32", TOL), ("f64", 1e-6)])  # f64 bound: pos_ij is float32 input
def test_lattice_sum_forward_matches_pytorch_reference(golden_ops, precision, tol):
    g = golden_ops
    edges, pos_ij, _ = _geom(g)
    ref = "f32" if precision == "f32" else "f64"
    z, psi = oracle.lattice_sum_fwd(g["in_a"], pos_ij, g["in_trans"], g["in_batch"], edges, K, DIST_MAX, WSCALE,
                                    precision=precision)
    assert rel_err(z, g[f"{ref}_phi"]) < tol
    assert rel_err(psi, g[f"{ref}_psi"]) < max(tol, 2e-7)  # pos_ij itself is float32 in both builds
    z2, psiW = oracle.lattice_sum_fwd(g["in_a"], pos_ij, g["in_trans"], g["in_batch"], edges, K, DIST_MAX, WSCALE,
                                      W=g["in_W"], precision=precision)
    assert np.array_equal(z, z2)
    assert rel_err(psiW, g[f"{ref}_psiW"]) < max(tol, 2e-7)


@pytest.mark.parametrize("precision,tol", [("f32", TOL), ("f64", 1e-6)])
def test_lattice_sum_backward_matches_pytorch_reference(golden_ops, precision, tol):
    g = golden_ops
    edges, pos_ij, _ = _geom(g)
    z, _ = oracle.lattice_sum_fwd(g["in_a"], pos_ij, g["in_trans"], g["in_batch"], edges, K, DIST_MAX, WSCALE,
                                  W=g["in_W"], precision=precision)
    ga, gW = oracle.lattice_sum_bwd(g["in_a"], pos_ij, g["in_trans"], g["in_batch"], edges, z, g[f"{precision}_g_phi"],
                                    g[f"{precision}_g_psiW"], K, DIST_MAX, WSCALE, W=g["in_W"], precision=precision)
    assert rel_err(ga, g[f"{precision}_g_a"]) < tol
    assert rel_err(gW, g[f"{precision}_g_W"]) < tol


@pytest.mark.parametrize("precision,tol", [("f32", TOL), ("f64", 1e-10)])
def test_attention_matches_pytorch_reference(golden_ops, precision, tol):
    g = golden_ops
    p = precision
    edges = g["f32_edges"]
    qs = g["in_q"].astype(np.float64 if p == "f64" else np.float32) / np.sqrt(D).astype(np.float32 if p == "f32" else np.float64)
    prob, out = oracle.fused_attn_fwd(qs, g["in_k"], g["in_v"], g[f"{p}_phi"], g[f"{p}_psiW"], edges, precision=p)
    assert rel_err(prob, g[f"{p}_prob"]) < tol
    assert rel_err(out, g[f"{p}_out"]) < tol
    gq, gk, gv, ga, gb = oracle.fused_attn_bwd(qs, g["in_k"], g["in_v"], g[f"{p}_psiW"], edges, prob, out, g["in_go"],
                                               precision=p)
    assert rel_err(gq / np.sqrt(D), g[f"{p}_g_q"]) < tol  # chain factor of the q / sqrt(D) pre-scaling
    assert rel_err(gk, g[f"{p}_g_k"]) < tol
    assert rel_err(gv, g[f"{p}_g_v"]) < tol
    assert rel_err(ga, g[f"{p}_g_phi"]) < tol
    assert rel_err(gb, g[f"{p}_g_psiW"]) < tol


def _random_case(seed, crystals=6, nmax=6, lengths=(2.5, 8.0)):
    cb = make_crystals(seed, crystals, uniform_atoms(1, nmax), length_range=lengths)
    edges = oracle.edge_index(cb.sizes)
    pos_ij, rvecs, vcell, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    rng = np.random.default_rng(seed)
    N = cb.num_atoms
    sig = 1.4 * (0.6 + 0.9 * rng.random((N, H)))
    a = (-0.5 / sig ** 2).astype(np.float32)
    W = (rng.standard_normal((1, H, D, K)) * 0.1).astype(np.float32)
    return cb, edges, pos_ij, rvlen, a, W, rng


needs_ref = pytest.mark.skipif(not oracle.have_ref(), reason="reference kernels were not compiled for the CPU here")


@needs_ref
@pytest.mark.parametrize("cutoff", [-3.5, 7.5, 12.0])
def test_restatement_equals_compiled_reference_kernels_lattice_sum(cutoff):
    """Adaptive and static cut-off rules (which the PyTorch path does not have): same integers, same floats."""
    cb, edges, pos_ij, rvlen, a, W, rng = _random_case(7)
    z, v, box = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, K, DIST_MAX, WSCALE, W=W, rvlen=rvlen,
                                       cutoff_radius=cutoff, return_box=True)
    zr, vr = oracle.ref_real_enc_proj_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, K, DIST_MAX, WSCALE, W, rvlen, cutoff)
    assert box.min() >= 2 and box.max() >= 3  # the case really leaves the minimum box
    assert np.array_equal(z, zr)
    assert rel_err(v, vr) < 1e-6
    z0, psi = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, K, DIST_MAX, WSCALE, rvlen=rvlen,
                                     cutoff_radius=cutoff)
    zr0, psir = oracle.ref_real_enc_proj_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, K, DIST_MAX, WSCALE, None, rvlen,
                                             cutoff, proj=False)
    assert np.array_equal(z0, zr0) and rel_err(psi, psir) < 1e-6
    gz = rng.standard_normal(z.shape).astype(np.float32)
    gv = rng.standard_normal(v.shape).astype(np.float32)
    ga, gW = oracle.lattice_sum_bwd(a, pos_ij, cb.trans_vec, cb.batch, edges, z, gz, gv, K, DIST_MAX, WSCALE, W=W,
                                    rvlen=rvlen, cutoff_radius=cutoff)
    gar, gWr = oracle.ref_real_enc_proj_bwd(a, pos_ij, cb.trans_vec, cb.batch, edges, z, gz, gv, K, DIST_MAX, WSCALE, W,
                                            rvlen, cutoff)
    assert rel_err(ga, gar) < 1e-6 and rel_err(gW, gWr) < 1e-5
    gpsi = rng.standard_normal(psi.shape).astype(np.float32)
    ga2, _ = oracle.lattice_sum_bwd(a, pos_ij, cb.trans_vec, cb.batch, edges, z, gz, gpsi, K, DIST_MAX, WSCALE,
                                    rvlen=rvlen, cutoff_radius=cutoff)
    ga2r, _ = oracle.ref_real_enc_proj_bwd(a, pos_ij, cb.trans_vec, cb.batch, edges, z, gz, gpsi, K, DIST_MAX, WSCALE,
                                           None, rvlen, cutoff, proj=False)
    assert rel_err(ga2, ga2r) < 1e-6


@needs_ref
def test_restatement_equals_compiled_reference_kernels_k0():
    cb, edges, pos_ij, rvlen, a, W, rng = _random_case(8)
    z, _ = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, 0, DIST_MAX, WSCALE, rvlen=rvlen,
                                  cutoff_radius=-3.5)
    zr, _ = oracle.ref_real_enc_proj_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, 0, DIST_MAX, WSCALE, None, rvlen, -3.5)
    assert np.array_equal(z, zr)
    gz = rng.standard_normal(z.shape).astype(np.float32)
    ga, _ = oracle.lattice_sum_bwd(a, pos_ij, cb.trans_vec, cb.batch, edges, z, gz, None, 0, DIST_MAX, WSCALE,
                                   rvlen=rvlen, cutoff_radius=-3.5)
    gar, _ = oracle.ref_real_enc_proj_bwd(a, pos_ij, cb.trans_vec, cb.batch, edges, z, gz, None, 0, DIST_MAX, WSCALE,
                                          None, rvlen, -3.5)
    assert rel_err(ga, gar) < 1e-6


@needs_ref
@pytest.mark.parametrize("nmax", [6, 70])  # 70 atoms: more than one 64-wide block of the pairwise softmax sum
def test_restatement_equals_compiled_reference_kernels_attention(nmax):
    cb, edges, pos_ij, rvlen, a, W, rng = _random_case(9, crystals=3, nmax=nmax)
    N, E = cb.num_atoms, edges.shape[1]
    q = (rng.standard_normal((N, H, D)) * 0.5).astype(np.float32)
    k, v, go = (rng.standard_normal((N, H, D)).astype(np.float32) for _ in range(3))
    aij = rng.standard_normal((E, H)).astype(np.float32)
    bij = rng.standard_normal((E, H, D)).astype(np.float32)
    for v3 in (True, False):
        prob, out = oracle.fused_attn_fwd(q, k, v, aij, bij, edges, run_len=8 if v3 else 0)
        pr, outr = oracle.ref_fused_dpa_fwd(q, k, v, aij, bij, edges, v3=v3)
        assert np.array_equal(prob, pr) and np.array_equal(out, outr)
    mine = oracle.fused_attn_bwd(q, k, v, bij, edges, prob, out, go)
    ref = oracle.ref_fused_dpa_bwd(q, k, v, aij, bij, cb.batch, edges, cb.sizes, prob, out, go)
    for x, y in zip(mine, ref):
        assert np.array_equal(x, y)


@needs_ref
def test_restatement_equals_compiled_reference_kernels_mean():
    cb = make_crystals(3, 9, uniform_atoms(1, 40))
    x = np.random.default_rng(0).standard_normal((cb.num_atoms, 128)).astype(np.float32)
    assert np.array_equal(oracle.segment_mean(x, cb.sizes), oracle.ref_irregular_mean(x, cb.sizes))
    ref = np.stack([x[cb.batch == b].astype(np.float64).mean(0) for b in range(cb.num_crystals)])
    assert rel_err(oracle.segment_mean(x, cb.sizes), ref) < 1e-6


def test_box_rule_integers():
    """R = ceil((c + 0.01) |b| / 2pi) with c = 3.5 sqrt(-0.5/a), floor at minimum_range; fixed box when cutoff is 0."""
    rv = np.array([2 * np.pi / 2.0, 2 * np.pi / 3.47, 2 * np.pi / 10.0], np.float32)
    a = np.array([-0.5 / 1.98 ** 2, -0.5 / 1.0 ** 2], np.float32)
    b = oracle.box(a, rv, -3.5, 2, 2)
    assert b.tolist() == [[4, 3, 2], [2, 2, 2]]
    assert oracle.box(a, rv, -3.5, 2, 0).tolist() == [[4, 3, 1], [2, 2, 1]]
    assert oracle.box(a, rv, 0.0, 2, 2).tolist() == [[2, 2, 2], [2, 2, 2]]
    assert oracle.box(a, rv, 6.0, 2, 0).tolist() == [[4, 2, 1], [4, 2, 1]]
