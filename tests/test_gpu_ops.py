"""GPU parity of the operator-level kernels against the CPU oracle and the reference-made golden vectors.
Every call goes through the C ABI (crystalformer_b200.ops -> ctypes -> libcrystalformer_b200.so)."""
import numpy as np
import pytest
import torch

import oracle
from conftest import rel_err
from crystalformer_b200.synthetic import make_config, make_crystals, uniform_atoms

pytestmark = pytest.mark.gpu

H, D, K = 8, 16, 64
DIST_MAX, WSCALE = 14.0, 1.0
TOL = 1e-4  # fp32 parity bound (max|x-ref| / max|ref| per tensor)


@pytest.fixture(scope="module")
def ops():
    from crystalformer_b200 import ops as _ops
    assert torch.cuda.is_available()
    return _ops


def dev(x):
    return torch.as_tensor(np.ascontiguousarray(x)).cuda()


def case(seed, crystals=8, nmax=6, lengths=(2.5, 8.0), nmin=1):
    cb = make_crystals(seed, crystals, uniform_atoms(nmin, nmax), length_range=lengths)
    edges = oracle.edge_index(cb.sizes)
    pos_ij, rvecs, vcell, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    rng = np.random.default_rng(seed)
    sig = 1.4 * (0.6 + 0.9 * rng.random((cb.num_atoms, H)))
    a = (-0.5 / sig ** 2).astype(np.float32)
    W = (rng.standard_normal((1, H, D, K)) * 0.1).astype(np.float32)
    return cb, edges, pos_ij, rvlen, a, W, rng


def test_batch_prepare_matches_reference_layout(ops):
    cb = make_crystals(21, 40, uniform_atoms(1, 9))
    sizes = dev(cb.sizes)
    atom_start, edge_start = ops.crystal_offsets(sizes)
    assert atom_start.cpu().tolist() == np.concatenate([[0], np.cumsum(cb.sizes)]).tolist()
    assert edge_start.cpu().tolist() == np.concatenate([[0], np.cumsum(cb.sizes ** 2)]).tolist()
    o = ops.batch_prepare(dev(cb.pos), dev(cb.trans_vec), sizes, atom_start, edge_start, cb.num_atoms, cb.num_edges)
    edges = oracle.edge_index(cb.sizes)
    pos_ij, rvecs, vcell, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    assert np.array_equal(o["edges"].cpu().numpy(), edges)                 # integers: bit exact
    assert np.array_equal(o["batch"].cpu().numpy(), cb.batch)
    assert np.array_equal(o["row_start"].cpu().numpy(), oracle.row_starts(edges, cb.num_atoms))
    assert np.array_equal(o["pos_ij"].cpu().numpy(), pos_ij)               # one float subtraction: bit exact
    assert rel_err(o["vcell"].cpu().numpy(), vcell) < 1e-6
    assert rel_err(o["rvecs"].cpu().numpy(), rvecs) < 1e-6
    assert rel_err(o["rvlen"].cpu().numpy(), rvlen) < 1e-6


@pytest.mark.parametrize("cutoff,minimum", [(-3.5, 2), (-3.5, 0), (7.5, 2), (12.0, 0), (0.0, 2)])
def test_translation_boxes_are_bit_exact(ops, cutoff, minimum):
    cb, edges, pos_ij, rvlen, a, W, rng = case(31, crystals=30)
    box = ops.lattice_box(dev(a), dev(cb.batch), dev(edges), dev(rvlen), cutoff, 2, minimum).cpu().numpy()
    _, _, ref = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, 0, DIST_MAX, WSCALE, rvlen=rvlen,
                                       cutoff_radius=cutoff, minimum_range=minimum, return_box=True)
    assert np.array_equal(box, ref)
    if cutoff != 0.0:
        assert ref.max() > 2
    # one width per (edge, head)
    ae = (-0.5 / (1.4 * (0.5 + rng.random((edges.shape[1], H)))) ** 2).astype(np.float32)
    box = ops.lattice_box(dev(ae), dev(cb.batch), dev(edges), dev(rvlen), cutoff, 2, minimum, a_per_edge=True).cpu().numpy()
    _, _, ref = oracle.lattice_sum_fwd(ae, pos_ij, cb.trans_vec, cb.batch, edges, 0, DIST_MAX, WSCALE, rvlen=rvlen,
                                       cutoff_radius=cutoff, minimum_range=minimum, a_per_edge=True, return_box=True)
    assert np.array_equal(box, ref)


def test_lattice_sum_forward_against_golden(ops, golden_ops):
    """Fixed (2R+1)^3 box, as the reference's PyTorch path enumerates it."""
    g = golden_ops
    edges = g["f32_edges"]
    pos_ij, _, _, _ = oracle.geometry(g["in_pos"], g["in_trans"], edges)
    args = (dev(g["in_a"]), dev(pos_ij), dev(g["in_trans"]), dev(g["in_batch"]), dev(edges), K, DIST_MAX, WSCALE)
    z, psi = ops.lattice_sum_fwd(*args)
    assert rel_err(z.cpu().numpy(), g["f32_phi"]) < TOL and rel_err(z.cpu().numpy(), g["f64_phi"]) < TOL
    assert rel_err(psi.cpu().numpy(), g["f32_psi"]) < TOL and rel_err(psi.cpu().numpy(), g["f64_psi"]) < TOL
    z2, psiW = ops.lattice_sum_fwd(*args, W=dev(g["in_W"]))
    assert torch.equal(z, z2)
    assert rel_err(psiW.cpu().numpy(), g["f32_psiW"]) < TOL and rel_err(psiW.cpu().numpy(), g["f64_psiW"]) < TOL
    z3, none = ops.lattice_sum_fwd(dev(g["in_a"]), dev(pos_ij), dev(g["in_trans"]), dev(g["in_batch"]), dev(edges), 0,
                                   DIST_MAX, WSCALE)
    assert none is None and rel_err(z3.cpu().numpy(), g["f64_phi"]) < TOL


@pytest.mark.parametrize("cutoff,minimum", [(-3.5, 2), (-3.5, 0), (7.5, 2), (0.0, 2)])
@pytest.mark.parametrize("floor", [-30.0, -1000.0])
def test_lattice_sum_forward_against_oracle(ops, cutoff, minimum, floor):
    """Adaptive / static cut-off rules, heads with different boxes, all W layouts, one width per edge."""
    cb, edges, pos_ij, rvlen, a, W, rng = case(32, crystals=10, nmax=7)
    E, N = edges.shape[1], cb.num_atoms
    ops.set_weight_floor_log2(floor)
    try:
        common = dict(rvlen=rvlen, cutoff_radius=cutoff, lattice_range=2, minimum_range=minimum)
        dcommon = dict(rvlen=dev(rvlen), cutoff_radius=cutoff, lattice_range=2, minimum_range=minimum)
        base = (dev(a), dev(pos_ij), dev(cb.trans_vec), dev(cb.batch), dev(edges), K, DIST_MAX, WSCALE)
        z64, psi64 = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, K, DIST_MAX, WSCALE,
                                            precision="f64", **common)
        z, psi = ops.lattice_sum_fwd(*base, **dcommon)
        assert rel_err(z.cpu().numpy(), z64) < TOL and rel_err(psi.cpu().numpy(), psi64) < TOL
        for Wn in (W, np.repeat(W, N, 0) * rng.random((N, 1, 1, 1)).astype(np.float32),
                   np.repeat(W, E, 0) * rng.random((E, 1, 1, 1)).astype(np.float32)):
            _, ref = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, K, DIST_MAX, WSCALE, W=Wn,
                                            precision="f64", **common)
            _, got = ops.lattice_sum_fwd(*base, W=dev(Wn), **dcommon)
            assert rel_err(got.cpu().numpy(), ref) < TOL
        ae = (-0.5 / (1.4 * (0.5 + rng.random((E, H)))) ** 2).astype(np.float32)
        zr, pr = oracle.lattice_sum_fwd(ae, pos_ij, cb.trans_vec, cb.batch, edges, K, DIST_MAX, WSCALE,
                                        a_per_edge=True, precision="f64", **common)
        zg, pg = ops.lattice_sum_fwd(dev(ae), *base[1:], a_per_edge=True, **dcommon)
        assert rel_err(zg.cpu().numpy(), zr) < TOL and rel_err(pg.cpu().numpy(), pr) < TOL
        zk0, _ = ops.lattice_sum_fwd(*base[:5], 0, DIST_MAX, WSCALE, **dcommon)
        assert rel_err(zk0.cpu().numpy(), z64) < TOL
    finally:
        ops.set_weight_floor_log2(-30.0)


def test_lattice_sum_forward_ragged_and_degenerate(ops):
    """Single-atom cells (only the self edge), an empty batch, and run-to-run bitwise determinism."""
    cb, edges, pos_ij, rvlen, a, W, rng = case(33, crystals=5, nmax=1)
    z, psi = ops.lattice_sum_fwd(dev(a), dev(pos_ij), dev(cb.trans_vec), dev(cb.batch), dev(edges), K, DIST_MAX, WSCALE,
                                 rvlen=dev(rvlen), cutoff_radius=-3.5)
    zr, pr = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, K, DIST_MAX, WSCALE, rvlen=rvlen,
                                    cutoff_radius=-3.5, precision="f64")
    assert rel_err(z.cpu().numpy(), zr) < TOL and rel_err(psi.cpu().numpy(), pr) < TOL
    e0 = torch.zeros((2, 0), dtype=torch.int64, device="cuda")
    z0, p0 = ops.lattice_sum_fwd(dev(a), torch.zeros((0, 3), device="cuda"), dev(cb.trans_vec), dev(cb.batch), e0, K,
                                 DIST_MAX, WSCALE)
    assert z0.shape == (0, H) and p0.shape == (0, H, K)
    cb, edges, pos_ij, rvlen, a, W, rng = case(34, crystals=12, nmax=12)
    args = (dev(a), dev(pos_ij), dev(cb.trans_vec), dev(cb.batch), dev(edges), K, DIST_MAX, WSCALE)
    r1 = ops.lattice_sum_fwd(*args, W=dev(W), rvlen=dev(rvlen), cutoff_radius=-3.5)
    r2 = ops.lattice_sum_fwd(*args, W=dev(W), rvlen=dev(rvlen), cutoff_radius=-3.5)
    assert torch.equal(r1[0], r2[0]) and torch.equal(r1[1], r2[1])


def test_attention_against_golden(ops, golden_ops):
    g = golden_ops
    edges = g["f32_edges"]
    N = g["in_q"].shape[0]
    row_start = dev(oracle.row_starts(edges, N))
    qs = dev(g["in_q"]) / np.float32(np.sqrt(D))
    prob, out = ops.fused_attn_fwd(qs, dev(g["in_k"]), dev(g["in_v"]), dev(g["f32_phi"]), dev(g["f32_psiW"]),
                                   dev(edges), row_start)
    assert rel_err(prob.cpu().numpy(), g["f64_prob"]) < TOL and rel_err(out.cpu().numpy(), g["f64_out"]) < TOL
    gq, gk, gv, ga, gb = ops.fused_attn_bwd(qs, dev(g["in_k"]), dev(g["in_v"]), dev(g["f32_psiW"]), dev(edges),
                                            row_start, prob, out, dev(g["in_go"]))
    assert rel_err(gq.cpu().numpy() / np.sqrt(D), g["f64_g_q"]) < TOL
    assert rel_err(gk.cpu().numpy(), g["f64_g_k"]) < TOL and rel_err(gv.cpu().numpy(), g["f64_g_v"]) < TOL
    assert rel_err(ga.cpu().numpy(), g["f64_g_phi"]) < TOL and rel_err(gb.cpu().numpy(), g["f64_g_psiW"]) < TOL


@pytest.mark.parametrize("nmax,with_pos", [(6, True), (70, True), (400, False)])
def test_attention_against_oracle(ops, nmax, with_pos):
    """Crystals beyond one warp of keys, beyond the reference's 64-wide summation block and its 320-atom limit."""
    cb = make_crystals(41, 3, uniform_atoms(max(1, nmax - 3), nmax))
    edges = oracle.edge_index(cb.sizes)
    N, E = cb.num_atoms, edges.shape[1]
    rng = np.random.default_rng(41)
    q = (rng.standard_normal((N, H, D)) * 0.5).astype(np.float32)
    k, v, go = (rng.standard_normal((N, H, D)).astype(np.float32) for _ in range(3))
    aij = rng.standard_normal((E, H)).astype(np.float32) if with_pos else None
    bij = rng.standard_normal((E, H, D)).astype(np.float32) if with_pos else None
    pr, outr = oracle.fused_attn_fwd(q, k, v, aij, bij, edges, precision="f64")
    row_start = dev(oracle.row_starts(edges, N))
    dn = lambda x: None if x is None else dev(x)
    prob, out = ops.fused_attn_fwd(dev(q), dev(k), dev(v), dn(aij), dn(bij), dev(edges), row_start)
    assert rel_err(prob.cpu().numpy(), pr) < TOL and rel_err(out.cpu().numpy(), outr) < TOL
    ref = oracle.fused_attn_bwd(q, k, v, bij, edges, pr, outr, go, precision="f64")
    got = ops.fused_attn_bwd(dev(q), dev(k), dev(v), dn(bij), dev(edges), row_start, prob, out, dev(go))
    for x, y in zip(got, ref):
        if y is not None:
            assert rel_err(x.cpu().numpy(), y) < TOL
    again = ops.fused_attn_bwd(dev(q), dev(k), dev(v), dn(bij), dev(edges), row_start, prob, out, dev(go))
    assert all(torch.equal(x, y) for x, y in zip(got, again) if x is not None)


def test_segment_mean_is_bit_exact(ops):
    cb = make_crystals(51, 37, uniform_atoms(1, 200))
    x = np.random.default_rng(0).standard_normal((cb.num_atoms, 128)).astype(np.float32)
    start = dev(np.concatenate([[0], np.cumsum(cb.sizes)]).astype(np.int64))
    got = ops.segment_mean(dev(x), start).cpu().numpy()
    assert np.array_equal(got, oracle.segment_mean(x, cb.sizes))


def test_errors_are_reported_not_thrown_away(ops):
    from crystalformer_b200._lib import CrystalformerB200Error
    a = torch.zeros((4, 4), device="cuda")  # H = 4 is not compiled
    with pytest.raises(CrystalformerB200Error) as err:
        ops.lattice_sum_fwd(a, torch.zeros((4, 3), device="cuda"), torch.zeros((1, 3, 3), device="cuda"),
                            torch.zeros(4, dtype=torch.int64, device="cuda"),
                            torch.zeros((2, 4), dtype=torch.int64, device="cuda"), K, DIST_MAX, WSCALE)
    assert err.value.code == -2 and "H=4" in str(err.value)
    with pytest.raises(RuntimeError):
        ops.lattice_sum_fwd(torch.zeros((4, 8)), torch.zeros((4, 3)), torch.zeros((1, 3, 3)),
                            torch.zeros(4, dtype=torch.int64), torch.zeros((2, 4), dtype=torch.int64), K, DIST_MAX, WSCALE)


@pytest.mark.parametrize("crystals,nmax", [(1, 5), (37, 9), (128, 30), (1500, 4)])
def test_row_order_is_the_stable_descending_sort_of_the_row_costs(ops, crystals, nmax):
    """The single-launch ordering kernel against torch's stable sort of cf_row_cost; integers, so bit exact."""
    cb = make_crystals(50 + crystals, crystals, uniform_atoms(1, nmax))
    sizes, trans = dev(cb.sizes), dev(cb.trans_vec)
    atom_start, _ = ops.crystal_offsets(sizes)
    cost = ops.row_cost(atom_start, trans, cb.num_atoms)
    # the cost model itself: 1500 + n (1 + sphere / |det T|)
    n = cb.sizes[cb.batch].astype(np.float64)
    vol = np.abs(np.linalg.det(cb.trans_vec.astype(np.float64)))[cb.batch]
    ref_cost = 1500.0 + n * (1.0 + 4.18879020478639 * 15.0 ** 3 / vol)
    assert rel_err(cost.cpu().numpy(), ref_cost) < 1e-5
    want = torch.argsort(cost, descending=True, stable=True).to(torch.int32)
    got = ops.row_order(atom_start, trans, cb.num_atoms)
    assert torch.equal(got, want)
