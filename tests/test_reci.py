"""Reciprocal-space lattice sum: the oracle against the reference-made golden vectors and the reference's own kernels
compiled for the CPU (no GPU needed), then the CUDA kernels against the oracle (``-m gpu``).

Tolerances.  S is a sum of signed cosine terms, so phi = log max(S, 1e-6) + ... is compared through S where S may come
close to zero: |dS| <= 1e-4 max|S|; on the golden case (S >= 0.7 everywhere) phi and the gradient are compared
directly with the suite's 1e-4 relative bound."""
import os

import numpy as np
import pytest

import oracle
from conftest import REPO, rel_err
from crystalformer_b200.synthetic import make_crystals, uniform_atoms

TOL = 1e-4
H = 8


@pytest.fixture(scope="module")
def golden():
    return dict(np.load(os.path.join(REPO, "tests", "golden", "golden_reci.npz")))


def geometry(sizes, pos, trans, batch):
    edges = oracle.edge_index(sizes)
    pos_ij, rvecs, vcell, _ = oracle.geometry(pos, trans, edges)
    return edges, pos_ij, rvecs, vcell, oracle.reci_phase(pos_ij, rvecs, batch, edges)


def norm_grad(a, gz, edges, N):
    """d/da of the 1.5 log(-4 pi a) term, which the reference's autograd path has and its CUDA kernel leaves out."""
    start = oracle.row_starts(edges, N)
    rows = np.zeros((N, H))
    np.add.at(rows, edges[0], gz.astype(np.float64))
    assert start[-1] == edges.shape[1]
    return 1.5 / a.astype(np.float64) * rows


def test_oracle_matches_reference_pytorch_path(golden):
    G = golden
    sizes, pos, trans, batch, a, gz = (G["in_" + k] for k in ("sizes", "pos", "trans", "batch", "a", "gz"))
    edges, pos_ij, rvecs, vcell, kr = geometry(sizes, pos, trans, batch)
    assert np.array_equal(edges, G["f32_edges"])
    assert rel_err(vcell, G["f32_vcell"]) < 1e-6
    for prec, tol in (("f32", TOL), ("f64", 1e-6)):  # f64: inputs are the float32 geometry, hence 1e-6 and not 1e-12
        z, s = oracle.reci_sum_fwd(a, kr, rvecs, vcell, batch, edges, precision=prec)
        assert s.min() > 0.5
        assert rel_err(z, G[prec + "_phi"]) < tol
        ga = oracle.reci_sum_bwd(a, kr, rvecs, batch, edges, gz, s, precision=prec)
        assert rel_err(ga + norm_grad(a, gz, edges, len(batch)), G[prec + "_g_a"]) < tol


def test_nested_summation_variant_agrees(golden):
    G = golden
    sizes, pos, trans, batch, a = (G["in_" + k] for k in ("sizes", "pos", "trans", "batch", "a"))
    edges, pos_ij, rvecs, vcell, kr = geometry(sizes, pos, trans, batch)
    z0, _ = oracle.reci_sum_fwd(a, kr, rvecs, vcell, batch, edges)
    z1, _ = oracle.reci_sum_fwd(a, kr, rvecs, vcell, batch, edges, nested=True)
    assert rel_err(z1, z0) < 1e-6


@pytest.mark.skipif(not oracle.have_ref(), reason="reference kernels were not compiled for the CPU here")
@pytest.mark.parametrize("width", [0.5, 1.0, 3.0])
def test_oracle_is_bit_identical_to_reference_kernels(width):
    cb = make_crystals(31, 9, uniform_atoms(1, 8), length_range=(3.0, 12.0))
    edges, pos_ij, rvecs, vcell, kr = geometry(cb.sizes, cb.pos, cb.trans_vec, cb.batch)
    rng = np.random.default_rng(7)
    a = (-0.5 * (width * (0.5 + rng.random((cb.num_atoms, H)))) ** 2).astype(np.float32)
    z, s = oracle.reci_sum_fwd(a, kr, rvecs, vcell, cb.batch, edges)
    zr, sr = oracle.ref_reci_enc_fwd(a, kr, rvecs, vcell, cb.batch, edges)
    assert np.array_equal(s, sr) and np.array_equal(z, zr)  # clamped and negative sums included
    gz = rng.standard_normal(z.shape).astype(np.float32)
    ga = oracle.reci_sum_bwd(a, kr, rvecs, cb.batch, edges, gz, s)
    gr = oracle.ref_reci_enc_bwd(a, kr, rvecs, vcell, cb.batch, edges, zr, gz, sr)
    assert np.array_equal(ga, gr)


# ---- CUDA kernels -------------------------------------------------------------------------------------------------
def dev(x):
    import torch
    return torch.as_tensor(np.ascontiguousarray(x)).cuda()


@pytest.mark.gpu
def test_gpu_matches_golden(golden):
    from crystalformer_b200 import ops
    G = golden
    sizes, pos, trans, batch, a, gz = (G["in_" + k] for k in ("sizes", "pos", "trans", "batch", "a", "gz"))
    edges, pos_ij, rvecs, vcell, kr = geometry(sizes, pos, trans, batch)
    start = dev(oracle.row_starts(edges, len(batch)))
    kr_gpu = ops.reci_phase(dev(pos_ij), dev(rvecs), dev(batch), dev(edges))
    assert rel_err(kr_gpu.cpu().numpy(), kr) < 1e-6
    z, s = ops.reci_sum_fwd(dev(a), kr_gpu, dev(rvecs), dev(vcell), dev(batch), start, edges.shape[1], 2)
    assert rel_err(z.cpu().numpy(), G["f64_phi"]) < TOL
    ga = ops.reci_sum_bwd(dev(a), kr_gpu, dev(rvecs), dev(batch), start, dev(gz), s, 2)
    assert rel_err(ga.cpu().numpy() + norm_grad(a, gz, edges, len(batch)), G["f64_g_a"]) < TOL


@pytest.mark.gpu
@pytest.mark.parametrize("width,R", [(0.5, 2), (1.0, 2), (3.0, 2), (1.5, 1), (1.5, 4)])
def test_gpu_matches_oracle(width, R):
    """Ragged crystals of 1..70 atoms (rows longer than one pass of the thread block included), widths for which the
    truncated sum goes negative and is clamped, other box sizes than the reference's compiled R = 2."""
    from crystalformer_b200 import ops
    cb = make_crystals(33, 12, lambda r, n: np.concatenate([r.integers(1, 12, n - 2), [70, 33]]), length_range=(3.0, 12.0))
    edges, pos_ij, rvecs, vcell, kr = geometry(cb.sizes, cb.pos, cb.trans_vec, cb.batch)
    rng = np.random.default_rng(9)
    a = (-0.5 * (width * (0.5 + rng.random((cb.num_atoms, H)))) ** 2).astype(np.float32)
    zo, so = oracle.reci_sum_fwd(a, kr, rvecs, vcell, cb.batch, edges, lattice_range=R, precision="f64")
    start = dev(oracle.row_starts(edges, cb.num_atoms))
    z, s = ops.reci_sum_fwd(dev(a), dev(kr), dev(rvecs), dev(vcell), dev(cb.batch), start, edges.shape[1], R)
    s_np, z_np = s.cpu().numpy(), z.cpu().numpy()
    assert np.abs(s_np - so).max() <= TOL * np.abs(so).max()
    ok = so > 0.05  # where the log is well conditioned the phases themselves agree
    assert np.abs(z_np - zo)[ok].max() <= 20 * TOL * np.abs(zo).max()
    clamped = so < 0.5e-6
    if clamped.any():  # far below the clamp both sides return log(1e-6) + normalisation
        assert np.abs(z_np - zo)[clamped & (s_np < 1e-6)].max() <= TOL * np.abs(zo).max()
    # backward with the oracle's own S as the saved sum, so that only the gradient kernel is compared
    gz = rng.standard_normal(zo.shape).astype(np.float32)
    go = oracle.reci_sum_bwd(a, kr, rvecs, cb.batch, edges, gz, so.astype(np.float32), lattice_range=R, precision="f64")
    ga = ops.reci_sum_bwd(dev(a), dev(kr), dev(rvecs), dev(cb.batch), start, dev(gz), dev(so.astype(np.float32)), R)
    # entries with S barely above the 1e-6 clamp weigh in with 1/S ~ 1e6, which amplifies float rounding: where the
    # reference's own float arithmetic (the f32 oracle) is further than TOL from the f64 result, that distance bounds
    g32 = oracle.reci_sum_bwd(a, kr, rvecs, cb.batch, edges, gz, so.astype(np.float32), lattice_range=R)
    assert rel_err(ga.cpu().numpy(), go) < max(TOL, 2 * rel_err(g32, go))
    # run-to-run bitwise reproducibility
    z2, s2 = ops.reci_sum_fwd(dev(a), dev(kr), dev(rvecs), dev(vcell), dev(cb.batch), start, edges.shape[1], R)
    assert np.array_equal(z2.cpu().numpy(), z_np) and np.array_equal(s2.cpu().numpy(), s_np)


@pytest.mark.gpu
def test_dropin_function_and_module_domains():
    """ReciPeriodicEncodingFuncCUDA under autograd, and the attention module in the reci / multihead domains against
    the same module evaluated from oracle-made phi."""
    import torch
    from crystalformer_b200.cuda_funcs import ReciPeriodicEncodingFuncCUDA, compile_kernels
    compile_kernels(2, 8, 16, 64, 16, True)
    cb = make_crystals(35, 6, uniform_atoms(1, 7), length_range=(3.0, 9.0))
    edges, pos_ij, rvecs, vcell, kr = geometry(cb.sizes, cb.pos, cb.trans_vec, cb.batch)
    rng = np.random.default_rng(11)
    a_np = (-0.5 * (2.5 + 2.0 * rng.random((cb.num_atoms, H))) ** 2).astype(np.float32)
    a = dev(a_np).requires_grad_(True)
    z = ReciPeriodicEncodingFuncCUDA.apply(a, dev(kr), dev(rvecs), dev(vcell), dev(cb.batch), dev(edges))
    gz = rng.standard_normal(z.shape).astype(np.float32)
    (z * dev(gz)).sum().backward()
    zo, so = oracle.reci_sum_fwd(a_np, kr, rvecs, vcell, cb.batch, edges, precision="f64")
    go = oracle.reci_sum_bwd(a_np, kr, rvecs, cb.batch, edges, gz, so, precision="f64")
    assert rel_err(z.detach().cpu().numpy(), zo) < TOL
    assert rel_err(a.grad.cpu().numpy(), go) < TOL

    from crystalformer_b200.attention import CrystalformerMultiheadAttentionCUDA
    from crystalformer_b200.encoder import BatchGeometry
    from crystalformer_b200.params import LatticeformerParams
    g = BatchGeometry(dev(cb.pos), dev(cb.trans_vec), dev(cb.sizes))
    x = dev(rng.standard_normal((cb.num_atoms, 128)).astype(np.float32))
    for domain in ("reci", "multihead"):
        P = LatticeformerParams(domain=domain, scale_reci=[2.2], value_pe_dist_real=64)
        P = P.getLayerParameters(0)
        torch.manual_seed(0)
        att = CrystalformerMultiheadAttentionCUDA(128, 8, dropout=0.0, params=P).cuda().eval()
        with torch.no_grad():
            att.gauss_scale.copy_(torch.tensor([1.0, 0.0]))
            y = att(x, x, x, g.batch, g.batch, g.edges, g.pos_ij, None, dev(cb.trans_vec), g.kr_base, g.rvecs, g.vcell,
                    None, need_weights=False, rvlen=g.rvlen)[0]
            # the same forward from oracle-made phi (and psi W for the real-space half)
            w_in = torch.cat((att.q_proj_weight, att.k_proj_weight, att.v_proj_weight), 0)
            q, k, v = torch.nn.functional.linear(x, w_in, att.in_proj_bias).split(128, dim=1)
            q, k, v = (t.reshape(-1, 8, 16) for t in (q, k, v))
            a_mod = att._widths(x, q).cpu().numpy()
        if domain == "reci":
            phi, _ = oracle.reci_sum_fwd(a_mod, kr, rvecs, vcell, cb.batch, edges, precision="f64")
            vals = None
        else:
            rvlen = np.linalg.norm(rvecs, axis=-1).astype(np.float32)
            a_real = np.concatenate([a_mod[:, :4], a_mod[:, :4]], 1)
            W = att.pe_dist_proj.detach().cpu().numpy()
            W = np.concatenate([W[:, :4], W[:, :4]], 1)
            zr, vr = oracle.lattice_sum_fwd(a_real, pos_ij, cb.trans_vec, cb.batch, edges, 64, 14.0, 1.0, W=W,
                                            rvlen=rvlen, cutoff_radius=-3.5, precision="f64")
            a_rec = np.concatenate([a_mod[:, 4:], a_mod[:, 4:]], 1)
            zq, _ = oracle.reci_sum_fwd(a_rec, kr, rvecs, vcell, cb.batch, edges, precision="f64")
            phi = np.concatenate([zr[:, :4], zq[:, 4:]], 1)
            vals = np.concatenate([vr[:, :4], np.zeros_like(vr[:, 4:])], 1)
        _, out = oracle.fused_attn_fwd((q / 4).cpu().numpy(), k.cpu().numpy(), v.cpu().numpy(), phi, vals, edges,
                                       precision="f64")
        with torch.no_grad():
            ref = torch.nn.functional.linear(dev(out.reshape(-1, 128).astype(np.float32)), att.out_proj.weight,
                                             att.out_proj.bias)
        assert rel_err(y.cpu().numpy(), ref.cpu().numpy()) < TOL, domain
