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


def oracle_rows(cb, pick, q, k, v, a, W, Kbins):
    """float64 oracle output for every row of the crystals `pick`: (row indices into the batch, reference rows)."""
    sub = cb.select(pick)
    starts = np.concatenate([[0], np.cumsum(cb.sizes)])
    rows = np.concatenate([np.arange(starts[c], starts[c + 1]) for c in pick])
    e_sub = oracle.edge_index(sub.sizes)
    pij, _, _, rvl = oracle.geometry(sub.pos, sub.trans_vec, e_sub)
    qn, kn, vn, an = (t[rows].cpu().numpy() for t in (q, k, v, a))
    zr, pw = oracle.lattice_sum_fwd(an, pij, sub.trans_vec, sub.batch, e_sub, Kbins, DIST_MAX, WSCALE,
                                    W=None if W is None else W.cpu().numpy()[None], rvlen=rvl, cutoff_radius=-3.5,
                                    precision="f64")
    prob, ref = oracle.fused_attn_fwd(qn, kn, vn, zr, pw, e_sub, precision="f64")
    return rows, ref, (sub, e_sub, pij, rvl, zr, pw, prob)


@pytest.mark.parametrize("cfg,Kbins", [("cfg0", 64), ("cfg2", 0), ("cfg4", 64)])
def test_listed_attention_at_full_size(ops, cfg, Kbins):
    """The kernels that the one-call forwards run - term lists built once per batch - at the sizes of the benchmark
    configurations (cfg2: 7-layer model without the value encoding, K = 0, crystals of up to 60 atoms): invariants,
    agreement with the enumerating kernels and with the operator split, and every row of a few crystals against the
    float64 oracle."""
    cb = make_config(cfg, num_crystals=16 if cfg == "cfg4" else None)
    prep = prepared(ops, cb)
    N = cb.num_atoms
    q, k, v, a, W = random_inputs(N, 11)
    if Kbins == 0:
        W = None
    tv, max_atoms = dev(cb.trans_vec), int(cb.sizes.max())
    geo = (prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"], prep["row_start"], max_atoms)
    a_widest = float(a.max())
    lists = ops.term_list_build(*geo, -3.5, 2, 2, a_widest)
    out, logit, lse, _ = ops.infinite_attn_fwd(q, k, v, a, *geo, Kbins, DIST_MAX, WSCALE, W, -3.5, 2, 2, term_lists=lists)
    plain = ops.infinite_attn_fwd(q, k, v, a, *geo, Kbins, DIST_MAX, WSCALE, W, -3.5, 2, 2)
    assert torch.isfinite(out).all() and torch.isfinite(logit).all()
    p = torch.exp(logit - lse[prep["edges"][0]])
    row_sum = torch.zeros((N, H), device="cuda").index_add_(0, prep["edges"][0], p)
    assert float((row_sum - 1).abs().max()) < 1e-5
    assert rel_err(out.cpu().numpy(), plain[0].cpu().numpy()) < 5e-6
    assert rel_err(logit.cpu().numpy(), plain[1].cpu().numpy()) < 5e-6
    z, psiW = ops.lattice_sum_fwd(a, prep["pos_ij"], tv, prep["batch"], prep["edges"], Kbins, DIST_MAX, WSCALE, W=W,
                                  rvlen=prep["rvlen"], cutoff_radius=-3.5)
    _, out_split = ops.fused_attn_fwd(q, k, v, z, psiW, prep["edges"], prep["row_start"])
    assert rel_err(out.cpu().numpy(), out_split.cpu().numpy()) < TOL
    small = [int(c) for c in np.argsort(cb.sizes)[:2]] if cfg == "cfg4" else [3, 17, 40]
    rows, ref, _ = oracle_rows(cb, small, q, k, v, a, W, Kbins)
    assert rel_err(out[rows].cpu().numpy(), ref) < TOL
    if Kbins == 64 and max_atoms <= 32:  # the row-list organisation of the same batch
        rl = ops.row_list_build(*geo, -3.5, 2, 2, a_widest)
        out_sorted, lse_sorted = ops.infinite_attn_fwd_sorted(q, k, v, a, *geo, Kbins, DIST_MAX, WSCALE, W, -3.5, 2, 2, rl)
        assert rel_err(out_sorted[rows].cpu().numpy(), ref) < TOL
        assert rel_err(out_sorted.cpu().numpy(), out.cpu().numpy()) < 2e-5


def test_listed_backward_against_the_float64_oracle_at_cfg3_size(ops):
    """cf_infinite_attn_bwd_listed on the 256-crystal training batch (term lists as in a training step): the gradients
    of every row of three crystals against the float64 oracle chain (attention backward -> lattice-sum backward)."""
    cb = make_config("cfg3")
    prep = prepared(ops, cb)
    N = cb.num_atoms
    q, k, v, a, W = random_inputs(N, 13)
    go = torch.randn((N, H, D), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    tv, max_atoms = dev(cb.trans_vec), int(cb.sizes.max())
    geo = (prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"], prep["row_start"], max_atoms)
    lists = ops.term_list_build(*geo, -3.5, 2, 2, float(a.max()))
    args = (q, k, v, a, *geo, K, DIST_MAX, WSCALE, W, -3.5, 2, 2)
    out, logit, lse, _ = ops.infinite_attn_fwd(*args, term_lists=lists)
    gq, gk, gv, ga = ops.infinite_attn_bwd(*args, logit, lse, out, go, term_lists=lists)
    pick = [5, 77, 201]
    rows, ref, (sub, e_sub, pij, rvl, zr, pw, prob) = oracle_rows(cb, pick, q, k, v, a, W, K)
    qn, kn, vn, an, gon = (t[rows].cpu().numpy() for t in (q, k, v, a, go))
    rq, rk, rv, rphi, rpsiW = oracle.fused_attn_bwd(qn, kn, vn, pw, e_sub, prob, ref, gon, precision="f64")
    ra, _ = oracle.lattice_sum_bwd(an, pij, sub.trans_vec, sub.batch, e_sub, zr, rphi, rpsiW, K, DIST_MAX, WSCALE,
                                   W=W.cpu().numpy()[None], rvlen=rvl, cutoff_radius=-3.5, lattice_range=2, minimum_range=2,
                                   precision="f64")
    assert rel_err(out[rows].cpu().numpy(), ref) < TOL
    for got, want, name in ((gq, rq, "gq"), (gk, rk, "gk"), (gv, rv, "gv"), (ga, ra, "ga")):
        assert rel_err(got[rows].cpu().numpy(), want) < TOL, name


@pytest.mark.parametrize("config,crystals", [("cfg0", 24), ("cfg3", 20)])
def test_one_call_model_forward_of_the_bench_configuration_against_the_cpu_model(config, crystals):
    """The path the benchmark times - cf_model_forward: embedding inside the first dense block, row lists, the sorted
    row kernel, the fused dense blocks, pooling + head - on the 4-layer, ff 512, K = 64 model over 24 crystals of the
    headline configuration (at most 30 atoms: two key tiles) and 20 of the training configuration (up to 40 atoms: four
    key tiles), against the CPU restatement of the reference model with the same state_dict."""
    import types
    import bench
    from oracle.model_cpu import forward_cpu
    cb = make_config(config, num_crystals=crystals)
    model, params = bench.make_model(4, 64)
    model = model.cuda()
    batch = bench.to_device_batch(cb, torch.device("cuda"))
    bench.fix_gauss_scale(model, batch)
    with torch.no_grad():
        y = model(batch)
        model.native = False  # the same model operator by operator (torch modules + the fused attention operator)
        y_ops = model(batch)
        model.native = True
    state = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    y_cpu = forward_cpu(state, params, cb, use_ref=False)
    assert rel_err(y.cpu().numpy(), y_cpu) < TOL
    assert rel_err(y_ops.cpu().numpy(), y_cpu) < TOL
