"""GPU parity of the row-list path (cf_row_list_build + cf_infinite_attn_fwd_sorted: distance-sorted row lists, one
warp per row, tensor-core sums) against the float64 oracle chain lattice sum -> edge-indexed attention, against the
reference-made golden vectors and against the enumerating kernel."""
import numpy as np
import pytest
import torch

import oracle
from conftest import rel_err
from crystalformer_b200.synthetic import make_config, make_crystals, uniform_atoms

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
    return ops.batch_prepare(dev(cb.pos), dev(cb.trans_vec), sizes, atom_start, edge_start, cb.num_atoms, cb.num_edges)


def carve(work, N, E):
    """Views of a row-list workspace (the layout of csrc/row_list.cuh)."""
    up = lambda v: (v + 255) & ~255
    at = 0
    rowdir = work[at:at + 32 * N].view(torch.int32).view(N, 8); at += up(32 * N)
    dmin = work[at:at + 4 * E].view(torch.float32); at += up(4 * E)
    sched = work[at:at + 256].view(torch.int32).view(16, 4); at += 256
    leftover = work[at:at + 4 * N].view(torch.int32); at += up(4 * N)
    tasks = work[at:at + 8 * N].view(torch.int32).view(2, N); at += up(8 * N)
    cursor = work[at:at + 8].view(torch.int64)
    task_count = work[at + 8:at + 16].view(torch.int32); at += 256
    pool = work[at:].view(torch.float32).view(-1, 2)
    return rowdir, dmin, sched, leftover, cursor, pool, tasks, task_count


def sorted_forward(ops, cb, prep, q, k, v, a, W, cutoff, minimum, a_widest, row_order=None):
    tv, max_atoms = dev(cb.trans_vec), int(cb.sizes.max())
    lists = ops.row_list_build(prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"], prep["row_start"], max_atoms,
                               cutoff, 2, minimum, a_widest, row_order=row_order)
    out, lse = ops.infinite_attn_fwd_sorted(dev(q), dev(k), dev(v), dev(a), prep["pos_ij"], tv, prep["rvlen"], prep["batch"],
                                            prep["edges"], prep["row_start"], max_atoms, K, DIST_MAX, WSCALE, dev(W), cutoff,
                                            2, minimum, lists)
    return out, lse, lists


def test_sorted_forward_against_golden(ops, golden_ops):
    g = golden_ops
    cb = make_crystals(11, 7, uniform_atoms(1, 6), length_range=(3.0, 9.0))  # the crystals of the golden file
    assert np.array_equal(cb.pos, g["in_pos"])
    prep = prepare(ops, cb)
    qs = g["in_q"] / np.float32(np.sqrt(D))
    a_widest = float(g["in_a"].max())
    out, lse, _ = sorted_forward(ops, cb, prep, qs, g["in_k"], g["in_v"], g["in_a"], g["in_W"][0], 0.0, 2, a_widest)
    assert rel_err(out.cpu().numpy(), g["f64_out"]) < TOL


@pytest.mark.parametrize("cutoff,minimum,nmax,floor", [(-3.5, 2, 7, -30.0), (-3.5, 0, 7, -30.0), (7.5, 2, 5, -30.0),
                                                       (0.0, 2, 30, -30.0), (-3.5, 2, 16, -30.0), (-3.5, 2, 24, -30.0),
                                                       (-3.5, 0, 32, -30.0), (-3.5, 2, 7, -1000.0), (0.0, 2, 20, -1000.0)])
def test_sorted_rows_against_oracle_chain(ops, cutoff, minimum, nmax, floor):
    """Widths span a factor of 2.5 (heads have different boxes, masked per head from the entries' |n| bytes).  Cells of
    2.5 Angstrom with tens of atoms give rows of more than 4096 entries, which fall back to the enumerating kernel inside
    the same call; with the weight floor switched off the lists hold whole boxes and nothing is skipped."""
    cb = make_crystals(61, 10, uniform_atoms(max(1, nmax // 3), nmax), length_range=(2.5, 9.0))
    prep = prepare(ops, cb)
    N = cb.num_atoms
    rng = np.random.default_rng(61)
    sig = 1.4 * (0.6 + 0.9 * rng.random((N, H)))
    a = (-0.5 / sig ** 2).astype(np.float32)
    a_widest = float(-0.5 / (1.4 * 1.5) ** 2)  # no sigma above 1.4 x 1.5
    W = (rng.standard_normal((H, D, K)) * 0.1).astype(np.float32)
    q = (rng.standard_normal((N, H, D)) * 0.5).astype(np.float32)
    k, v = (rng.standard_normal((N, H, D)).astype(np.float32) for _ in range(2))
    ops.set_weight_floor_log2(floor)
    try:
        out, lse, lists = sorted_forward(ops, cb, prep, q, k, v, a, W, cutoff, minimum, a_widest)
        again, lse2, _ = sorted_forward(ops, cb, prep, q, k, v, a, W, cutoff, minimum, a_widest)
        plain = ops.infinite_attn_fwd(dev(q), dev(k), dev(v), dev(a), prep["pos_ij"], dev(cb.trans_vec), prep["rvlen"],
                                      prep["batch"], prep["edges"], prep["row_start"], int(cb.sizes.max()), K, DIST_MAX,
                                      WSCALE, dev(W), cutoff, 2, minimum)
    finally:
        ops.set_weight_floor_log2(-30.0)
    assert torch.equal(out, again) and torch.equal(lse, lse2)  # one warp per row, fixed order: bitwise repeatable
    edges = oracle.edge_index(cb.sizes)
    pos_ij, _, _, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    z, psiW = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, K, DIST_MAX, WSCALE, W=W[None], rvlen=rvlen,
                                     cutoff_radius=cutoff, minimum_range=minimum, precision="f64")
    prob, ref = oracle.fused_attn_fwd(q, k, v, z, psiW, edges, precision="f64")
    assert rel_err(out.cpu().numpy(), ref) < TOL
    assert rel_err(out.cpu().numpy(), plain[0].cpu().numpy()) < 2e-5
    # lse = log sum_j exp(q.k + phi): from the oracle's phi
    logit = np.einsum("ehd,ehd->eh", q[edges[0]].astype(np.float64), k[edges[1]].astype(np.float64)) + z
    ref_lse = np.full((N, H), -np.inf)
    np.logaddexp.at(ref_lse, edges[0], logit)
    assert np.abs(lse.cpu().numpy() - ref_lse).max() < 1e-4 * max(1.0, np.abs(ref_lse).max())
    # how many rows took which kernel (the call's scheduling block is the last one)
    rowdir, _, sched, *_ = carve(lists, N, cb.num_edges)
    no_list = int((rowdir[:, 4] < 0).sum())
    assert int(sched[15, 1]) >= no_list
    if nmax <= 16 and floor > -100:
        assert no_list == 0


@pytest.mark.parametrize("nmax,Kb,cutoff,lengths", [(48, 64, -3.5, (4.0, 11.0)), (60, 64, -3.5, (4.0, 11.0)),
                                                    (64, 64, 0.0, (4.0, 11.0)), (20, 0, -3.5, (4.0, 11.0)),
                                                    (40, 0, -3.5, (4.0, 11.0)), (60, 0, 0.0, (4.0, 11.0)),
                                                    (56, 64, -3.5, (2.5, 4.5)), (56, 0, -3.5, (2.5, 4.5)),
                                                    (24, 0, -3.5, (2.5, 3.5))])
def test_sorted_rows_up_to_64_keys_and_without_basis(ops, nmax, Kb, cutoff, lengths):
    """Crystals of up to 64 atoms (four key tiles; a lane looks after two keys) and the variant without a radial basis
    (K = 0: no histogram, no projection), against the float64 oracle chain and the enumerating kernel.  The cases with
    cells of a few Angstrom have rows of more than 4096 entries, which are left over to the enumerating row kernel
    inside the same call (it enumerates phi edge by edge there: neither a phi kernel nor term lists serve those rows)."""
    cb = make_crystals(73, 8, uniform_atoms(max(1, nmax // 2), nmax), length_range=lengths)
    prep = prepare(ops, cb)
    N = cb.num_atoms
    rng = np.random.default_rng(73)
    sig = 1.4 * (0.6 + 0.9 * rng.random((N, H)))
    a = (-0.5 / sig ** 2).astype(np.float32)
    a_widest = float(-0.5 / (1.4 * 1.5) ** 2)
    W = (rng.standard_normal((H, D, 64)) * 0.1).astype(np.float32) if Kb else None
    q = (rng.standard_normal((N, H, D)) * 0.5).astype(np.float32)
    k, v = (rng.standard_normal((N, H, D)).astype(np.float32) for _ in range(2))
    tv, max_atoms = dev(cb.trans_vec), int(cb.sizes.max())
    assert max_atoms > 32 or Kb == 0
    lists = ops.row_list_build(prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"], prep["row_start"], max_atoms,
                               cutoff, 2, 2, a_widest)
    run = lambda: ops.infinite_attn_fwd_sorted(dev(q), dev(k), dev(v), dev(a), prep["pos_ij"], tv, prep["rvlen"], prep["batch"],
                                               prep["edges"], prep["row_start"], max_atoms, Kb, DIST_MAX, WSCALE,
                                               None if W is None else dev(W), cutoff, 2, 2, lists)
    out, lse = run()
    again, lse2 = run()
    assert torch.equal(out, again) and torch.equal(lse, lse2)
    plain = ops.infinite_attn_fwd(dev(q), dev(k), dev(v), dev(a), prep["pos_ij"], tv, prep["rvlen"], prep["batch"],
                                  prep["edges"], prep["row_start"], max_atoms, Kb, DIST_MAX, WSCALE,
                                  None if W is None else dev(W), cutoff, 2, 2)
    assert rel_err(out.cpu().numpy(), plain[0].cpu().numpy()) < 2e-5
    edges = oracle.edge_index(cb.sizes)
    pos_ij, _, _, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    z, psiW = oracle.lattice_sum_fwd(a, pos_ij, cb.trans_vec, cb.batch, edges, Kb, DIST_MAX, WSCALE,
                                     W=None if W is None else W[None], rvlen=rvlen, cutoff_radius=cutoff, minimum_range=2,
                                     precision="f64")
    prob, ref = oracle.fused_attn_fwd(q, k, v, z, psiW if Kb else None, edges, precision="f64")
    assert rel_err(out.cpu().numpy(), ref) < TOL
    logit = np.einsum("ehd,ehd->eh", q[edges[0]].astype(np.float64), k[edges[1]].astype(np.float64)) + z
    ref_lse = np.full((N, H), -np.inf)
    np.logaddexp.at(ref_lse, edges[0], logit)
    assert np.abs(lse.cpu().numpy() - ref_lse).max() < 1e-4 * max(1.0, np.abs(ref_lse).max())
    # rows computed by the enumerating kernel: those without a list (more than 4096 entries)
    rowdir, _, sched, *_ = carve(lists, N, cb.num_edges)
    no_list = int((rowdir[:, 4] < 0).sum())
    assert int(sched[15, 1]) >= no_list
    assert (no_list > 0) == (lengths[1] < 5.0)


def test_row_lists_are_sorted_and_complete(ops):
    """Structure of the lists: every row's entries ascend in d2, keys are the row's keys, the per-edge minimum is the
    smallest listed d2 of the edge, and the entries of a row are exactly the entries of its edges' term lists."""
    cb = make_crystals(7, 12, uniform_atoms(2, 14), length_range=(3.0, 10.0))
    prep = prepare(ops, cb)
    N, E = cb.num_atoms, cb.num_edges
    a_widest = float(-0.5 * 0.5 / 1.4 ** 2)
    tv, max_atoms = dev(cb.trans_vec), int(cb.sizes.max())
    order = torch.randperm(N, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3)).to(torch.int32)
    work = ops.row_list_build(prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"], prep["row_start"], max_atoms,
                              -3.5, 2, 2, a_widest, row_order=order)
    term, _ = ops.term_list_build(prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"], prep["row_start"],
                                  max_atoms, -3.5, 2, 2, a_widest)
    torch.cuda.synchronize()
    rowdir, dmin, sched, _, cursor, pool, tasks, task_count = (t.cpu() for t in carve(work, N, E))
    t_count = term[4 * E:8 * E].view(torch.int32).cpu().numpy()  # directory of the term lists: start, count, dmin
    t_dmin = term[8 * E:12 * E].view(torch.float32).cpu().numpy()
    row_start = prep["row_start"].cpu().numpy()
    assert int(sched.abs().sum()) == 0
    seen = listed = 0
    for slot in range(N):
        i, a0, n, c, start, chunks, e0, _ = (int(x) for x in rowdir[slot])
        assert i == int(order[slot]) and e0 == row_start[i] and n == row_start[i + 1] - row_start[i] and c == cb.batch[i]
        if start < 0:  # a row of more than 4096 entries (a nearly flat cell): left to the enumerating kernel
            continue
        listed += 1
        assert start % 8 == 0
        ent = pool[start:start + 8 * chunks]
        d2 = ent[:, 0].numpy()
        key = ent[:, 1].contiguous().view(torch.int32).numpy()
        real = key != 0x7f7f7f00
        total = int(real.sum())
        assert real[:total].all() and 8 * (chunks - 1) < total <= 8 * chunks
        assert (np.diff(d2) >= 0).all()
        j = key[:total] & 255
        assert (j < n).all()
        assert total == t_count[e0:e0 + n].sum()
        for jj in range(n):
            assert dmin[e0 + jj] == d2[:total][j == jj].min() == t_dmin[e0 + jj]
        seen += 8 * chunks
    assert int(cursor[0]) == seen and listed >= N // 2
    # the two task lists partition the rows: long lists (shared by a block's warps) and the rest
    n_shared, n_single = int(task_count[0]), int(task_count[1])
    assert n_shared + n_single == N
    shared, single = tasks[0, :n_shared].numpy(), tasks[1, :n_single].numpy()
    assert sorted(np.concatenate([shared, single]).tolist()) == list(range(N))
    assert (rowdir[shared, 5] > 64).all() and ((rowdir[single, 5] <= 64) | (rowdir[single, 4] < 0)).all()


def test_sorted_rows_at_bench_size_match_the_listed_kernel(ops):
    """The 128-crystal batch of the headline configuration: row lists against term lists (two organisations of the
    same set of terms) and against the float32 oracle on a sample of crystals."""
    cb = make_config("cfg0")
    prep = prepare(ops, cb)
    N, E = cb.num_atoms, cb.num_edges
    rng = np.random.default_rng(0)
    func = 0.5 + rng.random((N, H)) * 1.5                      # the positive function's range at default settings
    a = (func * (-0.5 / 1.4 ** 2)).astype(np.float32)
    a_widest = float(0.5 * -0.5 / 1.4 ** 2)
    W = (rng.standard_normal((H, D, K)) * 0.1).astype(np.float32)
    q = (rng.standard_normal((N, H, D)) * 0.3).astype(np.float32)
    k, v = (rng.standard_normal((N, H, D)).astype(np.float32) for _ in range(2))
    tv, max_atoms = dev(cb.trans_vec), int(cb.sizes.max())
    out, lse, lists = sorted_forward(ops, cb, prep, q, k, v, a, W, -3.5, 2, a_widest)
    term = ops.term_list_build(prep["pos_ij"], tv, prep["rvlen"], prep["batch"], prep["edges"], prep["row_start"], max_atoms,
                               -3.5, 2, 2, a_widest)
    listed = ops.infinite_attn_fwd(dev(q), dev(k), dev(v), dev(a), prep["pos_ij"], tv, prep["rvlen"], prep["batch"],
                                   prep["edges"], prep["row_start"], max_atoms, K, DIST_MAX, WSCALE, dev(W), -3.5, 2, 2,
                                   term_lists=term)
    assert rel_err(out.cpu().numpy(), listed[0].cpu().numpy()) < 2e-5
    assert np.abs((lse - listed[2]).cpu().numpy()).max() < 2e-5
    rowdir, _, sched, _, _, _, _, task_count = carve(lists, N, E)
    assert int(task_count[0]) + int(task_count[1]) == N and int(task_count[0]) > 0 and int(sched[15, 1]) == 0
    sample = cb.select(range(12))
    n_s = sample.num_atoms
    edges = oracle.edge_index(sample.sizes)
    pos_ij, _, _, rvlen = oracle.geometry(sample.pos, sample.trans_vec, edges)
    z, psiW = oracle.lattice_sum_fwd(a[:n_s], pos_ij, sample.trans_vec, sample.batch, edges, K, DIST_MAX, WSCALE, W=W[None],
                                     rvlen=rvlen, cutoff_radius=-3.5, minimum_range=2, precision="f64")
    _, ref = oracle.fused_attn_fwd(q[:n_s], k[:n_s], v[:n_s], z, psiW, edges, precision="f64")
    assert rel_err(out[:n_s].cpu().numpy(), ref) < TOL
