"""The scratch-free variant of the lattice-sum backward (cf_lattice_sum_bwd_static), called through the C ABI.

Some callers of the library cannot allocate device memory at call time (all their memory was budgeted at start-up,
or they bind the library from a runtime without a device allocator, or an allocation would stall a latency-critical
loop).  For them the per-edge scratch of the backward is an array inside the library image.  This file checks that the
variant returns what the ordinary entry point returns - on two calls in a row with different inputs, because the
array is shared by all calls and keeps the previous call's contents - and that oversized calls are refused.
The file name sorts last so that a run stopping at the first failure has already run every other test."""
import ctypes
from ctypes import c_double, c_int, c_int64, c_void_p

import numpy as np
import pytest
import torch

import oracle
from crystalformer_b200.synthetic import make_crystals, uniform_atoms

pytestmark = pytest.mark.gpu

H, K = 8, 64
DIST_MAX, WSCALE = 14.0, 1.0


def dev(x):
    return torch.as_tensor(np.ascontiguousarray(x)).cuda()


def ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


def make_case(seed, crystals, nmax):
    cb = make_crystals(seed, crystals, uniform_atoms(1, nmax), length_range=(2.5, 9.0))
    edges = oracle.edge_index(cb.sizes)
    pos_ij, _, _, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    rng = np.random.default_rng(seed)
    N, E = cb.num_atoms, edges.shape[1]
    a = (-0.5 / (1.4 * (0.6 + 0.9 * rng.random((N, H)))) ** 2).astype(np.float32)
    t = dict(a=dev(a), pos_ij=dev(pos_ij), tvecs=dev(cb.trans_vec), batch=dev(cb.batch), edges=dev(edges),
             row_start=dev(oracle.row_starts(edges, N)), rvlen=dev(rvlen),
             gz=dev(rng.standard_normal((E, H)).astype(np.float32)),
             gpsi=dev(rng.standard_normal((E, H, K)).astype(np.float32)))
    return N, E, t


def run_both(ops, _lib, N, E, t):
    z, _ = ops.lattice_sum_fwd(t["a"], t["pos_ij"], t["tvecs"], t["batch"], t["edges"], K, DIST_MAX, WSCALE,
                               rvlen=t["rvlen"], cutoff_radius=-3.5)
    ga_ref, _ = ops.lattice_sum_bwd(t["a"], t["pos_ij"], t["tvecs"], t["batch"], t["edges"], t["row_start"], z, t["gz"],
                                    t["gpsi"], K, DIST_MAX, WSCALE, rvlen=t["rvlen"], cutoff_radius=-3.5)
    ga = torch.full((N, H), float("nan"), device="cuda")
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.call("cf_lattice_sum_bwd_static", ptr(t["a"]), ptr(t["pos_ij"]), ptr(t["tvecs"]), ptr(t["batch"]), ptr(t["edges"]),
              ptr(t["row_start"]), ptr(z), ptr(t["gz"]), ptr(t["gpsi"]), c_int64(N), c_int64(H), c_int64(E), c_int64(K),
              c_double(DIST_MAX), c_double(WSCALE), ptr(t["rvlen"]), c_double(-3.5), c_int(2), c_int(2), ptr(ga), ptr(None),
              stream)
    torch.cuda.synchronize()
    return ga, ga_ref, z


def test_static_scratch_variant_matches_the_ordinary_entry_point_twice_in_a_row():
    from crystalformer_b200 import _lib, ops
    for seed, crystals, nmax in ((91, 12, 9), (92, 5, 6)):  # the second call is smaller: stale contents stay behind it
        N, E, t = make_case(seed, crystals, nmax)
        ga, ga_ref, z = run_both(ops, _lib, N, E, t)
        assert torch.isfinite(ga).all()
        err = float((ga - ga_ref).abs().max() / ga_ref.abs().max())
        assert err < 1e-4, err  # the tolerance of the other fp32 parity tests; in practice the bits are equal
        # ... and against the float64 CPU oracle of the reference's backward kernel (real_enc_bwd.cu)
        c = lambda x: x.cpu().numpy()
        ga_cpu, _ = oracle.lattice_sum_bwd(c(t["a"]), c(t["pos_ij"]), c(t["tvecs"]), c(t["batch"]), c(t["edges"]), c(z),
                                           c(t["gz"]), c(t["gpsi"]), K, DIST_MAX, WSCALE, rvlen=c(t["rvlen"]),
                                           cutoff_radius=-3.5, lattice_range=2, minimum_range=2, precision="f64")
        assert float(np.abs(c(ga) - ga_cpu).max() / np.abs(ga_cpu).max()) < 1e-4


def test_static_scratch_variant_refuses_too_many_edges():
    from crystalformer_b200 import _lib
    null = c_void_p(0)
    with pytest.raises(_lib.CrystalformerB200Error) as e:
        _lib.call("cf_lattice_sum_bwd_static", null, null, null, null, null, null, null, null, null, c_int64(10), c_int64(8),
                  c_int64(262144 + 1), c_int64(64), c_double(14.0), c_double(1.0), null, c_double(0.0), c_int(2), c_int(2),
                  null, null, null)
    assert e.value.code == -4 and "exceeds the built-in scratch" in str(e.value)
