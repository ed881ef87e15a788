"""The drop-in autograd functions and module options around the kernels, on the GPU:
``RealPeriodicEncodingFuncCUDA`` (the reference's non-projecting wrapper, models/cuda_funcs/real_space_enc.py:17-247,
including its projection outside the kernel and the per-edge gradient of W), the per-batch edge cache of the attention
module, and a value projection shared by the heads (value_pe_headed = False)."""
import types

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


def dev(x):
    return None if x is None else torch.as_tensor(np.ascontiguousarray(x)).cuda()


@pytest.mark.parametrize("project,adaptive", [(False, True), (True, True), (True, False)])
def test_real_periodic_encoding_function(project, adaptive):
    """apply(a, pos_ij, None, tvecs, batch, edges, K, dist_max, wscale, W[, rvlen, cutoff]) -> (phi, psi or W psi) and
    its gradients with respect to a and W, against the float64 oracle of the reference's kernels."""
    from crystalformer_b200.cuda_funcs import KernelManager, RealPeriodicEncodingFuncCUDA, compile_kernels
    compile_kernels(2, H, D, K, D, True)
    cb = make_crystals(33, 6, uniform_atoms(1, 7), length_range=(2.5, 8.0))
    edges = oracle.edge_index(cb.sizes)
    pos_ij, _, _, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    rng = np.random.default_rng(33)
    N, E = cb.num_atoms, edges.shape[1]
    a_np = (-0.5 / (1.4 * (0.6 + 0.9 * rng.random((N, H)))) ** 2).astype(np.float32)
    W_np = (rng.standard_normal((1, H, D, K)) * 0.1).astype(np.float32) if project else None
    a = dev(a_np).requires_grad_(True)
    W = dev(W_np).requires_grad_(True) if project else None
    extra = (dev(rvlen), -3.5) if adaptive else ()
    z, v = RealPeriodicEncodingFuncCUDA.apply(a, dev(pos_ij), None, dev(cb.trans_vec), dev(cb.batch), dev(edges), K,
                                              DIST_MAX, WSCALE, W, *extra)
    gz = rng.standard_normal((E, H)).astype(np.float32)
    gv = rng.standard_normal(tuple(v.shape)).astype(np.float32)
    ((z * dev(gz)).sum() + (v * dev(gv)).sum()).backward()
    kw = dict(rvlen=rvlen if adaptive else None, cutoff_radius=-3.5 if adaptive else 0.0, lattice_range=2, minimum_range=2,
              precision="f64")
    zr, vr = oracle.lattice_sum_fwd(a_np, pos_ij, cb.trans_vec, cb.batch, edges, K, DIST_MAX, WSCALE, W=W_np, **kw)
    ra, rW = oracle.lattice_sum_bwd(a_np, pos_ij, cb.trans_vec, cb.batch, edges, zr, gz, gv, K, DIST_MAX, WSCALE, W=W_np, **kw)
    assert rel_err(z.detach().cpu().numpy(), zr) < TOL and rel_err(v.detach().cpu().numpy(), vr) < TOL
    assert rel_err(a.grad.cpu().numpy(), ra) < TOL
    if project:
        assert W.grad.shape == W.shape and rel_err(W.grad.cpu().numpy(), np.asarray(rW).reshape(W_np.shape)) < TOL
    assert KernelManager.LATTICE_RANGE == 2


def test_edge_cache_does_not_confuse_batches_with_equal_edge_counts():
    """Two batches with the same E = sum n^2 but other crystal sizes ([2,3] and [3,2]): when the first edge tensor is
    freed the allocator may give the second one the same address; the cached CSR offsets must not be handed to it."""
    from crystalformer_b200.attention import edge_info
    def edges_of(sizes):
        return dev(oracle.edge_index(np.asarray(sizes, dtype=np.int64)))
    e1 = edges_of([2, 3])
    ptr = e1.data_ptr()
    row1, max1, _ = edge_info(e1, 5)
    assert row1.cpu().tolist() == [0, 2, 4, 7, 10, 13] and max1 == 3
    del e1  # (the cache entry keeps the tensor alive, so the address cannot come back while the entry exists)
    e2 = edges_of([3, 2])
    row2, max2, _ = edge_info(e2, 5)
    assert row2.cpu().tolist() == [0, 3, 6, 9, 11, 13] and max2 == 3
    assert e2.data_ptr() != ptr


def test_value_projection_shared_by_the_heads():
    """value_pe_headed = False: pe_dist_proj is (1, 1, Dv, K); the kernels get one view of it per head.  Forward
    (one-call inference path and module path) and the gradient of the shared matrix against a model whose per-head
    projection holds eight copies of it."""
    from crystalformer_b200.model import Latticeformer, default_params
    cb = make_crystals(44, 5, uniform_atoms(2, 8), length_range=(3.0, 9.0))
    t = lambda x: dev(x)
    data = types.SimpleNamespace(x=t(cb.x), pos=t(cb.pos), batch=t(cb.batch), trans_vec=t(cb.trans_vec), sizes=t(cb.sizes))
    torch.manual_seed(4)
    shared = Latticeformer(default_params(num_layers=2, value_pe_headed=False)).cuda()
    torch.manual_seed(4)
    headed = Latticeformer(default_params(num_layers=2, value_pe_headed=True)).cuda()
    state = shared.state_dict()
    for key, val in list(state.items()):
        if key.endswith("pe_dist_proj"):
            assert tuple(val.shape) == (1, 1, D, K)
            state[key] = val.expand(1, H, D, K).clone()
    headed.load_state_dict(state)
    for m in (shared, headed):
        m.train()
        with torch.no_grad():
            m(data)  # fixes gauss_scale
    headed.load_state_dict({**headed.state_dict(), **{k: v for k, v in shared.state_dict().items() if "gauss_scale" in k}})
    shared.eval(); headed.eval()
    with torch.no_grad():
        y_shared, y_headed = shared(data), headed(data)
    assert rel_err(y_shared.cpu().numpy(), y_headed.cpu().numpy()) < 1e-5
    shared.train(); headed.train()
    shared(data).sum().backward()
    headed(data).sum().backward()
    g_shared = shared.encoder.layers[0].self_attn.pe_dist_proj.grad
    g_headed = headed.encoder.layers[0].self_attn.pe_dist_proj.grad
    assert tuple(g_shared.shape) == (1, 1, D, K)
    assert rel_err(g_shared.cpu().numpy(), g_headed.sum(dim=1, keepdim=True).cpu().numpy()) < 1e-4
