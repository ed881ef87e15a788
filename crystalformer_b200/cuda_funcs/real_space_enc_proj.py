"""``RealPeriodicEncodingWithProjFuncCUDA`` with the reference's interface
(models/cuda_funcs/real_space_enc_proj.py:18-178): phi (E,H) and W psi (E,H,Dv), gradients for ``a_ik`` and ``W_k``."""
import torch

from ._common import ops, row_starts
from .kernel_manager import KernelManager


class RealPeriodicEncodingWithProjFuncCUDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale, W_k,
                rvlen_n=None, cutoff_radius=None):
        # a_ik (points, heads); rpos_ij_e (edges, 3); tvecs_n (batch, 3, 3); batch_i (points); edge_ij_e (2, edges)
        # dist2_min_e is accepted for signature compatibility and ignored, as the reference kernels ignore it
        # (models/kernels/real_enc_proj_fwd.cu:91 `if (1 || ...)`).
        a_ik = a_ik.contiguous().detach()
        if W_k is not None:
            assert W_k.dim() in (3, 4)
            W_k = W_k.detach().contiguous()
        cutoff = float(cutoff_radius) if (cutoff_radius is not None and rvlen_n is not None) else 0.0
        z_ek, v_ekd = ops.lattice_sum_fwd(
            a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, int(K), float(dist_max), float(wscale), W=W_k, rvlen=rvlen_n,
            cutoff_radius=cutoff, lattice_range=KernelManager.LATTICE_RANGE, minimum_range=KernelManager.MINIMUM_RANGE)
        ctx.save_for_backward(a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, W_k, z_ek)
        ctx.K, ctx.dist_max, ctx.wscale, ctx.cutoff = int(K), float(dist_max), float(wscale), cutoff
        ctx.n_inputs = 10 if rvlen_n is None else 12
        ctx.box = (KernelManager.LATTICE_RANGE, KernelManager.MINIMUM_RANGE)
        if K <= 0:
            return z_ek,
        return z_ek, v_ekd

    @staticmethod
    def backward(ctx, gz_ek, gv_ekd=None):
        a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, W_k, z_ek = ctx.saved_tensors
        N = a_ik.shape[0]
        e_start_i = row_starts(edge_ij_e, N)
        gz_ek = gz_ek.contiguous()
        if ctx.K > 0:
            gv_ekd = torch.zeros(z_ek.shape + ((W_k.shape[-2] if W_k is not None else ctx.K),), dtype=z_ek.dtype,
                                 device=z_ek.device) if gv_ekd is None else gv_ekd.contiguous()
        ga_ik, gW_k = ops.lattice_sum_bwd(
            a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, e_start_i, z_ek, gz_ek, gv_ekd, ctx.K, ctx.dist_max, ctx.wscale,
            W=W_k, rvlen=rvlen_n, cutoff_radius=ctx.cutoff, lattice_range=ctx.box[0], minimum_range=ctx.box[1])
        if gW_k is not None and W_k.dim() == 3:
            gW_k = gW_k[0]
        grads = [ga_ik, None, None, None, None, None, None, None, None, gW_k, None, None]
        return tuple(grads[:ctx.n_inputs])
