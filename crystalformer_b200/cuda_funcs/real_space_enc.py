"""``RealPeriodicEncodingFuncCUDA`` with the reference's interface (models/cuda_funcs/real_space_enc.py:17-247):
phi (E,H) and psi (E,H,K); when ``W_k`` is given the projection W psi is done outside the kernel, as in the reference
(:116-121), and its gradient is the per-edge outer product (:191)."""
import torch

from ._common import ops, row_starts
from .kernel_manager import KernelManager


class RealPeriodicEncodingFuncCUDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a_ik, rpos_ij_e, dist2_min_e, tvecs_n, batch_i, edge_ij_e, K, dist_max, wscale, W_k,
                rvlen_n=None, cutoff_radius=None):
        a_ik = a_ik.contiguous().detach()
        E, H = edge_ij_e.shape[1], a_ik.shape[1]
        cutoff = float(cutoff_radius) if (cutoff_radius is not None and rvlen_n is not None) else 0.0
        z_ek, v_ekd = ops.lattice_sum_fwd(
            a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, int(K), float(dist_max), float(wscale), W=None, rvlen=rvlen_n,
            cutoff_radius=cutoff, lattice_range=KernelManager.LATTICE_RANGE, minimum_range=KernelManager.MINIMUM_RANGE)
        if W_k is not None and K > 0:
            W_k = W_k.detach().contiguous()
            assert W_k.dim() in (3, 4)
            W_num = 1 if W_k.dim() == 3 else W_k.shape[0]
            assert W_num in (E, 1)
            v_out = (W_k @ v_ekd[..., None]).reshape(E, H, -1)
        else:
            W_k = None
            v_out, v_ekd = v_ekd, None
        ctx.save_for_backward(a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, W_k, z_ek, v_ekd)
        ctx.K, ctx.dist_max, ctx.wscale, ctx.cutoff = int(K), float(dist_max), float(wscale), cutoff
        ctx.n_inputs = 10 if rvlen_n is None else 12
        ctx.box = (KernelManager.LATTICE_RANGE, KernelManager.MINIMUM_RANGE)
        if K <= 0:
            return z_ek,
        return z_ek, v_out

    @staticmethod
    def backward(ctx, gz_ek, gv_ekd=None):
        a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, rvlen_n, W_k, z_ek, v_ekd = ctx.saved_tensors
        N = a_ik.shape[0]
        e_start_i = row_starts(edge_ij_e, N)
        gW_k = None
        if ctx.K > 0:
            if gv_ekd is None:
                gv_ekd = torch.zeros(z_ek.shape + (ctx.K if W_k is None else W_k.shape[-2],), dtype=z_ek.dtype,
                                     device=z_ek.device)
            if W_k is not None:
                gW_k = gv_ekd[..., :, None] * v_ekd[..., None, :]          # (E,H,Dv,K); autograd sums it to W's shape
                gv_ekd = (W_k.transpose(-1, -2) @ gv_ekd[..., None]).squeeze(-1)
            gv_ekd = gv_ekd.contiguous()
        ga_ik, _ = ops.lattice_sum_bwd(
            a_ik, rpos_ij_e, tvecs_n, batch_i, edge_ij_e, e_start_i, z_ek, gz_ek.contiguous(), gv_ekd, ctx.K,
            ctx.dist_max, ctx.wscale, W=None, rvlen=rvlen_n, cutoff_radius=ctx.cutoff, lattice_range=ctx.box[0],
            minimum_range=ctx.box[1])
        if gW_k is not None and W_k.shape[0] == 1 and W_k.dim() == 4:
            gW_k = gW_k.sum(dim=0, keepdim=True)
        elif gW_k is not None and W_k.dim() == 3:
            gW_k = gW_k.sum(dim=0)
        grads = [ga_ik, None, None, None, None, None, None, None, None, gW_k, None, None]
        return tuple(grads[:ctx.n_inputs])
