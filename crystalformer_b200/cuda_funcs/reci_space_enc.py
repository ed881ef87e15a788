"""``ReciPeriodicEncodingFuncCUDA`` with the reference's interface (models/cuda_funcs/reci_space_enc.py:17-99):
``apply(a_ik, kr_base_e, rvecs_n, vcell_n, batch_i, edge_ij_e) -> z_ek`` (E,H), the log of the reciprocal-space
lattice sum plus the normalisation 1.5 log(-4 pi a) - log V.  The gradient reaches ``a_ik`` only and, as in the
reference's kernel, does not include the derivative of the normalisation term."""
import torch

from ._common import ops, row_starts
from .kernel_manager import KernelManager


class ReciPeriodicEncodingFuncCUDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a_ik, kr_base_e, rvecs_n, vcell_n, batch_i, edge_ij_e):
        a_ik = a_ik.contiguous().detach()
        N, E = a_ik.shape[0], edge_ij_e.shape[1]
        e_start_i = row_starts(edge_ij_e, N)
        z_ek, sumexp_ek = ops.reci_sum_fwd(a_ik, kr_base_e, rvecs_n, vcell_n, batch_i, e_start_i, E,
                                           KernelManager.LATTICE_RANGE)
        ctx.save_for_backward(a_ik, kr_base_e, rvecs_n, batch_i, e_start_i, sumexp_ek)
        ctx.lattice_range = KernelManager.LATTICE_RANGE
        return z_ek

    @staticmethod
    def backward(ctx, gz_ek):
        a_ik, kr_base_e, rvecs_n, batch_i, e_start_i, sumexp_ek = ctx.saved_tensors
        ga_ik = ops.reci_sum_bwd(a_ik, kr_base_e, rvecs_n, batch_i, e_start_i, gz_ek.detach().contiguous(), sumexp_ek,
                                 ctx.lattice_range)
        return ga_ik, None, None, None, None, None
