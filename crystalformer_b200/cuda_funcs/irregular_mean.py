"""``IrregularMeanCUDA`` with the reference's interface (models/cuda_funcs/irregular_mean.py:19-69): deterministic
per-crystal mean of atom features; the backward is the plain broadcast division the reference uses (:60-69)."""
import torch

from ._common import ops


class IrregularMeanCUDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_ik, batch_i, sizes):
        dev = x_ik.device
        if sizes is None:
            B = int(batch_i.max().item()) + 1
            sizes = torch.zeros(B, dtype=torch.long, device=dev)
            sizes.scatter_add_(0, batch_i, torch.ones(batch_i.shape, dtype=torch.long, device=dev))
        start_n = torch.constant_pad_nd(torch.cumsum(sizes, 0), (1, 0)).contiguous()
        o_nk = ops.segment_mean(x_ik.contiguous().detach(), start_n)
        ctx.save_for_backward(batch_i, sizes)
        return o_nk

    @staticmethod
    def backward(ctx, go_nk):
        batch_i, sizes = ctx.saved_tensors
        shape = [go_nk.shape[0]] + [1 for _ in go_nk.shape[1:]]
        gx_ik = (go_nk / sizes.reshape(shape).float())[batch_i]
        return gx_ik, None, None
