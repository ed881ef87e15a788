"""Placeholder for the reference's ``ReciPeriodicEncodingFuncCUDA`` (models/cuda_funcs/reci_space_enc.py:17-99).

The reciprocal-space (Fourier) lattice sum serves the ``reci`` / ``multihead`` / ``real-reci`` domains only; the
real-space path this library accelerates does not use it.  The name is exported because the reference's attention
module imports it; calling it raises."""
import torch


class ReciPeriodicEncodingFuncCUDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, *args):
        raise NotImplementedError(
            "crystalformer_b200 implements the real-space domain only (domain='real'); the reciprocal-space "
            "encoding is not part of the accelerated path")

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError
