"""Helpers shared by the autograd wrappers."""
import torch

from .. import ops


def row_starts(edge_ij_e: torch.Tensor, N: int) -> torch.Tensor:
    """CSR offsets of the edge list by source atom, built as the reference does (models/cuda_funcs/fused_dpa.py:24-26):
    a scatter-add of int64 ones followed by a cumulative sum; deterministic and synchronisation-free."""
    e_start_i = torch.zeros(N + 1, dtype=torch.int64, device=edge_ij_e.device)
    e_start_i.scatter_add_(0, edge_ij_e[0] + 1, torch.ones_like(edge_ij_e[0]))
    return e_start_i.cumsum(0)


__all__ = ["ops", "row_starts"]
