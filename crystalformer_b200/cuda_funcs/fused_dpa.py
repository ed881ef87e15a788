"""``FusedDotProductAttentionCUDA`` with the reference's interface (models/cuda_funcs/fused_dpa.py:17-208)."""
import torch

from ._common import ops, row_starts


class FusedDotProductAttentionCUDA(torch.autograd.Function):
    @staticmethod
    def forward(ctx, que_ihk, key_ihk, val_ihk, aij_eh, bij_ehk, batch_i, edge_ij_e):
        # que/key/val (points, heads, head_dim), que already divided by sqrt(head_dim); aij (edges, heads) or None;
        # bij (edges, heads, head_dim) or None
        N = que_ihk.shape[0]
        e_start_i = row_starts(edge_ij_e, N)
        que_ihk, key_ihk, val_ihk = (t.contiguous().detach() for t in (que_ihk, key_ihk, val_ihk))
        aij_eh = aij_eh.contiguous().detach() if aij_eh is not None else None
        bij_ehk = bij_ehk.contiguous().detach() if bij_ehk is not None else None
        edge_ij_e = edge_ij_e.contiguous()
        prob_eh, output = ops.fused_attn_fwd(que_ihk, key_ihk, val_ihk, aij_eh, bij_ehk, edge_ij_e, e_start_i)
        ctx.save_for_backward(que_ihk, key_ihk, val_ihk, bij_ehk, edge_ij_e, e_start_i, prob_eh, output)
        ctx.has_aij = aij_eh is not None
        return output

    @staticmethod
    def backward(ctx, go_ihk):
        que_ihk, key_ihk, val_ihk, bij_ehk, edge_ij_e, e_start_i, prob_eh, output = ctx.saved_tensors
        gque, gkey, gval, gaij, gbij = ops.fused_attn_bwd(
            que_ihk, key_ihk, val_ihk, bij_ehk, edge_ij_e, e_start_i, prob_eh, output, go_ihk.contiguous().detach())
        return gque, gkey, gval, (gaij if ctx.has_aij else None), gbij, None, None
