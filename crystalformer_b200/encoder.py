"""Encoder stack with the reference's interface (models/indexed_latticeformer_encoder.py:620-890):
``CrystalformerEncoderCUDA(d_model, nhead, num_encoder_layers, dim_feedforward, ...).forward(src, pos, batch, trans,
sizes, onehot=None)`` and ``CrystalformerEncoderLayerCUDA``.  Parameter names, post-norm layout, T-Fixup scaling and
the feed-forward block are the reference's; the batch geometry (all-pairs edge list, CSR offsets, relative positions,
reciprocal lattice) is built by one device-side call instead of the reference's host loop over crystals
(``get_edge_index`` :15-32 and ``compute_lattice_distances_for_cuda`` :183-253)."""
from __future__ import annotations

from typing import Callable, Optional, Union

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Dropout, Identity, LayerNorm, Linear, Module, ModuleList
from torch.nn.init import constant_, xavier_uniform_

from . import ops
from .attention import CrystalformerMultiheadAttentionCUDA, register_edge_info
from .cuda_funcs import compile_kernels
from .params import LatticeformerParams


def _get_activation_fn(activation):
    if activation == "relu":
        return F.relu
    if activation == "gelu":
        return F.gelu
    raise RuntimeError("activation should be relu/gelu, not {}".format(activation))


class BatchGeometry:
    """Everything the attention layers need besides the atom features, computed once per batch on the device."""

    def __init__(self, pos: Tensor, trans: Tensor, sizes: Tensor, num_atoms: Optional[int] = None,
                 num_edges: Optional[int] = None, max_atoms: Optional[int] = None):
        sizes = sizes.to(device=pos.device, dtype=torch.int64)
        if num_atoms is None or num_edges is None or max_atoms is None:
            host = sizes.tolist()  # the one device->host read per batch (the reference does the same, :201)
            num_atoms, num_edges, max_atoms = sum(host), sum(n * n for n in host), max(host) if host else 1
        self.atom_start, self.edge_start = ops.crystal_offsets(sizes)
        prep = ops.batch_prepare(pos.float(), trans.float(), sizes, self.atom_start, self.edge_start, num_atoms, num_edges)
        self.batch, self.edges, self.row_start = prep["batch"], prep["edges"], prep["row_start"]
        self.pos_ij, self.rvecs, self.vcell, self.rvlen = prep["pos_ij"], prep["rvecs"], prep["vcell"], prep["rvlen"]
        self.sizes, self.max_atoms = sizes, int(max_atoms)
        register_edge_info(self.edges, self.row_start, self.max_atoms)


class CrystalformerEncoderLayerCUDA(Module):
    __constants__ = ["norm_first"]

    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1,
                 activation: Union[str, Callable[[Tensor], Tensor]] = F.relu, layer_norm_eps: float = 1e-5,
                 norm_first: bool = False, no_layer_norm=False, params=LatticeformerParams(), k_dim=0, v_dim=0,
                 device=None, dtype=None) -> None:
        assert params.domain in ("real",), "crystalformer_b200 implements the real-space domain only"
        self.domain = params.domain
        super().__init__()
        self.self_attn = CrystalformerMultiheadAttentionCUDA(d_model, nhead, dropout=dropout, kdim=k_dim, vdim=v_dim,
                                                             params=params)
        self.linear1 = Linear(d_model, dim_feedforward)
        self.dropout = Dropout(dropout) if dropout > 0 else Identity()
        self.linear2 = Linear(dim_feedforward, d_model)
        self.norm_first = norm_first
        self.norm1 = LayerNorm(d_model, eps=layer_norm_eps) if not no_layer_norm else Identity()
        self.norm2 = LayerNorm(d_model, eps=layer_norm_eps) if not no_layer_norm else Identity()
        self.dropout1 = Dropout(dropout) if dropout > 0 else Identity()
        self.dropout2 = Dropout(dropout) if dropout > 0 else Identity()
        self.activation = _get_activation_fn(activation) if isinstance(activation, str) else activation
        self._reset_parameters()

    def _reset_parameters(self):
        xavier_uniform_(self.linear1.weight)
        xavier_uniform_(self.linear2.weight)
        constant_(self.linear1.bias, 0)
        constant_(self.linear2.bias, 0)

    def fixup_initialization(self, num_layers):
        """T-Fixup: scale four weight matrices by 0.67 L^(-1/4) (models/indexed_latticeformer_encoder.py:818-835)."""
        scale = 0.67 * (num_layers) ** (-1. / 4.)
        with torch.no_grad():
            for name in ("linear1.weight", "linear2.weight", "self_attn.out_proj.weight", "self_attn.v_proj_weight"):
                self.get_parameter(name).mul_(scale)

    def forward(self, src: Tensor, batch: Tensor, edges: Tensor, pos_ij: Tensor = None, dist2_min: Tensor = None,
                trans: Tensor = None, kr_base: Tensor = None, rvecs: Tensor = None, vcell: Tensor = None,
                onehot: Tensor = None, rvlen: Tensor = None) -> Tensor:
        assert pos_ij is not None and trans is not None
        x = src
        if self.norm_first:
            x = x + self._sa_block(self.norm1(x), batch, edges, pos_ij, dist2_min, trans, kr_base, rvecs, vcell, onehot, rvlen)
            x = x + self._ff_block(self.norm2(x))
        else:
            x = self.norm1(x + self._sa_block(x, batch, edges, pos_ij, dist2_min, trans, kr_base, rvecs, vcell, onehot, rvlen))
            x = self.norm2(x + self._ff_block(x))
        return x

    def _sa_block(self, x, batch, edges, pos_ij, dist2_min, trans, kr_base, rvecs, vcell, onehot, rvlen):
        x = self.self_attn(x, x, x, batch, batch, edges, pos_ij, dist2_min, trans, kr_base, rvecs, vcell, onehot,
                           need_weights=False, rvlen=rvlen)[0]
        return self.dropout1(x)

    def _ff_block(self, x: Tensor) -> Tensor:
        x = self.linear2(self.dropout(self.activation(self.linear1(x))))
        return self.dropout2(x)


class CrystalformerEncoderCUDA(Module):
    def __init__(self, d_model: int = 512, nhead: int = 8, num_encoder_layers: int = 6, dim_feedforward: int = 2048,
                 dropout: float = 0.1, activation: Union[str, Callable[[Tensor], Tensor]] = F.relu,
                 layer_norm_eps: float = 1e-5, norm_first: bool = False, t_fixup_init=False, no_layer_norm=False,
                 lattice_params: LatticeformerParams = LatticeformerParams(), k_dim=0, v_dim=0, device=None,
                 dtype=None) -> None:
        super().__init__()
        assert lattice_params.domain in ("real",), "crystalformer_b200 implements the real-space domain only"
        self.lattice_params = lattice_params
        self.layers = ModuleList([
            CrystalformerEncoderLayerCUDA(d_model, nhead, dim_feedforward, dropout, activation, layer_norm_eps, norm_first,
                                          no_layer_norm, params=lattice_params.getLayerParameters(i), k_dim=k_dim,
                                          v_dim=v_dim)
            for i in range(num_encoder_layers)])
        if t_fixup_init:
            for layer in self.layers:
                layer.fixup_initialization(num_encoder_layers)
        self.num_layers = num_encoder_layers
        self.norm = LayerNorm(d_model, eps=layer_norm_eps) if not no_layer_norm else None
        self.d_model = d_model
        self.nhead = nhead
        v_head_dim = v_dim if v_dim > 0 else d_model // nhead
        k_head_dim = k_dim if k_dim > 0 else d_model // nhead
        compile_kernels(lattice_params.lattice_range, nhead, k_head_dim, lattice_params.value_pe_dist_real, v_head_dim,
                        lattice_params.minimum_range)

    def forward(self, src: Tensor, pos: Tensor, batch: Tensor, trans: Tensor, sizes: Tensor, onehot: Tensor = None,
                geometry: Optional[BatchGeometry] = None) -> Tensor:
        """Reference signature (…encoder.py:699) plus an optional pre-built ``BatchGeometry``."""
        if src.size(-1) != self.d_model:
            raise RuntimeError("the feature number of src and tgt must be equal to d_model")
        g = geometry if geometry is not None else BatchGeometry(pos, trans, sizes)
        output = src
        for mod in self.layers:
            output = mod(output, g.batch, g.edges, g.pos_ij, None, trans, None, g.rvecs, g.vcell, onehot, rvlen=g.rvlen)
        if self.norm is not None:
            output = self.norm(output)
        return output
