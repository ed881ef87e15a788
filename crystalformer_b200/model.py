"""Model shell with the reference's interface and state_dict keys (models/latticeformer.py:32-302):
98-dim one-hot species -> Linear embedding -> encoder -> (optional projection) -> per-crystal pooling -> MLP head.
Only what the benchmark configurations use is implemented: ``pooling`` in {"avr", "max"}, ``pre_pooling_op`` in
{"no", "relu", "w+relu"}, ``norm_type`` in {"no", "id", "ln"}; the reference's single-process multi-GPU split is
replaced by one process per GPU (``crystalformer_b200.sharding``)."""
from __future__ import annotations

import copy
import types
from typing import Optional

import torch
import torch.nn as nn

from .cuda_funcs import IrregularMeanCUDA
from .encoder import BatchGeometry, CrystalformerEncoderCUDA
from .params import DEFAULT_MODEL_PARAMS, LatticeformerParams


def default_params(**overrides) -> types.SimpleNamespace:
    """Attribute bag carrying the keys of the reference's params/latticeformer/default.json."""
    p = copy.deepcopy(DEFAULT_MODEL_PARAMS)
    p.update(overrides)
    return types.SimpleNamespace(**p)


def avr_pool(x, batch, sizes):
    """Deterministic per-crystal mean (models/pooling.py:19-25 with the CUDA branch)."""
    return IrregularMeanCUDA.apply(x, batch, sizes)


def max_pool(x, batch, sizes):
    """Per-crystal maximum (models/pooling.py:14-17), without the host loop."""
    B = sizes.shape[0]
    out = torch.full((B, x.shape[1]), float("-inf"), dtype=x.dtype, device=x.device)
    return out.scatter_reduce(0, batch[:, None].expand_as(x), x, reduce="amax", include_self=True)


class Latticeformer(nn.Module):
    def __init__(self, params):
        super().__init__()
        embedding_dim = copy.deepcopy(params.embedding_dim)
        self.params = params
        num_layers = getattr(params, "num_layers", 4)
        model_dim = getattr(params, "model_dim", 128)
        ff_dim = getattr(params, "ff_dim", 512)
        t_fixup_init = getattr(params, "t_fixup_init", True)
        self.pooling = getattr(params, "pooling", "max")
        pre_pooling_op = getattr(params, "pre_pooling_op", "w+bn+relu")
        dropout = getattr(params, "dropout", 0.1)
        head_num = getattr(params, "head_num", 8)
        v_dim = getattr(params, "v_dim", 0)
        k_dim = getattr(params, "k_dim", 0)
        norm_type = getattr(params, "norm_type", "bn")
        t_activation = getattr(params, "t_activation", "relu")
        if getattr(params, "use_cgcnn_feat", False) or getattr(params, "scale_grad", 0.0) > 0:
            raise NotImplementedError("use_cgcnn_feat / scale_grad are not supported")

        lattice_params = LatticeformerParams()
        lattice_params.parseFromArgs(params)

        self.ATOM_FEAT_DIM = 98
        self.input_embeddings = nn.Linear(self.ATOM_FEAT_DIM, model_dim, bias=False)
        emb_scale = model_dim ** (-0.5)
        if t_fixup_init:
            emb_scale *= (9 * num_layers) ** (-1 / 4)
        nn.init.normal_(self.input_embeddings.weight, mean=0, std=emb_scale)

        self.encoder = CrystalformerEncoderCUDA(
            model_dim, head_num, activation=t_activation, num_encoder_layers=num_layers, dim_feedforward=ff_dim,
            dropout=dropout, t_fixup_init=t_fixup_init, no_layer_norm=t_fixup_init, lattice_params=lattice_params,
            k_dim=k_dim, v_dim=v_dim)

        if norm_type == "ln":
            norm = nn.LayerNorm
        elif norm_type in ("id", "no"):
            norm = nn.Identity
        else:
            raise NotImplementedError(f"norm_type: {norm_type}")

        dim_pooled = model_dim
        self.proj_before_pooling = lambda x: x
        if pre_pooling_op == "w+relu":
            dim_pooled = embedding_dim.pop(0)
            self.proj_before_pooling = nn.Sequential(nn.Linear(model_dim, dim_pooled), nn.ReLU(True))
        elif pre_pooling_op == "relu":
            self.proj_before_pooling = nn.ReLU(True)
        elif pre_pooling_op != "no":
            raise NotImplementedError(f"pre_pooling_op: {pre_pooling_op}")

        if self.pooling == "max":
            self.pooling_layer = max_pool
        elif self.pooling == "avr":
            self.pooling_layer = avr_pool
        else:
            raise NotImplementedError(f"pooling: {self.pooling}")

        final_dim = 1 if isinstance(params.targets, str) else len(params.targets)
        in_dim = [dim_pooled] + embedding_dim[:-1]
        layers = []
        for di, do in zip(in_dim, embedding_dim):
            layers += [nn.Linear(di, do), norm(do), nn.ReLU(True)]
        layers.append(nn.Linear(embedding_dim[-1], final_dim))
        self.mlp = nn.Sequential(*layers)

    def forward(self, data, geometry: Optional[BatchGeometry] = None):
        """``data`` carries x (N,98), pos (N,3), batch (N), trans_vec (B,3,3), sizes (B) like the reference's PyG batch."""
        x = self.input_embeddings(data.x)
        g = geometry if geometry is not None else BatchGeometry(data.pos, data.trans_vec, data.sizes)
        x = self.encoder(x, data.pos, g.batch, data.trans_vec, g.sizes, geometry=g)
        x = self.proj_before_pooling(x)
        x = self.pooling_layer(x, g.batch, g.sizes)
        return self.mlp(x)
