"""CPU restatement of the reference model's forward pass for the real-space configuration.  TEST INFRASTRUCTURE ONLY
(used by the smoke check and by the CPU-baseline / reference legs of bench.py; never by the shipped package).

Host-side steps are plain torch-CPU calls that follow the reference line by line; the position encodings and the
attention go through the CPU oracle (``oracle.lattice_sum_fwd`` / ``oracle.fused_attn_fwd``) or, with
``use_ref=True``, through the reference project's own kernel sources compiled for the CPU (``oracle/_ref``).

  embedding                models/latticeformer.py:224
  edges, geometry          models/indexed_latticeformer_encoder.py:15-32, 183-253
  per layer: in-proj, a    models/indexed_lattice_multi_head_attention_cuda.py:582-596, 640-722
             phi, W psi    models/cuda_funcs/real_space_enc_proj.py:20-97 (kernel real_enc_proj_fwd)
             attention     models/cuda_funcs/fused_dpa.py:19-61 (kernel fused_dpa_fwd_v3)
             out-proj, FFN models/indexed_latticeformer_encoder.py:848-890 (post-norm, LayerNorm = Identity)
  pooling, head            models/pooling.py:19-25, models/latticeformer.py:291-302
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

import oracle


def _np(t):
    return t.detach().cpu().numpy()


def forward_cpu(state: dict, params, cb, use_ref: bool = False) -> np.ndarray:
    """``state``: state_dict of the model (torch CPU tensors or numpy); ``params``: attribute bag with the keys of the
    reference's default.json; ``cb``: a ``CrystalBatch``.  Returns the (B, n_targets) outputs as float32."""
    st = {k: torch.as_tensor(np.asarray(v)) if not torch.is_tensor(v) else v.detach().cpu() for k, v in state.items()}
    H = params.head_num
    K = params.value_pe_dist_real
    lattice_range = params.lattice_range
    minimum_range = lattice_range if params.minimum_range else 0
    beta = float(params.positive_func.split("=")[1]) if "=" in params.positive_func else 1.0
    assert params.positive_func.startswith("elu") and params.domain == "real" and params.gauss_state == "q"

    x = F.linear(torch.as_tensor(cb.x), st["input_embeddings.weight"])
    edges = oracle.edge_index(cb.sizes)
    pos_ij, rvecs, vcell, rvlen = oracle.geometry(cb.pos, cb.trans_vec, edges)
    N = cb.num_atoms
    scale_real = params.scale_real
    for layer in range(params.num_layers):
        pre = f"encoder.layers.{layer}."
        sr = scale_real[layer % len(scale_real)] if isinstance(scale_real, (list, tuple)) else scale_real
        wq, wk, wv = (st[pre + f"self_attn.{n}_proj_weight"] for n in "qkv")
        bq, bk, bv = st[pre + "self_attn.in_proj_bias"].split([wq.shape[0], wk.shape[0], wv.shape[0]])
        q, k, v = F.linear(x, wq, bq), F.linear(x, wk, bk), F.linear(x, wv, bv)
        D = q.shape[1] // H
        q, k, v = q.view(N, H, D), k.view(N, H, D), v.view(N, H, D)
        alpha = (q.reshape(N, H, 1, D) @ st[pre + "self_attn.lattice_pos_weights"].reshape(H, D, 1)).view(N, H)
        if params.normalize_gauss:
            gs = st[pre + "self_attn.gauss_scale"]
            if gs[0] > 0:
                scale, shift = gs[0], gs[1]
            else:
                scale, shift = torch.reciprocal(alpha.std()), -alpha.mean()
            alpha = (alpha + shift) * scale
        lb = params.gauss_lb_real
        a = ((1.0 - lb) * F.elu(alpha * (beta / (1.0 - lb))) + 1.0) * (-0.5 * sr ** -2)
        dist_max = params.value_pe_dist_max
        if dist_max < 0:
            dist_max = (-dist_max) * sr
        if params.adaptive_cutoff_sigma < 0:
            cutoff = params.adaptive_cutoff_sigma
        elif params.adaptive_cutoff_sigma > 0:
            cutoff = sr * lb ** (-0.5) * params.adaptive_cutoff_sigma
        else:
            cutoff = 0.0
        W = _np(st[pre + "self_attn.pe_dist_proj"]) if K > 0 else None
        a_np = _np(a)
        if use_ref:
            z, vals = oracle.ref_real_enc_proj_fwd(a_np, pos_ij, cb.trans_vec, cb.batch, edges, K, dist_max,
                                                   params.value_pe_width_scale, W, rvlen, cutoff)
            _, o = oracle.ref_fused_dpa_fwd(_np(q / math.sqrt(D)), _np(k), _np(v), z, vals, edges, v3=True, K=K)
        else:
            z, vals = oracle.lattice_sum_fwd(a_np, pos_ij, cb.trans_vec, cb.batch, edges, K, dist_max,
                                             params.value_pe_width_scale, W=W, rvlen=rvlen if cutoff != 0.0 else None,
                                             cutoff_radius=cutoff, lattice_range=lattice_range,
                                             minimum_range=minimum_range)
            _, o = oracle.fused_attn_fwd(_np(q / math.sqrt(D)), _np(k), _np(v), z, vals, edges)
        o = torch.as_tensor(o).reshape(N, H * D)
        x = x + F.linear(o, st[pre + "self_attn.out_proj.weight"], st[pre + "self_attn.out_proj.bias"])
        ff = F.linear(F.relu(F.linear(x, st[pre + "linear1.weight"], st[pre + "linear1.bias"])),
                      st[pre + "linear2.weight"], st[pre + "linear2.bias"])
        x = x + ff
    pooled = torch.as_tensor(oracle.segment_mean(_np(x), cb.sizes))
    n_mlp = len([k for k in st if k.startswith("mlp.") and k.endswith(".weight")])
    y = pooled
    idx = sorted(int(k.split(".")[1]) for k in st if k.startswith("mlp.") and k.endswith(".weight"))
    for t, i in enumerate(idx):
        y = F.linear(y, st[f"mlp.{i}.weight"], st[f"mlp.{i}.bias"])
        if t < n_mlp - 1:
            y = F.relu(y)
    return _np(y).astype(np.float32)
