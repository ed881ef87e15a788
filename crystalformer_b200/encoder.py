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

import ctypes

from . import _lib, ops
from .attention import CrystalformerMultiheadAttentionCUDA, heaviest_first, register_edge_info
from .cuda_funcs import compile_kernels
from .params import LatticeformerParams


def _get_activation_fn(activation):
    if activation == "relu":
        return F.relu
    if activation == "gelu":
        return F.gelu
    raise RuntimeError("activation should be relu/gelu, not {}".format(activation))


def _tf32(x: Tensor) -> Tensor:
    """x rounded to TF32 (10-bit mantissa, ties away from zero), as cvt.rna.tf32.f32 does."""
    bits = x.contiguous().view(torch.int32)
    return ((bits + 0x1000) & ~0x1FFF).view(torch.float32)


def _bf16_pair(low: Tensor, high: Tensor) -> Tensor:
    """float32-typed words whose lower / upper 16 bits are ``low`` / ``high`` rounded to bfloat16 (nearest even)."""
    lo_bits = low.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
    hi_bits = high.to(torch.bfloat16).view(torch.int16).to(torch.int32) << 16
    return (hi_bits | lo_bits).view(torch.float32)


def pack_dense_weight(W: Tensor) -> Tensor:
    """A Linear weight (out, in) in the fragment order of the fused dense kernel: float4 entries
    [(nt * in/8 + ks) * 32 + lane] = (hi W[n,k], hi W[n,k+4], c W[n,k], c W[n,k+4]) with n = 8 nt + lane // 4,
    k = 8 ks + lane % 4, hi = TF32 rounding and c(w) the word {lower half: bf16(hi(w)), upper half: bf16(w - hi(w))},
    the operands of the kernel's main (TF32) and correction (bfloat16, 16-deep) products.  Returned flat."""
    out_f, in_f = W.shape
    assert out_f % 8 == 0 and in_f % 8 == 0
    W = W.detach().float().contiguous()
    hi = _tf32(W)
    corr = _bf16_pair(hi, W - hi)

    def frag(M):  # (out, in) -> (nt, ks, g, t, half)
        return M.view(out_f // 8, 8, in_f // 8, 2, 4).permute(0, 2, 1, 4, 3)

    return torch.cat((frag(hi), frag(corr)), dim=-1).contiguous().reshape(-1)


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
        self.row_order = ops.row_order(self.atom_start, trans.float(), num_atoms)
        self._kr_base = None
        register_edge_info(self.edges, self.row_start, self.max_atoms, self.row_order)

    @property
    def kr_base(self) -> Tensor:
        """(E,3) phases rvecs . pos_ij of the reciprocal-space domains (…encoder.py:249-251), built on first use."""
        if self._kr_base is None:
            self._kr_base = ops.reci_phase(self.pos_ij, self.rvecs, self.batch, self.edges)
        return self._kr_base


class CrystalformerEncoderLayerCUDA(Module):
    __constants__ = ["norm_first"]

    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1,
                 activation: Union[str, Callable[[Tensor], Tensor]] = F.relu, layer_norm_eps: float = 1e-5,
                 norm_first: bool = False, no_layer_norm=False, params=LatticeformerParams(), k_dim=0, v_dim=0,
                 device=None, dtype=None) -> None:
        assert params.domain in ("real", "reci", "RECI", "multihead"), f"unsupported domain {params.domain!r}"
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
        self.native = True  # use the one-call inference path whenever it applies
        self.dense_fused = True  # ... with the projections and feed-forward of a layer boundary fused into one kernel
        v_head_dim = v_dim if v_dim > 0 else d_model // nhead
        k_head_dim = k_dim if k_dim > 0 else d_model // nhead
        compile_kernels(lattice_params.lattice_range, nhead, k_head_dim, lattice_params.value_pe_dist_real, v_head_dim,
                        lattice_params.minimum_range)

    # -----------------------------------------------------------------------------------------------------------
    # Inference fast path: the whole stack in one call into the library (cf_encoder_forward).
    # -----------------------------------------------------------------------------------------------------------
    def _native_ok(self) -> bool:
        if self.training or torch.is_grad_enabled() or self.norm is not None or self.d_model != 128 or self.nhead != 8:
            return False
        for layer in self.layers:
            att, P = layer.self_attn, layer.self_attn.params
            if not (P.domain == "real" and P.positive_func.startswith("elu") and P.gauss_state == "q" and P.normalize_gauss and att.fused
                    and P.value_pe_condproj == "no" and P.norm_func_mode == 0 and att.kdim == 128 and att.vdim == 128
                    and att.in_proj_bias is not None and layer.activation is F.relu and not layer.norm_first
                    and isinstance(layer.norm1, Identity)):
                return False
            if not att._scale_known:
                att._scale_known = bool(att.gauss_scale[0] > 0)
                if not att._scale_known:
                    return False
        return True

    def _packed_weights(self, device):
        """Device pointers and scalars of every layer in the layout cf_encoder_forward expects; rebuilt only when a
        parameter or buffer changed (in-place updates bump ``_version``)."""
        params = [p for p in self.parameters()] + [b for b in self.buffers()]  # (gauss_scale is a buffer)
        key = (device, self.dense_fused, tuple(p._version for p in params), tuple(p.data_ptr() for p in params))
        cache = getattr(self, "_native_cache", None)
        if cache is not None and cache[0] == key:
            return cache[1]
        keep, ptrs, scalars = [], [], []
        for layer in self.layers:
            att, P = layer.self_attn, layer.self_attn.params
            wqkv = torch.cat((att.q_proj_weight, att.k_proj_weight, att.v_proj_weight), 0).detach().float().contiguous()
            tensors = [wqkv, att.in_proj_bias, att.lattice_pos_weights,
                       att.headed_pe_proj(), att.out_proj.weight, att.out_proj.bias,
                       layer.linear1.weight, layer.linear1.bias, layer.linear2.weight, layer.linear2.bias, None]
            tensors = [None if t is None else t.detach().float().contiguous() for t in tensors]
            if self.dense_fused and layer.linear1.weight.shape[0] % 128 == 0:
                # slot 10: in-projection, out-projection and feed-forward weights packed for the fused dense kernel
                tensors[10] = torch.cat([pack_dense_weight(m) for m in
                                         (wqkv, att.out_proj.weight, layer.linear1.weight, layer.linear2.weight)])
            keep.append(tensors)
            ptrs += [0 if t is None else t.data_ptr() for t in tensors]
            beta = float(P.positive_func.split("=")[1]) if "=" in P.positive_func else 1.0
            dist_max = P.value_pe_dist_max
            if dist_max < 0:
                dist_max = (-dist_max) * P.scale_real
            gs = att.gauss_scale.detach().cpu().tolist()
            scalars += [gs[0], gs[1], -0.5 * P.scale_real ** -2, beta, P.gauss_lb_real, dist_max]
        packed = dict(keep=keep, ptrs=(ctypes.c_void_p * len(ptrs))(*ptrs), scalars=(ctypes.c_double * len(scalars))(*scalars),
                      ff=self.layers[0].linear1.weight.shape[0])
        self._native_cache = (key, packed)
        return packed

    def _cutoff(self) -> float:
        """The cut-off argument of the kernels: 0 fixed box, < 0 adaptive (sigmas), > 0 static radius in Angstrom."""
        P = self.lattice_params
        if P.adaptive_cutoff_sigma < 0:
            return float(P.adaptive_cutoff_sigma)
        if P.adaptive_cutoff_sigma > 0:
            sr = P.scale_real[0] if isinstance(P.scale_real, (list, tuple)) else P.scale_real
            return float(sr * P.gauss_lb_real ** (-0.5) * P.adaptive_cutoff_sigma)
        return 0.0

    def _forward_native(self, src: Tensor, trans: Tensor, g: "BatchGeometry") -> Tensor:
        P = self.lattice_params
        dev = src.device
        w = self._packed_weights(dev)
        N, E, B = src.shape[0], g.edges.shape[1], trans.shape[0]
        x = src.detach().float().contiguous().clone()
        lib = _lib.load()
        work = torch.empty(int(lib.cf_encoder_workspace_floats(N, E, w["ff"])), dtype=torch.float32, device=dev)
        cutoff = self._cutoff()
        with torch.cuda.device(dev):
            _lib.call("cf_encoder_forward", ctypes.c_void_p(torch.cuda.current_blas_handle()), len(self.layers),
                      w["ptrs"], w["scalars"], x.data_ptr(), g.pos_ij.data_ptr(), trans.data_ptr(),
                      g.rvlen.data_ptr() if cutoff != 0.0 else None, g.batch.data_ptr(), g.edges.data_ptr(),
                      g.row_start.data_ptr(), N, B, E, g.max_atoms, int(P.value_pe_dist_real), w["ff"],
                      float(P.value_pe_width_scale), cutoff, int(P.lattice_range),
                      int(P.lattice_range) if P.minimum_range else 0, work.data_ptr(), g.row_order.data_ptr(),
                      self._attention_events(),
                      torch.cuda.current_stream(dev).cuda_stream)
        return x

    def _attention_events(self):
        """When ``self.attention_event_log`` is a list, every native forward appends one (start, end) pair of timing
        events per layer, recorded by the library around that layer's attention kernels."""
        log = getattr(self, "attention_event_log", None)
        if log is None:
            return None
        pairs = []
        for _ in self.layers:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(); e.record()  # creates the underlying CUDA events; they are re-recorded by the library
            pairs += [s, e]
        log.extend(zip(pairs[0::2], pairs[1::2]))
        return (ctypes.c_void_p * len(pairs))(*[p.cuda_event for p in pairs])

    def forward(self, src: Tensor, pos: Tensor, batch: Tensor, trans: Tensor, sizes: Tensor, onehot: Tensor = None,
                geometry: Optional[BatchGeometry] = None) -> Tensor:
        """Reference signature (…encoder.py:699) plus an optional pre-built ``BatchGeometry``."""
        if src.size(-1) != self.d_model:
            raise RuntimeError("the feature number of src and tgt must be equal to d_model")
        g = geometry if geometry is not None else BatchGeometry(pos, trans, sizes)
        if self.native and self._native_ok():
            return self._forward_native(src, trans.float().contiguous(), g)
        output = src
        for mod in self.layers:
            kr_base = g.kr_base if mod.domain != "real" else None
            output = mod(output, g.batch, g.edges, g.pos_ij, None, trans, kr_base, g.rvecs, g.vcell, onehot, rvlen=g.rvlen)
        if self.norm is not None:
            output = self.norm(output)
        return output
