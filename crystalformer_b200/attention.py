"""Infinitely connected multi-head attention module with the reference's interface.

``CrystalformerMultiheadAttentionCUDA`` has the constructor, ``forward`` signature, parameter names (hence state_dict
keys) and initialisation of the reference class of the same name
(models/indexed_lattice_multi_head_attention_cuda.py:790-1016; the pure-PyTorch twin is
models/indexed_lattice_multi_head_attention.py:1501-1727).  The host-side steps - in-projection, the Gaussian width
``a`` per (atom, head), out-projection - follow ``crystalformer_multi_head_attention_forward_cuda`` (:462-788).  The
position encodings and the attention itself run in one fused operator (``InfiniteAttentionFunction``) instead of the
reference's ``RealPeriodicEncodingWithProjFuncCUDA`` + ``FusedDotProductAttentionCUDA`` pair; the pair is still
available (``fused=False`` or ``need_weights=True``) through ``crystalformer_b200.cuda_funcs``.  The reciprocal-space
domains (``reci``, ``RECI``, ``multihead``; :724-746) always take the operator pair, with
``ReciPeriodicEncodingFuncCUDA`` in place of (or beside) the real-space encoding.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import Tensor
from torch.nn import Module, Parameter
from torch.nn.init import constant_, normal_, xavier_uniform_
from torch.nn.modules.linear import NonDynamicallyQuantizableLinear

from . import ops
from .cuda_funcs import (FusedDotProductAttentionCUDA, RealPeriodicEncodingWithProjFuncCUDA,
                         ReciPeriodicEncodingFuncCUDA)
from .cuda_funcs.kernel_manager import KernelManager
from .params import LatticeformerParams

# ---------------------------------------------------------------------------------------------------------------
# Per-batch quantities derived from the edge list: CSR offsets and the largest crystal.  The reference rebuilds the
# CSR inside every wrapper call; here it is cached per edge tensor so that the layers of one forward share it.
# ---------------------------------------------------------------------------------------------------------------
_EDGE_CACHE: "OrderedDict[tuple, tuple]" = OrderedDict()


def heaviest_first(row_start: Tensor, cost: Optional[Tensor] = None) -> Tensor:
    """Atoms in the order in which the row kernels pick them up: by descending scheduling weight (``ops.row_cost``)
    or, without one, by the number of their keys."""
    if cost is None:
        cost = row_start[1:] - row_start[:-1]
    return torch.argsort(cost, descending=True, stable=True).to(torch.int32)


def register_edge_info(edges: Tensor, row_start: Tensor, max_atoms: int, row_order: Optional[Tensor] = None) -> None:
    """Lets a caller that already knows the CSR offsets and the largest crystal (e.g. the encoder, which builds the
    edge list on the device) avoid the device->host read that ``edge_info`` would need."""
    key = (edges.data_ptr(), tuple(edges.shape), edges.device, edges._version)
    if row_order is None:
        row_order = heaviest_first(row_start)
    # the entry holds `edges` itself: while it lives the allocator cannot hand the same address to another batch's
    # edge list (same E = sum n^2, other crystal sizes), which would otherwise hit this key with stale offsets
    _EDGE_CACHE[key] = (row_start, int(max_atoms), row_order, edges)
    while len(_EDGE_CACHE) > 16:
        _EDGE_CACHE.popitem(last=False)


def edge_info(edges: Tensor, N: int) -> Tuple[Tensor, int, Tensor]:
    key = (edges.data_ptr(), tuple(edges.shape), edges.device, edges._version)
    hit = _EDGE_CACHE.get(key)
    if hit is not None and hit[3] is edges:
        return hit[:3]
    row_start = torch.zeros(N + 1, dtype=torch.int64, device=edges.device)
    row_start.scatter_add_(0, edges[0] + 1, torch.ones_like(edges[0]))
    row_start = row_start.cumsum(0)
    max_atoms = int((row_start[1:] - row_start[:-1]).max().item()) if N > 0 else 1
    register_edge_info(edges, row_start, max_atoms)
    return _EDGE_CACHE[key][:3]


# Term lists (ops.term_list_build) of the batches in flight: the geometry is the same for every layer of a forward and
# for its backward, so the (key, translation) pairs that can matter are found once per batch and cut-off configuration.
_TERM_LIST_CACHE: "OrderedDict[tuple, tuple]" = OrderedDict()


def term_lists_for(edges: Tensor, pos_ij: Tensor, tvecs: Tensor, rvlen: Optional[Tensor], batch: Tensor,
                   row_start: Tensor, max_atoms: int, row_order: Optional[Tensor], cutoff: float, lattice_range: int,
                   minimum_range: int, a_widest: float):
    """The batch's term lists for Gaussian parameters a <= a_widest < 0, built on first use and shared by the layers
    of the batch; None when the kernels would not use them (weight floor switched off)."""
    floor = ops.get_weight_floor_log2()
    if not (a_widest < 0.0) or floor <= -200.0 or max_atoms > 1024:
        return None
    key = (edges.data_ptr(), tuple(edges.shape), edges.device, edges._version, pos_ij.data_ptr(), pos_ij._version,
           tvecs.data_ptr(), tvecs._version, float(cutoff), int(lattice_range), int(minimum_range), float(a_widest), floor)
    hit = _TERM_LIST_CACHE.get(key)
    if hit is None:
        hit = ops.term_list_build(pos_ij, tvecs, rvlen, batch, edges, row_start, max_atoms, cutoff, lattice_range,
                                  minimum_range, a_widest, row_order=row_order)
        # (the cache keeps the geometry tensors alive, so that their addresses cannot be reused while the entry lives)
        _TERM_LIST_CACHE[key] = hit + (edges, pos_ij, tvecs)
        while len(_TERM_LIST_CACHE) > 2:
            _TERM_LIST_CACHE.popitem(last=False)
    return hit[0], hit[1]


_HEAD_INDEX = {}


def _head_index(H: int, device) -> Tensor:
    """arange(H) on the device, made once."""
    key = (H, device)
    if key not in _HEAD_INDEX:
        _HEAD_INDEX[key] = torch.arange(H, device=device)
    return _HEAD_INDEX[key]


class InfiniteAttentionFunction(torch.autograd.Function):
    """out_i = sum_j softmax_j(q_i.k_j + phi_ij) (v_j + W psi_ij), phi/psi recomputed in forward and backward.

    Gradients flow to q (pre-scaled), k, v, a and W; never to positions or lattice vectors, as in the reference
    (models/cuda_funcs/real_space_enc.py:244-247 returns None for them)."""

    @staticmethod
    def forward(ctx, q, k, v, a, W, pos_ij, tvecs, rvlen, batch, edges, row_start, max_atoms, K, dist_max, wscale,
                cutoff, lattice_range, minimum_range, row_order=None, term_lists=None):
        q, k, v, a = (t.contiguous().detach() for t in (q, k, v, a))
        W3 = None
        if K > 0:
            W3 = W.detach().reshape(W.shape[-3], W.shape[-2], W.shape[-1]).contiguous()
        need_grad = any(ctx.needs_input_grad[:5])
        out, logit, lse, psi_row = ops.infinite_attn_fwd(
            q, k, v, a, pos_ij, tvecs, rvlen, batch, edges, row_start, max_atoms, K, dist_max, wscale, W3, cutoff,
            lattice_range, minimum_range, want_psi_row=need_grad and K > 0, row_order=row_order, term_lists=term_lists)
        if need_grad:
            ctx.row_order = row_order
            ctx.term_lists = term_lists
            ctx.save_for_backward(q, k, v, a, W3, pos_ij, tvecs, rvlen, batch, edges, row_start, logit, lse, out, psi_row)
            ctx.cfg = (max_atoms, K, dist_max, wscale, cutoff, lattice_range, minimum_range)
            ctx.w_shape = None if W is None else tuple(W.shape)
        return out

    @staticmethod
    def backward(ctx, gout):
        q, k, v, a, W3, pos_ij, tvecs, rvlen, batch, edges, row_start, logit, lse, out, psi_row = ctx.saved_tensors
        max_atoms, K, dist_max, wscale, cutoff, lattice_range, minimum_range = ctx.cfg
        gout = gout.contiguous()
        gq, gk, gv, ga = ops.infinite_attn_bwd(
            q, k, v, a, pos_ij, tvecs, rvlen, batch, edges, row_start, max_atoms, K, dist_max, wscale, W3, cutoff,
            lattice_range, minimum_range, logit, lse, out, gout, row_order=ctx.row_order, term_lists=ctx.term_lists)
        gW = None
        if K > 0 and ctx.needs_input_grad[4]:
            # gW[h] = sum_n gout[n,h,:] (x) psi_row[n,h,:]: the diagonal blocks of ONE (H D) x (H K) product over the
            # atoms (eight times the flops of the per-head products, and a fraction of their time at these sizes)
            N, H, D = gout.shape
            full = gout.reshape(N, H * D).t() @ psi_row.reshape(N, H * K)
            heads = _head_index(H, full.device)
            gW = full.view(H, D, H, K)[heads, :, heads, :].reshape(ctx.w_shape)  # (one gather instead of H slices)
        return (gq, gk, gv, ga, gW) + (None,) * 15


class EluWidthFunction(torch.autograd.Function):
    """a = c ((1 - lb) elu(t) + 1),  t = (q . w + shift) scale beta / (1 - lb)  per (atom, head): the default pipeline from
    the projected query to the Gaussian parameter (…attention_cuda.py:647-722 with positive_func "elu", gauss_state "q",
    normalize_gauss) as ONE autograd node.  Same arithmetic, in the same order, as the operation-by-operation code of
    ``_widths``; a training step records and replays eight operations per layer less."""

    @staticmethod
    def forward(ctx, q, w, scale, shift, beta, lb, c):
        alpha = (q * w).sum(dim=-1)
        t = ((alpha + shift) * scale) * (beta / (1.0 - lb))
        e = F.elu(t)
        ctx.save_for_backward(q, w, e, scale)
        ctx.factor = c * beta  # da/dalpha = c beta scale elu'(t)
        return ((1.0 - lb) * e + 1.0) * c

    @staticmethod
    def backward(ctx, ga):
        q, w, e, scale = ctx.saved_tensors
        # elu'(t) = 1 for t > 0, exp(t) = elu(t) + 1 otherwise
        galpha = ga * (torch.clamp(e, max=0.0) + 1.0) * (scale * ctx.factor)
        gq = galpha.unsqueeze(-1) * w if ctx.needs_input_grad[0] else None
        gw = torch.einsum("nh,nhd->hd", galpha, q).reshape(w.shape) if ctx.needs_input_grad[1] else None
        return gq, gw, None, None, None, None, None


def positive_function(name: str):
    """The map from the normalised alpha to a positive width factor (…attention_cuda.py:675-692)."""
    beta = float(name.split("=")[1]) if "=" in name else 1.0
    if name == "abs":
        return lambda x, lb: (1 - lb) * x.abs() + lb
    if name.startswith("softplus"):
        return lambda x, lb: F.softplus(x + 1 / beta * math.log(math.exp(beta * (1 - lb)) - 1), beta=beta) + lb
    if name.startswith("exp"):
        return lambda x, lb: (1.0 - lb) * torch.exp(x * (beta / (1.0 - lb))) + lb
    if name.startswith("elu"):
        return lambda x, lb: (1.0 - lb) * F.elu(x * (beta / (1.0 - lb))) + 1.0
    if name.startswith("sigmoid"):
        return lambda x, lb: (1 / lb - lb) * torch.sigmoid(x * (beta * (1 + lb) / (1.0 - lb)) + math.log(lb)) + lb
    raise NotImplementedError(f"Unkown positive_func: {name}")


class CrystalformerMultiheadAttentionCUDA(Module):
    """Drop-in for the reference module of the same name; see the module docstring."""

    def __init__(self, embed_dim, num_heads, dropout=0., bias=True, kdim=None, vdim=None,
                 params=LatticeformerParams(), device=None, dtype=None, fused: bool = True) -> None:
        factory_kwargs = {"device": device, "dtype": dtype}
        super().__init__()
        self.embed_dim = embed_dim
        self.kdim = kdim * num_heads if kdim is not None and kdim > 0 else embed_dim
        self.vdim = vdim * num_heads if vdim is not None and vdim > 0 else embed_dim
        if params.domain not in ("real", "reci", "RECI", "multihead"):
            raise NotImplementedError(f"domain {params.domain!r} is not supported")
        if params.domain == "multihead" and num_heads != 8:
            raise NotImplementedError("domain='multihead' needs 8 heads (4 real-space + 4 reciprocal-space)")
        if params.gauss_state not in ("q", "q-headdim", "q-kdim", "1", "x", "x-norm", "x-xavier"):
            raise NotImplementedError(f"gauss_state {params.gauss_state!r} is not supported")
        if params.value_pe_wave_real > 0 or params.value_pe_wave_reci > 0:
            raise NotImplementedError("value_pe_wave_real / value_pe_wave_reci > 0 is not supported")
        self.params = params
        self.fused = fused
        self.term_lists = True  # fused operator: find the translations that matter once per batch (ops.term_list_build)
        self.gauss_scale = Parameter(torch.zeros(2, **factory_kwargs), requires_grad=False)
        self.atten_scale = Parameter(torch.zeros(1, **factory_kwargs), requires_grad=False)
        self.num_heads = num_heads
        self.dropout = dropout
        self.head_dim = embed_dim // num_heads
        assert self.head_dim * num_heads == self.embed_dim, "embed_dim must be divisible by num_heads"

        self.q_proj_weight = Parameter(torch.empty((self.kdim, embed_dim), **factory_kwargs))
        self.k_proj_weight = Parameter(torch.empty((self.kdim, embed_dim), **factory_kwargs))
        self.v_proj_weight = Parameter(torch.empty((self.vdim, embed_dim), **factory_kwargs))
        if bias:
            self.in_proj_bias = Parameter(torch.empty(self.kdim * 2 + self.vdim, **factory_kwargs))
        else:
            self.register_parameter("in_proj_bias", None)
        self.out_proj = NonDynamicallyQuantizableLinear(self.vdim, embed_dim, bias=bias, **factory_kwargs)

        if params.gauss_state.startswith("q") or params.gauss_state == "1":
            self.lattice_pos_weights = Parameter(torch.empty((self.kdim), **factory_kwargs))
        else:
            self.lattice_pos_weights = Parameter(torch.empty((self.num_heads, embed_dim), **factory_kwargs))

        self.ATOM_NUM = 98
        head = self.num_heads if params.value_pe_headed else 1
        cond = 1 if params.value_pe_condproj == "no" else self.ATOM_NUM
        # …attention_cuda.py:869-878: the reciprocal-space domains size the (unused) projection by value_pe_dist_reci
        pe_dim = params.value_pe_dist_real if params.domain in ("real", "multihead") else params.value_pe_dist_reci
        self.pe_dist_proj = Parameter(torch.empty(cond, head, self.head_dim, pe_dim, **factory_kwargs)) \
            if pe_dim > 0 else None
        self.pe_wave_proj = None
        self._scale_known = False
        self._reset_parameters()

    def _load_from_state_dict(self, *args, **kwargs):
        self._scale_known = False
        return super()._load_from_state_dict(*args, **kwargs)

    def headed_pe_proj(self) -> Optional[Tensor]:
        """pe_dist_proj with one projection per head, (1, H, Dv, K): with value_pe_headed = False the parameter holds a
        single (Dv, K) matrix shared by the heads (...attention_cuda.py:869-878), which the kernels, compiled for one
        matrix per head, get as H views of it (autograd sums the heads' gradients back into the shared matrix)."""
        W = self.pe_dist_proj
        if W is not None and W.shape[1] == 1 and self.num_heads > 1:
            W = W.expand(W.shape[0], self.num_heads, W.shape[2], W.shape[3])
        return W

    def _reset_parameters(self):
        # …attention_cuda.py:882-948
        xavier_uniform_(self.q_proj_weight)
        xavier_uniform_(self.k_proj_weight)
        xavier_uniform_(self.v_proj_weight)
        xavier_uniform_(self.out_proj.weight)
        if self.in_proj_bias is not None:
            constant_(self.in_proj_bias, 0.)
            constant_(self.out_proj.bias, 0.)
        state = self.params.gauss_state
        if state in ("q", "q-headdim", "1"):
            normal_(self.lattice_pos_weights, 0., (self.kdim // self.num_heads) ** -0.5)
        elif state == "q-kdim":
            normal_(self.lattice_pos_weights, 0., (self.kdim) ** -0.5)
        elif state in ("x", "x-norm"):
            normal_(self.lattice_pos_weights, 0., (self.embed_dim) ** -0.5)
        elif state == "x-xavier":
            xavier_uniform_(self.lattice_pos_weights)
        if self.pe_dist_proj is not None:
            with torch.no_grad():
                for i, W in enumerate(self.pe_dist_proj):
                    if i != 0 and self.params.value_pe_condproj in ("I", "J", "IJ"):
                        W.set_(self.pe_dist_proj[0])
                    else:
                        W = W.view(-1, W.shape[-1])
                        xavier_uniform_(W, (W.shape[1]) ** -0.5)

    # -----------------------------------------------------------------------------------------------------------
    def _widths(self, query: Tensor, q: Tensor) -> Tensor:
        """a (N,H) < 0: the Gaussian parameter of every (atom, head) (…attention_cuda.py:640-735).  Real-space heads get
        -0.5 f / scale_real^2 (f the positive function of the normalised alpha), reciprocal-space heads
        -0.5 f scale_reci^2 ('reci'), -0.5 scale_reci^2 / f ('RECI'); 'multihead' = first half real, second half reci."""
        P = self.params
        N, H, Dq = q.shape
        w = self.lattice_pos_weights
        if P.gauss_state.startswith("q") and P.normalize_gauss and self._scale_known and P.domain == "real" \
                and P.positive_func.startswith("elu") and torch.is_grad_enabled():
            # training with the default pipeline: one autograd node
            beta = float(P.positive_func.split("=")[1]) if "=" in P.positive_func else 1.0
            return EluWidthFunction.apply(q, w.reshape(1, H, Dq), self.gauss_scale[0], self.gauss_scale[1], beta,
                                          float(P.gauss_lb_real), -0.5 * P.scale_real ** -2)
        if P.gauss_state.startswith("q"):
            # q_h . w_h per (atom, head): an element-wise product and a 16-term sum (the reference writes it as a batched
            # matrix product, ...attention_cuda.py:647, which launches a GEMM per head for a dot product)
            alpha = (q * w.reshape(1, H, Dq)).sum(dim=-1)
        elif P.gauss_state == "1":
            alpha = w.reshape(1, H, Dq).sum(dim=-1).expand(N, H)
        else:
            alpha = F.linear(query, w)
        alpha = alpha.view(N, H)
        if P.normalize_gauss:
            # The reference tests the stored scale on every call, a device->host read per layer; once the scale is
            # known to be set it cannot become unset except by loading a state_dict, so the answer is remembered.
            if not self._scale_known:
                self._scale_known = bool(self.gauss_scale[0] > 0)
            scale_available = self._scale_known
            if scale_available:
                scale, shift = self.gauss_scale[0], self.gauss_scale[1]
            else:
                scale = torch.reciprocal(alpha.detach().std())
                shift = -alpha.detach().mean()
            alpha = (alpha + shift) * scale
            if self.training and not scale_available:
                # saved once, in the first training step (…attention_cuda.py:669-673)
                torch.nn.init.constant_(self.gauss_scale[0], scale)
                torch.nn.init.constant_(self.gauss_scale[1], shift)
                self._scale_known = True
        func = positive_function(P.positive_func)
        if P.domain == "real":
            return func(alpha, P.gauss_lb_real) * (-0.5 * P.scale_real ** -2)
        if P.domain == "reci":
            return func(alpha, P.gauss_lb_reci) * (-0.5 * P.scale_reci ** 2)
        if P.domain == "RECI":
            return 1 / func(alpha, P.gauss_lb_reci) * (-0.5 * P.scale_reci ** 2)
        a1, a2 = alpha.chunk(2, 1)  # multihead
        return torch.cat((func(a1, P.gauss_lb_real) * (-0.5 * P.scale_real ** -2),
                          func(a2, P.gauss_lb_reci) * (-0.5 * P.scale_reci ** 2)), dim=1)

    def forward(self, query: Tensor, key: Tensor, value: Tensor, batch_q: Tensor, batch_kv: Tensor, edges: Tensor,
                points: Tensor, dist2_min: Tensor, tvecs: Tensor,
                kr_base: Optional[Tensor] = None, rvecs: Optional[Tensor] = None, vcell: Optional[Tensor] = None,
                onehot: Tensor = None, need_weights: bool = True, rvlen: Optional[Tensor] = None
                ) -> Tuple[Tensor, Optional[Tensor]]:
        """Same arguments as the reference (…attention_cuda.py:950-955): ``points`` is pos_ij (E,3), ``tvecs`` the
        lattice rows (B,3,3), ``rvecs`` the reciprocal rows (needed by the adaptive cut-off).  ``rvlen`` optionally
        passes the row norms of ``rvecs`` if the caller has them already."""
        P = self.params
        H = self.num_heads
        N = query.shape[0]
        if P.value_pe_condproj != "no":
            raise NotImplementedError("value_pe_condproj other than 'no' is not supported")
        if P.norm_func_mode != 0:
            raise NotImplementedError("norm_func_mode other than 0 is not supported")
        if batch_q is not batch_kv and not torch.equal(batch_q, batch_kv):
            raise NotImplementedError("only self-attention (batch_q == batch_kv) is supported")
        if self.training and self.dropout > 0.0:
            raise NotImplementedError("attention dropout is not supported by the fused kernels")

        # in-projection (…attention_cuda.py:582-596): one GEMM when q, k and v come from the same tensor
        if query is key and key is value:
            w_in = torch.cat((self.q_proj_weight, self.k_proj_weight, self.v_proj_weight), dim=0)
            q, k, v = F.linear(query, w_in, self.in_proj_bias).split((self.kdim, self.kdim, self.vdim), dim=1)
        else:
            b_q = b_k = b_v = None
            if self.in_proj_bias is not None:
                b_q, b_k, b_v = self.in_proj_bias.split([self.kdim, self.kdim, self.vdim])
            q = F.linear(query, self.q_proj_weight, b_q)
            k = F.linear(key, self.k_proj_weight, b_k)
            v = F.linear(value, self.v_proj_weight, b_v)
        Dq, Dv = self.kdim // H, self.vdim // H
        q = q.reshape(N, H, Dq)
        k = k.reshape(k.shape[0], H, Dq)
        v = v.reshape(v.shape[0], H, Dv)

        a = self._widths(query, q)

        dist_max = P.value_pe_dist_max
        if dist_max < 0:
            dist_max = (-dist_max) * P.scale_real
        K = P.value_pe_dist_real
        cutoff = 0.0
        if P.adaptive_cutoff_sigma < 0:
            cutoff = float(P.adaptive_cutoff_sigma)
        elif P.adaptive_cutoff_sigma > 0:
            cutoff = P.scale_real * P.gauss_lb_real ** (-0.5) * P.adaptive_cutoff_sigma
        if cutoff != 0.0:
            if rvlen is None:
                if rvecs is None:
                    raise ValueError("the adaptive cut-off needs rvecs (reciprocal lattice rows)")
                rvlen = torch.norm(rvecs, 2, dim=-1)
        else:
            rvlen = None
        lattice_range = int(P.lattice_range)
        minimum_range = lattice_range if P.minimum_range else 0
        q_scaled = q / math.sqrt(Dq)

        values = None
        if self.fused and not need_weights and P.domain == "real":
            row_start, max_atoms, row_order = edge_info(edges, N)
            # every positive function is bounded below by gauss_lb_real, so a <= gauss_lb_real x (-0.5 / scale_real^2)
            lists = None
            if getattr(self, "term_lists", True) and points is not None and P.gauss_lb_real > 0 \
                    and not isinstance(P.scale_real, (list, tuple)):
                lists = term_lists_for(edges, points, tvecs, rvlen, batch_q, row_start, max_atoms, row_order, cutoff,
                                       lattice_range, minimum_range, -0.5 * P.gauss_lb_real / float(P.scale_real) ** 2)
            attn = InfiniteAttentionFunction.apply(
                q_scaled, k, v, a, self.headed_pe_proj(), points, tvecs, rvlen, batch_q, edges, row_start, max_atoms, K,
                float(dist_max), float(P.value_pe_width_scale), cutoff, lattice_range, minimum_range, row_order, lists)
            weights = None
        else:
            # the reference's operator split, through the drop-in autograd functions
            saved = (KernelManager.LATTICE_RANGE, KernelManager.MINIMUM_RANGE)
            KernelManager.LATTICE_RANGE, KernelManager.MINIMUM_RANGE = lattice_range, minimum_range
            try:
                phi = None
                if P.domain in ("real", "multihead"):
                    extra = (rvlen, cutoff) if cutoff != 0.0 else ()
                    a_real, W = a, self.headed_pe_proj()
                    if P.domain == "multihead":
                        # the kernels are compiled for eight heads: the four real-space heads are computed twice and
                        # the copy is dropped (…attention_cuda.py:731-746 passes half the heads to each operator)
                        a_real = torch.cat((a[:, :H // 2], a[:, :H // 2]), dim=1)
                        if W is not None and W.shape[1] == H:
                            W = torch.cat((W[:, :H // 2], W[:, :H // 2]), dim=1)
                    res = RealPeriodicEncodingWithProjFuncCUDA.apply(
                        a_real, points, dist2_min, tvecs, batch_q, edges, K, float(dist_max),
                        float(P.value_pe_width_scale), W, *extra)
                    phi = res[0]
                    values = res[1] if len(res) > 1 else None
                if P.domain != "real":
                    if kr_base is None or rvecs is None or vcell is None:
                        raise ValueError("the reciprocal-space domains need kr_base, rvecs and vcell")
                    a_reci = a if P.domain != "multihead" else torch.cat((a[:, H // 2:], a[:, H // 2:]), dim=1)
                    phi_reci = ReciPeriodicEncodingFuncCUDA.apply(a_reci, kr_base, rvecs, vcell, batch_q, edges)
                    if P.domain == "multihead":
                        phi = torch.cat((phi[:, :H // 2], phi_reci[:, H // 2:]), dim=1)
                        if values is not None:
                            values = torch.cat((values[:, :H // 2], torch.zeros_like(values[:, H // 2:])), dim=1)
                    else:
                        phi = phi_reci
            finally:
                KernelManager.LATTICE_RANGE, KernelManager.MINIMUM_RANGE = saved
            attn = FusedDotProductAttentionCUDA.apply(q_scaled, k, v, phi, values, batch_q, edges)
            weights = None
            if need_weights:
                with torch.no_grad():
                    row_start = edge_info(edges, N)[0]
                    prob, _ = ops.fused_attn_fwd(q_scaled.detach(), k.detach(), v.detach(), phi.detach(),
                                                 None if values is None else values.detach(), edges, row_start)
                    weights = prob.mean(dim=1)

        attn_output = F.linear(attn.reshape(N, Dv * H), self.out_proj.weight, self.out_proj.bias)
        if need_weights:
            return attn_output, weights
        return attn_output, values


