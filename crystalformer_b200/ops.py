"""Thin torch-tensor front end of the C ABI: checks tensors, allocates outputs with torch and passes raw pointers.

Every function launches on ``torch.cuda.current_stream`` of the tensors' device and returns without synchronising.
These are the building blocks of the drop-in autograd functions in ``crystalformer_b200.cuda_funcs`` and of the
fused attention module; they have no CPU path.
"""
from __future__ import annotations

from ctypes import c_double, c_int, c_int64, c_void_p
from typing import Optional, Tuple

import torch

from . import _lib

HEADS = 8
HEAD_DIM = 16


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0) if t is None else c_void_p(t.data_ptr())


def _stream(device) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _want(t: Optional[torch.Tensor], dtype, name: str, device=None) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: crystalformer_b200 has no CPU path")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if device is not None and t.device != device:
        raise RuntimeError(f"{name} is on {t.device}, expected {device}")
    return t if t.is_contiguous() else t.contiguous()


def _check_projection(W: Optional[torch.Tensor], H: int, K: int, name: str) -> None:
    """The kernels index W as one (Dv, K) matrix per head: a projection shared by the heads (shape (..., 1, Dv, K)) must
    be expanded to H heads by the caller, or the kernels would read past its end."""
    if W is not None and K > 0 and (W.dim() < 3 or W.shape[-3] != H or W.shape[-1] != K):
        raise ValueError(f"{name}: W must end in (H={H}, Dv, K={K}), got {tuple(W.shape)}")


def set_sorted_rows(enabled: bool) -> None:
    """Whether the one-call forwards may use row lists and the sorted row kernel (cf_set_sorted_rows)."""
    _lib.load().cf_set_sorted_rows(c_int(1 if enabled else 0))


def set_chained_launches(enabled: bool) -> None:
    """Whether the one-call forwards chain their kernels by programmatic dependent launches (cf_set_chained_launches)."""
    _lib.load().cf_set_chained_launches(c_int(1 if enabled else 0))


def set_row_stats(words: Optional[torch.Tensor]) -> None:
    """Work counters of the sorted row kernel (cf_set_row_stats): a zeroed CUDA int64 tensor of four words, or None to
    switch the counting off.  The tensor must stay alive while set."""
    _lib.load().cf_set_row_stats(_ptr(words))


def set_weight_floor_log2(value: float) -> None:
    _lib.load().cf_set_weight_floor_log2(c_double(value))


def get_weight_floor_log2() -> float:
    return float(_lib.load().cf_get_weight_floor_log2())


def crystal_offsets(sizes: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(atom_start, edge_start), each (B+1) int64: exclusive prefix sums of sizes and sizes^2."""
    sizes = _want(sizes, torch.int64, "sizes")
    B = sizes.shape[0]
    atom_start = torch.empty(B + 1, dtype=torch.int64, device=sizes.device)
    edge_start = torch.empty(B + 1, dtype=torch.int64, device=sizes.device)
    with torch.cuda.device(sizes.device):
        _lib.call("cf_crystal_offsets", _ptr(sizes), c_int64(B), _ptr(atom_start), _ptr(edge_start), _stream(sizes.device))
    return atom_start, edge_start


def batch_prepare(pos, trans, sizes, atom_start, edge_start, N: int, E: int, want_edges=True, want_pos_ij=True):
    """Device-side replacement of get_edge_index + compute_lattice_distances_for_cuda.  N and E are host integers
    (sum of sizes and of sizes^2) known to the caller.  Returns a dict of tensors."""
    dev = pos.device
    pos = _want(pos, torch.float32, "pos")
    trans = _want(trans, torch.float32, "trans", dev)
    sizes = _want(sizes, torch.int64, "sizes", dev)
    B = sizes.shape[0]
    o = dict(
        batch=torch.empty(N, dtype=torch.int64, device=dev),
        row_start=torch.empty(N + 1, dtype=torch.int64, device=dev),
        edges=torch.empty((2, E), dtype=torch.int64, device=dev) if want_edges else None,
        pos_ij=torch.empty((E, 3), dtype=torch.float32, device=dev) if want_pos_ij else None,
        rvecs=torch.empty((B, 3, 3), dtype=torch.float32, device=dev),
        vcell=torch.empty((B,), dtype=torch.float32, device=dev),
        rvlen=torch.empty((B, 3), dtype=torch.float32, device=dev),
    )
    with torch.cuda.device(dev):
        _lib.call("cf_batch_prepare", _ptr(pos), _ptr(trans), _ptr(sizes), _ptr(atom_start), _ptr(edge_start),
                  c_int64(B), c_int64(N), c_int64(E), _ptr(o["batch"]), _ptr(o["edges"]), _ptr(o["row_start"]),
                  _ptr(o["pos_ij"]), _ptr(o["rvecs"]), _ptr(o["vcell"]), _ptr(o["rvlen"]), _stream(dev))
    return o


def lattice_box(a, batch, edges, rvlen, cutoff_radius, lattice_range, minimum_range, a_per_edge=False):
    """(E,H,3) int32 half-widths of the translation box of every (edge, head)."""
    dev = a.device
    a = _want(a, torch.float32, "a")
    batch, edges = _want(batch, torch.int64, "batch", dev), _want(edges, torch.int64, "edges", dev)
    rvlen = _want(rvlen, torch.float32, "rvlen", dev)
    E, H, N = edges.shape[1], a.shape[1], batch.shape[0]
    box = torch.empty((E, H, 3), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_lattice_box", _ptr(a), c_int(int(a_per_edge)), _ptr(batch), _ptr(edges), c_int64(N), c_int64(H),
                  c_int64(E), _ptr(rvlen), c_double(cutoff_radius), c_int(lattice_range), c_int(minimum_range),
                  _ptr(box), _stream(dev))
    return box


def lattice_sum_fwd(a, pos_ij, tvecs, batch, edges, K, dist_max, wscale, W=None, rvlen=None, cutoff_radius=0.0,
                    lattice_range=2, minimum_range=2, a_per_edge=False, z=None, v=None):
    """phi (E,H) and psi (E,H,K) or W psi (E,H,Dv).  W: (H,Dv,K) or (W_num,H,Dv,K).  z / v may be preallocated."""
    dev = a.device
    a = _want(a, torch.float32, "a")
    pos_ij = _want(pos_ij, torch.float32, "pos_ij", dev)
    tvecs = _want(tvecs, torch.float32, "tvecs", dev)
    batch, edges = _want(batch, torch.int64, "batch", dev), _want(edges, torch.int64, "edges", dev)
    W, rvlen = _want(W, torch.float32, "W", dev), _want(rvlen, torch.float32, "rvlen", dev)
    E, H, N = edges.shape[1], a.shape[1], batch.shape[0]
    _check_projection(W, H, K, "lattice_sum_fwd")
    if W is not None:
        W_num = 1 if W.dim() == 3 else W.shape[0]
        Dv = W.shape[-2]
    else:
        W_num, Dv = 0, 0
    if z is None:
        z = torch.empty((E, H), dtype=torch.float32, device=dev)
    if K > 0 and v is None:
        v = torch.empty((E, H, Dv if W is not None else K), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_lattice_sum_fwd", _ptr(a), c_int(int(a_per_edge)), _ptr(pos_ij), _ptr(tvecs), _ptr(batch),
                  _ptr(edges), c_int64(N), c_int64(H), c_int64(E), c_int64(K), c_double(dist_max), c_double(wscale),
                  _ptr(W), c_int64(W_num), c_int64(Dv), _ptr(rvlen), c_double(cutoff_radius or 0.0),
                  c_int(lattice_range), c_int(minimum_range), _ptr(z), _ptr(v if K > 0 else None), _stream(dev))
    return z, (v if K > 0 else None)


def lattice_sum_bwd(a, pos_ij, tvecs, batch, edges, row_start, z, gz, gv, K, dist_max, wscale, W=None, rvlen=None,
                    cutoff_radius=0.0, lattice_range=2, minimum_range=2):
    """ga (N,H) and gW (shape of W; None without W).  gv is the gradient of psi (E,H,K) when W is None, else of
    W psi (E,H,Dv).  The projection is handled around the kernel with two GEMM-shaped torch calls:
    gpsi = W^T gv before it, gW = sum_e gv_e (x) psi_e after it (psi recomputed by the kernel)."""
    dev = a.device
    a = _want(a, torch.float32, "a")
    pos_ij = _want(pos_ij, torch.float32, "pos_ij", dev)
    tvecs = _want(tvecs, torch.float32, "tvecs", dev)
    batch, edges = _want(batch, torch.int64, "batch", dev), _want(edges, torch.int64, "edges", dev)
    row_start = _want(row_start, torch.int64, "row_start", dev)
    z, gz, gv = (_want(t, torch.float32, n, dev) for t, n in ((z, "z"), (gz, "gz"), (gv, "gv")))
    W, rvlen = _want(W, torch.float32, "W", dev), _want(rvlen, torch.float32, "rvlen", dev)
    E, H, N = edges.shape[1], a.shape[1], batch.shape[0]
    ga = torch.empty((N, H), dtype=torch.float32, device=dev)
    scratch = torch.empty((E, H), dtype=torch.float32, device=dev)
    gpsi = psi = None
    if K > 0:
        if W is None:
            gpsi = gv
        else:
            W4 = W if W.dim() == 4 else W[None]
            W_num = W4.shape[0]
            if W_num == 1:
                gpsi = torch.einsum("ehd,hdk->ehk", gv, W4[0]).contiguous()
            elif W_num == E:
                gpsi = torch.einsum("ehd,ehdk->ehk", gv, W4).contiguous()
            elif W_num == N:
                gpsi = torch.einsum("ehd,ehdk->ehk", gv, W4[edges[0]]).contiguous()
            else:
                raise ValueError(f"W_num={W_num} must be 1, E or N")
            psi = torch.empty((E, H, K), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_lattice_sum_bwd", _ptr(a), _ptr(pos_ij), _ptr(tvecs), _ptr(batch), _ptr(edges), _ptr(row_start),
                  _ptr(z), _ptr(gz), _ptr(gpsi), c_int64(N), c_int64(H), c_int64(E), c_int64(K), c_double(dist_max),
                  c_double(wscale), _ptr(rvlen), c_double(cutoff_radius or 0.0), c_int(lattice_range),
                  c_int(minimum_range), _ptr(ga), _ptr(psi), _ptr(scratch), _stream(dev))
    gW = None
    if psi is not None:
        if W_num == 1:
            gW = torch.einsum("ehd,ehk->hdk", gv, psi)[None]
        elif W_num == E:
            gW = gv[..., :, None] * psi[..., None, :]
        else:
            gW = torch.zeros((N,) + tuple(W4.shape[1:]), dtype=torch.float32, device=dev)
            gW.index_add_(0, edges[0], gv[..., :, None] * psi[..., None, :])
        if W.dim() == 3:
            gW = gW[0]
    return ga, gW


def fused_attn_fwd(q, k, v, aij, bij, edges, row_start):
    """prob (E,H), out (N,H,D); q already divided by sqrt(D)."""
    dev = q.device
    q, k, v = (_want(t, torch.float32, n, dev) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    aij, bij = _want(aij, torch.float32, "aij", dev), _want(bij, torch.float32, "bij", dev)
    edges, row_start = _want(edges, torch.int64, "edges", dev), _want(row_start, torch.int64, "row_start", dev)
    N, H, D = q.shape
    E = edges.shape[1]
    prob = torch.empty((E, H), dtype=torch.float32, device=dev)
    out = torch.empty((N, H, D), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_fused_attn_fwd", _ptr(q), _ptr(k), _ptr(v), _ptr(aij), _ptr(bij), _ptr(edges), _ptr(row_start),
                  c_int64(N), c_int64(H), c_int64(D), c_int64(E), _ptr(prob), _ptr(out), _stream(dev))
    return prob, out


def fused_attn_bwd(q, k, v, bij, edges, row_start, prob, out, gout):
    """(gq, gk, gv, gaij, gbij); gq is with respect to the pre-scaled q."""
    dev = q.device
    q, k, v, prob, out, gout = (_want(t, torch.float32, n, dev) for t, n in
                                ((q, "q"), (k, "k"), (v, "v"), (prob, "prob"), (out, "out"), (gout, "gout")))
    bij = _want(bij, torch.float32, "bij", dev)
    edges, row_start = _want(edges, torch.int64, "edges", dev), _want(row_start, torch.int64, "row_start", dev)
    N, H, D = q.shape
    E = edges.shape[1]
    gq, gk, gv = (torch.empty_like(q) for _ in range(3))
    gaij = torch.empty((E, H), dtype=torch.float32, device=dev)
    gbij = torch.empty((E, H, D), dtype=torch.float32, device=dev) if bij is not None else None
    with torch.cuda.device(dev):
        _lib.call("cf_fused_attn_bwd", _ptr(q), _ptr(k), _ptr(v), _ptr(bij), _ptr(edges), _ptr(row_start), c_int64(N),
                  c_int64(H), c_int64(D), c_int64(E), _ptr(prob), _ptr(out), _ptr(gout), _ptr(gq), _ptr(gk), _ptr(gv),
                  _ptr(gaij), _ptr(gbij), _stream(dev))
    return gq, gk, gv, gaij, gbij


def term_list_build(pos_ij, tvecs, rvlen, batch, edges, row_start, max_atoms, cutoff_radius, lattice_range,
                    minimum_range, a_widest, row_order=None):
    """Term lists of a batch (see cf_term_list_build): (workspace tensor, a_widest), to be handed to
    ``infinite_attn_fwd(..., term_lists=...)`` for every layer of the batch."""
    dev = pos_ij.device
    pos_ij, tvecs, rvlen = (_want(t, torch.float32, n, dev) for t, n in ((pos_ij, "pos_ij"), (tvecs, "tvecs"), (rvlen, "rvlen")))
    batch, edges, row_start = (_want(t, torch.int64, n, dev) for t, n in
                               ((batch, "batch"), (edges, "edges"), (row_start, "row_start")))
    N, E = batch.shape[0], edges.shape[1]
    work = torch.empty(int(_lib.load().cf_term_list_workspace_bytes(N, E)), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_term_list_build", _ptr(pos_ij), _ptr(tvecs), _ptr(rvlen), _ptr(batch), _ptr(edges), _ptr(row_start),
                  _ptr(_want(row_order, torch.int32, "row_order", dev)), c_int64(N), c_int64(E), c_int64(max_atoms),
                  c_double(cutoff_radius or 0.0), c_int(lattice_range), c_int(minimum_range), c_double(a_widest),
                  _ptr(work), _stream(dev))
    return work, float(a_widest)


def row_list_build(pos_ij, tvecs, rvlen, batch, edges, row_start, max_atoms, cutoff_radius, lattice_range,
                   minimum_range, a_widest, row_order=None):
    """Row lists of a batch of crystals of at most 64 atoms (see cf_row_list_build): the workspace tensor to hand to
    ``infinite_attn_fwd_sorted`` for every layer of the batch."""
    dev = pos_ij.device
    pos_ij, tvecs, rvlen = (_want(t, torch.float32, n, dev) for t, n in ((pos_ij, "pos_ij"), (tvecs, "tvecs"), (rvlen, "rvlen")))
    batch, edges, row_start = (_want(t, torch.int64, n, dev) for t, n in
                               ((batch, "batch"), (edges, "edges"), (row_start, "row_start")))
    N, E = batch.shape[0], edges.shape[1]
    work = torch.empty(int(_lib.load().cf_row_list_workspace_bytes(N, E)), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_row_list_build", _ptr(pos_ij), _ptr(tvecs), _ptr(rvlen), _ptr(batch), _ptr(edges), _ptr(row_start),
                  _ptr(_want(row_order, torch.int32, "row_order", dev)), c_int64(N), c_int64(E), c_int64(max_atoms),
                  c_double(cutoff_radius or 0.0), c_int(lattice_range), c_int(minimum_range), c_double(a_widest),
                  _ptr(work), _stream(dev))
    return work


def infinite_attn_fwd_sorted(q, k, v, a, pos_ij, tvecs, rvlen, batch, edges, row_start, max_atoms, K, dist_max, wscale,
                             W, cutoff_radius, lattice_range, minimum_range, row_lists):
    """Fused attention forward over a batch's row lists (inference; crystals of at most 64 atoms, K = 64 or 0).
    Returns (out (N,H,D), lse (N,H))."""
    dev = q.device
    q, k, v, a, tvecs = (_want(t, torch.float32, n, dev) for t, n in
                         ((q, "q"), (k, "k"), (v, "v"), (a, "a"), (tvecs, "tvecs")))
    pos_ij, rvlen, W = (_want(t, torch.float32, n, dev) for t, n in ((pos_ij, "pos_ij"), (rvlen, "rvlen"), (W, "W")))
    batch, edges, row_start = (_want(t, torch.int64, n, dev) for t, n in
                               ((batch, "batch"), (edges, "edges"), (row_start, "row_start")))
    N, H, D = q.shape
    _check_projection(W, H, K, "infinite_attn_fwd_sorted")
    E, B = edges.shape[1], tvecs.shape[0]
    out = torch.empty((N, H, D), dtype=torch.float32, device=dev)
    lse = torch.empty((N, H), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_infinite_attn_fwd_sorted", _ptr(q), _ptr(k), _ptr(v), _ptr(a), _ptr(pos_ij), _ptr(tvecs), _ptr(rvlen),
                  _ptr(batch), _ptr(edges), _ptr(row_start), c_int64(N), c_int64(B), c_int64(H), c_int64(D), c_int64(E),
                  c_int64(K), c_int64(max_atoms), c_double(dist_max), c_double(wscale), _ptr(W),
                  c_double(cutoff_radius or 0.0), c_int(lattice_range), c_int(minimum_range), _ptr(out), _ptr(lse),
                  _ptr(row_lists), _stream(dev))
    return out, lse


def infinite_attn_fwd(q, k, v, a, pos_ij, tvecs, rvlen, batch, edges, row_start, max_atoms, K, dist_max, wscale, W,
                      cutoff_radius, lattice_range, minimum_range, want_psi_row=False, pos=None, row_order=None,
                      term_lists=None):
    """Fused attention forward.  Geometry as pos_ij (E,3), or pos (N,3) when pos_ij is None.  ``term_lists`` (from
    ``term_list_build``, needs pos_ij) replaces the enumeration of translations by the batch's precomputed lists.
    Returns (out (N,H,D), logit (E,H), lse (N,H), psi_row (N,H,K) or None)."""
    dev = q.device
    q, k, v, a, tvecs = (_want(t, torch.float32, n, dev) for t, n in
                         ((q, "q"), (k, "k"), (v, "v"), (a, "a"), (tvecs, "tvecs")))
    pos_ij, pos = _want(pos_ij, torch.float32, "pos_ij", dev), _want(pos, torch.float32, "pos", dev)
    rvlen, W = _want(rvlen, torch.float32, "rvlen", dev), _want(W, torch.float32, "W", dev)
    batch, edges, row_start = (_want(t, torch.int64, n, dev) for t, n in
                               ((batch, "batch"), (edges, "edges"), (row_start, "row_start")))
    N, H, D = q.shape
    _check_projection(W, H, K, "infinite_attn_fwd")
    E, B = edges.shape[1], tvecs.shape[0]
    out = torch.empty((N, H, D), dtype=torch.float32, device=dev)
    logit = torch.empty((E, H), dtype=torch.float32, device=dev)
    lse = torch.empty((N, H), dtype=torch.float32, device=dev)
    psi_row = torch.empty((N, H, K), dtype=torch.float32, device=dev) if (want_psi_row and K > 0) else None
    if term_lists is not None:
        work, a_widest = term_lists
        with torch.cuda.device(dev):
            _lib.call("cf_infinite_attn_fwd_listed", _ptr(q), _ptr(k), _ptr(v), _ptr(a), _ptr(pos_ij), _ptr(tvecs),
                      _ptr(rvlen), _ptr(batch), _ptr(edges), _ptr(row_start), c_int64(N), c_int64(B), c_int64(H),
                      c_int64(D), c_int64(E), c_int64(K), c_int64(max_atoms), c_double(dist_max), c_double(wscale),
                      _ptr(W), c_double(cutoff_radius or 0.0), c_int(lattice_range), c_int(minimum_range), _ptr(out),
                      _ptr(logit), _ptr(lse), _ptr(psi_row), _ptr(_want(row_order, torch.int32, "row_order", dev)),
                      _ptr(work), c_double(a_widest), _stream(dev))
        return out, logit, lse, psi_row
    with torch.cuda.device(dev):
        _lib.call("cf_infinite_attn_fwd", _ptr(q), _ptr(k), _ptr(v), _ptr(a), _ptr(pos), _ptr(pos_ij), _ptr(tvecs),
                  _ptr(rvlen), _ptr(batch), _ptr(edges), _ptr(row_start), c_int64(N), c_int64(B), c_int64(H),
                  c_int64(D), c_int64(E), c_int64(K), c_int64(max_atoms), c_double(dist_max), c_double(wscale), _ptr(W),
                  c_double(cutoff_radius or 0.0), c_int(lattice_range), c_int(minimum_range), _ptr(out), _ptr(logit),
                  _ptr(lse), _ptr(psi_row), _ptr(_want(row_order, torch.int32, "row_order", dev)), _stream(dev))
    return out, logit, lse, psi_row


def infinite_attn_bwd(q, k, v, a, pos_ij, tvecs, rvlen, batch, edges, row_start, max_atoms, K, dist_max, wscale, W,
                      cutoff_radius, lattice_range, minimum_range, logit, lse, out, gout, pos=None, row_order=None,
                      term_lists=None):
    """Backward of infinite_attn_fwd: (gq, gk, gv, ga).  gq is with respect to the pre-scaled q.  ``term_lists``: the
    lists the forward was given (needs pos_ij)."""
    dev = q.device
    q, k, v, a, tvecs, logit, lse, out, gout = (_want(t, torch.float32, n, dev) for t, n in (
        (q, "q"), (k, "k"), (v, "v"), (a, "a"), (tvecs, "tvecs"), (logit, "logit"), (lse, "lse"), (out, "out"),
        (gout, "gout")))
    pos_ij, pos = _want(pos_ij, torch.float32, "pos_ij", dev), _want(pos, torch.float32, "pos", dev)
    rvlen, W = _want(rvlen, torch.float32, "rvlen", dev), _want(W, torch.float32, "W", dev)
    batch, edges, row_start = (_want(t, torch.int64, n, dev) for t, n in
                               ((batch, "batch"), (edges, "edges"), (row_start, "row_start")))
    N, H, D = q.shape
    _check_projection(W, H, K, "infinite_attn_bwd")
    E, B = edges.shape[1], tvecs.shape[0]
    gq, gk, gv = (torch.empty_like(q) for _ in range(3))
    ga = torch.empty((N, H), dtype=torch.float32, device=dev)
    glogit = torch.empty((E, H), dtype=torch.float32, device=dev)
    if term_lists is not None:
        work, a_widest = term_lists
        with torch.cuda.device(dev):
            _lib.call("cf_infinite_attn_bwd_listed", _ptr(q), _ptr(k), _ptr(v), _ptr(a), _ptr(pos_ij), _ptr(tvecs),
                      _ptr(rvlen), _ptr(batch), _ptr(edges), _ptr(row_start), c_int64(N), c_int64(B), c_int64(H),
                      c_int64(D), c_int64(E), c_int64(K), c_int64(max_atoms), c_double(dist_max), c_double(wscale),
                      _ptr(W), c_double(cutoff_radius or 0.0), c_int(lattice_range), c_int(minimum_range), _ptr(logit),
                      _ptr(lse), _ptr(out), _ptr(gout), _ptr(gq), _ptr(gk), _ptr(gv), _ptr(ga), _ptr(glogit),
                      _ptr(_want(row_order, torch.int32, "row_order", dev)), _ptr(work), c_double(a_widest), _stream(dev))
        return gq, gk, gv, ga
    with torch.cuda.device(dev):
        _lib.call("cf_infinite_attn_bwd", _ptr(q), _ptr(k), _ptr(v), _ptr(a), _ptr(pos), _ptr(pos_ij), _ptr(tvecs),
                  _ptr(rvlen), _ptr(batch), _ptr(edges), _ptr(row_start), c_int64(N), c_int64(B), c_int64(H),
                  c_int64(D), c_int64(E), c_int64(K), c_int64(max_atoms), c_double(dist_max), c_double(wscale), _ptr(W),
                  c_double(cutoff_radius or 0.0), c_int(lattice_range), c_int(minimum_range), _ptr(logit), _ptr(lse),
                  _ptr(out), _ptr(gout), _ptr(gq), _ptr(gk), _ptr(gv), _ptr(ga), _ptr(glogit),
                  _ptr(_want(row_order, torch.int32, "row_order", dev)), _stream(dev))
    return gq, gk, gv, ga


def row_cost(atom_start, trans, N: int, reach: float = 15.0):
    """(N,) float32 scheduling weights of the atoms' rows (see cf_row_cost)."""
    dev = trans.device
    atom_start, trans = _want(atom_start, torch.int64, "atom_start", dev), _want(trans, torch.float32, "trans", dev)
    cost = torch.empty((N,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_row_cost", _ptr(atom_start), _ptr(trans), c_int64(trans.shape[0]), c_int64(N), c_double(reach),
                  _ptr(cost), _stream(dev))
    return cost


ROW_ORDER_MAX_CRYSTALS = 2048


def row_order(atom_start, trans, N: int, reach: float = 15.0):
    """(N,) int32: the atoms by descending scheduling weight, ties by index (see cf_row_order / cf_row_cost)."""
    dev = trans.device
    atom_start, trans = _want(atom_start, torch.int64, "atom_start", dev), _want(trans, torch.float32, "trans", dev)
    B = trans.shape[0]
    if B > ROW_ORDER_MAX_CRYSTALS:
        return torch.argsort(row_cost(atom_start, trans, N, reach), descending=True, stable=True).to(torch.int32)
    order = torch.empty((N,), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_row_order", _ptr(atom_start), _ptr(trans), c_int64(B), c_int64(N), c_double(reach), _ptr(order),
                  _stream(dev))
    return order


def reci_phase(pos_ij, rvecs, batch, edges):
    """kr_base (E,3) = rvecs[crystal of the edge] . pos_ij."""
    dev = pos_ij.device
    pos_ij, rvecs = _want(pos_ij, torch.float32, "pos_ij", dev), _want(rvecs, torch.float32, "rvecs", dev)
    batch, edges = _want(batch, torch.int64, "batch", dev), _want(edges, torch.int64, "edges", dev)
    E = edges.shape[1]
    kr = torch.empty((E, 3), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_reci_phase", _ptr(pos_ij), _ptr(rvecs), _ptr(batch), _ptr(edges), c_int64(E), _ptr(kr), _stream(dev))
    return kr


def reci_sum_fwd(a, kr_base, rvecs, vcell, batch, row_start, E: int, lattice_range: int):
    """phi (E,H) and the raw sum S (E,H) of the reciprocal-space lattice sum."""
    dev = a.device
    a, kr_base, rvecs, vcell = (_want(t, torch.float32, n, dev) for t, n in
                                ((a, "a"), (kr_base, "kr_base"), (rvecs, "rvecs"), (vcell, "vcell")))
    batch, row_start = _want(batch, torch.int64, "batch", dev), _want(row_start, torch.int64, "row_start", dev)
    N, H = a.shape
    z = torch.empty((E, H), dtype=torch.float32, device=dev)
    s = torch.empty((E, H), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_reci_sum_fwd", _ptr(a), _ptr(kr_base), _ptr(rvecs), _ptr(vcell), _ptr(batch), _ptr(row_start),
                  c_int64(N), c_int64(H), c_int64(E), c_int(lattice_range), _ptr(z), _ptr(s), _stream(dev))
    return z, s


def reci_sum_bwd(a, kr_base, rvecs, batch, row_start, gz, sumexp, lattice_range: int):
    """ga (N,H); the 1.5 log(-4 pi a) term of phi is not differentiated (as in the reference's kernel)."""
    dev = a.device
    a, kr_base, rvecs, gz, sumexp = (_want(t, torch.float32, n, dev) for t, n in
                                     ((a, "a"), (kr_base, "kr_base"), (rvecs, "rvecs"), (gz, "gz"), (sumexp, "sumexp")))
    batch, row_start = _want(batch, torch.int64, "batch", dev), _want(row_start, torch.int64, "row_start", dev)
    N, H = a.shape
    E = gz.shape[0]
    ga = torch.empty((N, H), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_reci_sum_bwd", _ptr(a), _ptr(kr_base), _ptr(rvecs), _ptr(batch), _ptr(row_start), _ptr(gz),
                  _ptr(sumexp), c_int64(N), c_int64(H), c_int64(E), c_int(lattice_range), _ptr(ga), _stream(dev))
    return ga


def segment_mean(x, start):
    """Per-crystal mean: x (N,D) float32, start (B+1) int64 atom offsets -> (B,D)."""
    dev = x.device
    x = _want(x, torch.float32, "x")
    start = _want(start, torch.int64, "start", dev)
    B = start.shape[0] - 1
    D = x.numel() // max(x.shape[0], 1)
    out = torch.empty((B,) + tuple(x.shape[1:]), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.call("cf_segment_mean_fwd", _ptr(x), _ptr(start), c_int64(B), c_int64(D), _ptr(out), _stream(dev))
    return out


def pipe_probe(kind: int, blocks: int, threads: int, iters: int, sink: torch.Tensor) -> None:
    with torch.cuda.device(sink.device):
        _lib.call("cf_pipe_probe", c_int(kind), c_int(blocks), c_int(threads), c_int64(iters), _ptr(sink),
                  _stream(sink.device))
