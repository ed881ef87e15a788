"""CPU oracle for the infinitely-connected-attention hot path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` may import this
package; the shipped ``crystalformer_b200`` package never does and fails loudly without its CUDA library.

Two libraries back it, both loaded with ctypes and fed numpy arrays:

* ``libcf_oracle.so``  - ``cf_oracle.c``, a plain-C restatement of the reference kernels (float build ``f32`` with the
  reference's loop order, double build ``f64`` as arbiter).  Built by ``make`` in this directory.
* ``_ref/libcfref_k{64,0}.so`` - the reference project's *own* kernel sources compiled for the CPU by ``make ref``
  (needs the reference tree at build time; the built files are not in version control).  ``have_ref()`` says whether
  they are present.

Parity status: pinned.  ``tests/test_oracle_golden.py`` checks the C restatement against vectors produced by the
reference's PyTorch implementation (``tests/golden/``) and against the compiled reference kernels.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_double, c_int, c_longlong, c_void_p
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB: Optional[ctypes.CDLL] = None
_REF = {}


def build(ref: bool = True) -> None:
    """Compile the oracle (and the CPU build of the reference kernels when the reference tree is present)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)
    if ref and os.path.isdir(os.environ.get("CF_REFERENCE_ROOT", "/root/reference")):
        subprocess.run(["make", "-s", "-C", _HERE, "ref",
                        "REFERENCE=" + os.environ.get("CF_REFERENCE_ROOT", "/root/reference")], check=True)


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libcf_oracle.so")
        if not os.path.exists(path):
            build(ref=False)
        _LIB = ctypes.CDLL(path)
    return _LIB


def have_ref() -> bool:
    return all(os.path.exists(os.path.join(_HERE, "_ref", f"libcfref_k{k}.so")) for k in (64, 0))


def ref_lib(K: int) -> ctypes.CDLL:
    """The reference kernels compiled for the CPU with VPE_DIM = K (64 or 0), H = 8, D = 16, LATTICE_RANGE = 2."""
    if K not in _REF:
        _REF[K] = ctypes.CDLL(os.path.join(_HERE, "_ref", f"libcfref_k{K}.so"))
    return _REF[K]


def _p(x):
    return c_void_p(x.ctypes.data) if x is not None else c_void_p(0)


def _f32(x):
    return None if x is None else np.ascontiguousarray(x, dtype=np.float32)


def _i64(x):
    return None if x is None else np.ascontiguousarray(x, dtype=np.int64)


def _real(x, dtype):
    return None if x is None else np.ascontiguousarray(x, dtype=dtype)


def _np_dtype(precision: str):
    return {"f32": np.float32, "f64": np.float64}[precision]


def row_starts(edges: np.ndarray, N: int) -> np.ndarray:
    """CSR offsets of the edge list by source atom (models/cuda_funcs/fused_dpa.py:24-26)."""
    counts = np.bincount(np.asarray(edges[0], dtype=np.int64), minlength=N)
    return np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)


# ------------------------------------------------------------------------------------------------ restatement

def box(a, rvlen3, cutoff_radius, lattice_range, minimum_range):
    a = _f32(a).reshape(-1)
    rvlen3 = _f32(rvlen3)
    out = np.zeros((a.shape[0], 3), dtype=np.int32)
    lib().cfo_box_f32(_p(a), c_longlong(a.shape[0]), _p(rvlen3), c_double(cutoff_radius),
                      c_int(lattice_range), c_int(minimum_range), _p(out))
    return out


def edge_index(sizes):
    sizes = _i64(sizes)
    E = int((sizes * sizes).sum())
    edges = np.zeros((2, E), dtype=np.int64)
    lib().cfo_edge_index_f32(_p(sizes), c_longlong(sizes.shape[0]), _p(edges), c_longlong(E))
    return edges


def geometry(pos, trans, edges):
    pos, trans, edges = _f32(pos), _f32(trans), _i64(edges)
    B, E = trans.shape[0], edges.shape[1]
    pos_ij = np.zeros((E, 3), np.float32)
    rvecs = np.zeros((B, 3, 3), np.float32)
    vcell = np.zeros((B,), np.float32)
    rvlen = np.zeros((B, 3), np.float32)
    lib().cfo_geometry_f32(_p(pos), _p(trans), _p(edges), c_longlong(B), c_longlong(E), _p(pos_ij), _p(rvecs),
                           _p(vcell), _p(rvlen))
    return pos_ij, rvecs, vcell, rvlen


def lattice_sum_fwd(a, pos_ij, tvecs, batch, edges, K, dist_max, wscale, W=None, rvlen=None, cutoff_radius=0.0,
                    lattice_range=2, minimum_range=2, a_per_edge=False, nested=False, precision="f32",
                    return_box=False):
    """phi (E,H) and psi (E,H,K) or W psi (E,H,Dv); see cf_oracle.c cfo_lattice_sum_fwd."""
    dt = _np_dtype(precision)
    a, pos_ij, tvecs, batch, edges = _f32(a), _f32(pos_ij), _f32(tvecs), _i64(batch), _i64(edges)
    W, rvlen = _f32(W), _f32(rvlen)
    H, E, N = a.shape[1], edges.shape[1], batch.shape[0]
    if W is not None:
        if W.ndim == 3:
            W = W[None]
        W_num, Dv = W.shape[0], W.shape[2]
    else:
        W_num, Dv = 0, 0
    z = np.zeros((E, H), dt)
    v = np.zeros((E, H, Dv if W is not None else K), dt) if K > 0 else None
    bx = np.zeros((E, H, 3), np.int32) if return_box else None
    fn = getattr(lib(), f"cfo_lattice_sum_fwd_{precision}")
    fn(_p(a), c_int(int(a_per_edge)), _p(pos_ij), _p(tvecs), _p(batch), _p(edges), c_longlong(N), c_longlong(H),
       c_longlong(E), c_longlong(K), c_double(dist_max), c_double(wscale), _p(W), c_longlong(W_num), c_longlong(Dv),
       _p(rvlen), c_double(cutoff_radius), c_int(lattice_range), c_int(minimum_range), c_int(int(nested)), _p(z),
       _p(v), _p(bx))
    return (z, v, bx) if return_box else (z, v)


def lattice_sum_bwd(a, pos_ij, tvecs, batch, edges, z, gz, gv, K, dist_max, wscale, W=None, rvlen=None,
                    cutoff_radius=0.0, lattice_range=2, minimum_range=2, precision="f32"):
    """ga (N,H) and gW (W_num,H,Dv,K) (None without W); see cf_oracle.c cfo_lattice_sum_bwd."""
    dt = _np_dtype(precision)
    a, pos_ij, tvecs, batch, edges = _f32(a), _f32(pos_ij), _f32(tvecs), _i64(batch), _i64(edges)
    W, rvlen = _f32(W), _f32(rvlen)
    N, H, E = a.shape[0], a.shape[1], edges.shape[1]
    e_start = row_starts(edges, N)
    if W is not None:
        if W.ndim == 3:
            W = W[None]
        W_num, Dv = W.shape[0], W.shape[2]
        gW = np.zeros((W_num, H, Dv, K), dt)
    else:
        W_num, Dv, gW = 0, 0, None
    ga = np.zeros((N, H), dt)
    z, gz, gv = _real(z, dt), _real(gz, dt), _real(gv, dt)  # keep the converted copies alive across the call
    fn = getattr(lib(), f"cfo_lattice_sum_bwd_{precision}")
    fn(_p(a), _p(pos_ij), _p(tvecs), _p(batch), _p(edges), _p(e_start), _p(z), _p(gz),
       _p(gv), c_longlong(N), c_longlong(H), c_longlong(E), c_longlong(K), c_double(dist_max),
       c_double(wscale), _p(W), c_longlong(W_num), c_longlong(Dv), _p(rvlen), c_double(cutoff_radius),
       c_int(lattice_range), c_int(minimum_range), _p(ga), _p(gW))
    return ga, gW


def fused_attn_fwd(q, k, v, aij, bij, edges, run_len=8, max_sys_pow2=512, precision="f32"):
    """prob (E,H) and out (N,H,D); q already divided by sqrt(D); see cf_oracle.c cfo_fused_attn_fwd."""
    dt = _np_dtype(precision)
    q, k, v, aij, bij = (_real(t, dt) for t in (q, k, v, aij, bij))
    edges = _i64(edges)
    N, H, D = q.shape
    E = edges.shape[1]
    e_start = row_starts(edges, N)
    need = int(np.diff(e_start).max()) if N else 0
    while max_sys_pow2 < need:
        max_sys_pow2 *= 2
    prob = np.zeros((E, H), dt)
    out = np.zeros((N, H, D), dt)
    fn = getattr(lib(), f"cfo_fused_attn_fwd_{precision}")
    fn(_p(q), _p(k), _p(v), _p(aij), _p(bij), _p(edges), _p(e_start), c_longlong(N), c_longlong(H), c_longlong(E),
       c_longlong(D), c_int(run_len), c_int(max_sys_pow2), _p(prob), _p(out))
    return prob, out


def fused_attn_bwd(q, k, v, bij, edges, prob, out, go, precision="f32"):
    """(gq, gk, gv, gaij, gbij); see cf_oracle.c cfo_fused_attn_bwd."""
    dt = _np_dtype(precision)
    q, k, v, bij, prob, out, go = (_real(t, dt) for t in (q, k, v, bij, prob, out, go))
    edges = _i64(edges)
    N, H, D = q.shape
    E = edges.shape[1]
    e_start = row_starts(edges, N)
    gq, gk, gv = (np.zeros((N, H, D), dt) for _ in range(3))
    gaij = np.zeros((E, H), dt)
    gbij = np.zeros((E, H, D), dt) if bij is not None else None
    fn = getattr(lib(), f"cfo_fused_attn_bwd_{precision}")
    fn(_p(q), _p(k), _p(v), _p(bij), _p(edges), _p(e_start), c_longlong(N), c_longlong(H), c_longlong(E),
       c_longlong(D), _p(prob), _p(out), _p(go), _p(gq), _p(gk), _p(gv), _p(gaij), _p(gbij))
    return gq, gk, gv, gaij, gbij


def segment_mean(x, sizes, precision="f32"):
    dt = _np_dtype(precision)
    x = _real(x, dt)
    sizes = _i64(sizes)
    start = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    B, D = sizes.shape[0], x.shape[1]
    out = np.zeros((B, D), dt)
    getattr(lib(), f"cfo_segment_mean_{precision}")(_p(x), _p(start), c_longlong(B), c_longlong(D), _p(out))
    return out


# ------------------------------------------------------------------------------------ reference kernels on the CPU

def ref_real_enc_proj_fwd(a, pos_ij, tvecs, batch, edges, K, dist_max, wscale, W, rvlen, cutoff_radius, proj=True):
    """Runs the reference's real_enc_proj_fwd (proj=True) or real_enc_fwd kernel source on the CPU.
    Launch shape as models/cuda_funcs/real_space_enc_proj.py:53,72: grid E, block H."""
    a, pos_ij, tvecs, batch, edges, W, rvlen = _f32(a), _f32(pos_ij), _f32(tvecs), _i64(batch), _i64(edges), _f32(W), _f32(rvlen)
    N, H = a.shape
    E = edges.shape[1]
    L = ref_lib(K)
    z = np.zeros((E, H), np.float32)
    if proj:
        W_num = 0 if W is None else (1 if W.ndim == 3 else W.shape[0])
        Dv = 0 if W is None else W.shape[-2]
        v = np.zeros((E, H, Dv if W is not None else K), np.float32) if K > 0 else None
        L.cfref_real_enc_proj_fwd(c_longlong(E), c_int(H), _p(a), _p(pos_ij), c_void_p(0), _p(tvecs), _p(batch),
                                  _p(edges), c_longlong(N), c_longlong(H), c_longlong(E), c_longlong(K),
                                  c_double(dist_max), c_double(wscale), _p(W), c_longlong(W_num), _p(rvlen),
                                  c_double(cutoff_radius), _p(z), _p(v))
    else:
        v = np.zeros((E, H, K), np.float32) if K > 0 else None
        L.cfref_real_enc_fwd(c_longlong(E), c_int(H), _p(a), _p(pos_ij), c_void_p(0), _p(tvecs), _p(batch), _p(edges),
                             c_longlong(N), c_longlong(H), c_longlong(E), c_longlong(K), c_double(dist_max),
                             c_double(wscale), _p(rvlen), c_double(cutoff_radius), _p(z), _p(v))
    return z, v


def ref_real_enc_proj_bwd(a, pos_ij, tvecs, batch, edges, z, gz, gv, K, dist_max, wscale, W, rvlen, cutoff_radius,
                          proj=True):
    """Reference real_enc_proj_bwd / real_enc_bwd kernel source on the CPU (grid N, block H).  With W_num == 1 the
    kernel writes one (H,Dv,K) block per atom (models/cuda_funcs/real_space_enc_proj.py:127); they are summed here."""
    a, pos_ij, tvecs, batch, edges, W, rvlen = _f32(a), _f32(pos_ij), _f32(tvecs), _i64(batch), _i64(edges), _f32(W), _f32(rvlen)
    z, gz, gv = _f32(z), _f32(gz), _f32(gv)
    N, H = a.shape
    E = edges.shape[1]
    e_start = row_starts(edges, N)
    L = ref_lib(K)
    ga = np.zeros((N, H), np.float32)
    if proj:
        W_num = 0 if W is None else (1 if W.ndim == 3 else W.shape[0])
        gW = np.zeros((max(W_num, N),) + W.shape[-3:], np.float32) if W is not None else None
        L.cfref_real_enc_proj_bwd(c_longlong(N), c_int(H), _p(a), _p(pos_ij), _p(tvecs), _p(batch), _p(edges),
                                  _p(e_start), _p(z), _p(gz), _p(gv), c_longlong(N), c_longlong(H), c_longlong(E),
                                  c_double(dist_max), c_double(wscale), _p(W), c_longlong(W_num), _p(rvlen),
                                  c_double(cutoff_radius), _p(ga), _p(gW))
        if gW is not None and W_num == 1:
            gW = gW.sum(axis=0, keepdims=True)
        return ga, gW
    L.cfref_real_enc_bwd(c_longlong(N), c_int(H), _p(a), _p(pos_ij), _p(tvecs), _p(batch), _p(edges), _p(e_start),
                         _p(z), _p(gz), _p(gv), c_longlong(N), c_longlong(H), c_longlong(E), c_longlong(K),
                         c_double(dist_max), c_double(wscale), _p(rvlen), c_double(cutoff_radius), _p(ga))
    return ga, None


def ref_fused_dpa_fwd(q, k, v, aij, bij, edges, v3=True, K=64):
    q, k, v, aij, bij, edges = _f32(q), _f32(k), _f32(v), _f32(aij), _f32(bij), _i64(edges)
    N, H, D = q.shape
    E = edges.shape[1]
    e_start = row_starts(edges, N)
    prob = np.zeros((E, H), np.float32)
    out = np.zeros((N, H, D), np.float32)
    ref_lib(K).cfref_fused_dpa_fwd(c_longlong(N), c_int(H), c_int(int(v3)), _p(q), _p(k), _p(v), _p(aij), _p(bij),
                                   _p(edges), _p(e_start), c_longlong(N), c_longlong(H), c_longlong(E), _p(prob),
                                   _p(out))
    return prob, out


def _transpose_blocks(x, sizes):
    """(i,j) <-> (j,i) inside every crystal's n x n block of a per-edge array (what irregular_transpose does)."""
    out = np.empty_like(x)
    c = 0
    for n in sizes:
        n = int(n)
        blk = x[c:c + n * n].reshape((n, n) + x.shape[1:])
        out[c:c + n * n] = np.swapaxes(blk, 0, 1).reshape((n * n,) + x.shape[1:])
        c += n * n
    return out


def ref_fused_dpa_bwd(q, k, v, aij, bij, batch, edges, sizes, prob, out, go, K=64):
    """Reference fused_dpa_bwd + fused_dpa_bwd_q kernel sources on the CPU, with the key-major transposes the
    reference's host code performs around them (models/cuda_funcs/fused_dpa.py:157-206) done in numpy."""
    q, k, v, aij, bij, prob, out, go = (_f32(t) for t in (q, k, v, aij, bij, prob, out, go))
    batch, edges = _i64(batch), _i64(edges)
    N, H, D = q.shape
    E = edges.shape[1]
    e_start = row_starts(edges, N)
    tprob = _transpose_blocks(prob, sizes)
    tbij = _transpose_blocks(bij, sizes) if bij is not None else None
    gq, gk, gv = (np.zeros((N, H, D), np.float32) for _ in range(3))
    tga = np.zeros((E, H), np.float32)
    tgb = np.zeros((E, H, D), np.float32) if bij is not None else None
    L = ref_lib(K)
    L.cfref_fused_dpa_bwd(c_longlong(N), c_int(H), _p(q), _p(k), _p(v), _p(aij), _p(tbij), _p(batch), _p(edges),
                          _p(e_start), c_longlong(N), c_longlong(H), c_longlong(E), _p(tprob), _p(out), _p(go),
                          _p(gq), _p(gk), _p(gv), _p(tga), _p(tgb))
    ga = _transpose_blocks(tga, sizes)
    gb = _transpose_blocks(tgb, sizes) if tgb is not None else None
    L.cfref_fused_dpa_bwd_q(c_longlong(N), c_int(H), _p(k), _p(ga), _p(edges), _p(e_start), c_longlong(N),
                            c_longlong(H), c_longlong(E), _p(gq))
    return gq, gk, gv, ga, gb


def ref_irregular_mean(x, sizes, K=64):
    x, sizes = _f32(x), _i64(sizes)
    start = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    B, D = sizes.shape[0], x.shape[1]
    out = np.zeros((B, D), np.float32)
    bsz = min(32, D)
    ref_lib(K).cfref_irregular_mean_fwd(c_longlong((B * D + bsz - 1) // bsz), c_int(bsz), _p(x), _p(start),
                                        c_longlong(B), c_longlong(D), _p(out))
    return out


# ---- reciprocal-space lattice sum ---------------------------------------------------------------------------------
def reci_phase(pos_ij, rvecs, batch, edges):
    """kr_base (E,3) = rvecs[crystal of the edge] . pos_ij; see cf_oracle.c cfo_reci_phase."""
    pos_ij, rvecs, batch, edges = _f32(pos_ij), _f32(rvecs), _i64(batch), _i64(edges)
    E = edges.shape[1]
    kr = np.zeros((E, 3), np.float32)
    lib().cfo_reci_phase_f32(_p(pos_ij), _p(rvecs), _p(batch), _p(edges), c_longlong(E), _p(kr))
    return kr


def reci_sum_fwd(a, kr_base, rvecs, vcell, batch, edges, lattice_range=2, nested=False, precision="f32"):
    """phi (E,H) and the raw sum S (E,H); see cf_oracle.c cfo_reci_sum_fwd."""
    dt = _np_dtype(precision)
    a, kr_base, rvecs, vcell, batch, edges = _f32(a), _f32(kr_base), _f32(rvecs), _f32(vcell), _i64(batch), _i64(edges)
    N, H, E = a.shape[0], a.shape[1], edges.shape[1]
    z, s = np.zeros((E, H), dt), np.zeros((E, H), dt)
    getattr(lib(), f"cfo_reci_sum_fwd_{precision}")(
        _p(a), _p(kr_base), _p(rvecs), _p(vcell), _p(batch), _p(edges), c_longlong(N), c_longlong(H), c_longlong(E),
        c_int(lattice_range), c_int(int(nested)), _p(z), _p(s))
    return z, s


def reci_sum_bwd(a, kr_base, rvecs, batch, edges, gz, sumexp, lattice_range=2, nested=False, precision="f32"):
    """ga (N,H); see cf_oracle.c cfo_reci_sum_bwd."""
    dt = _np_dtype(precision)
    a, kr_base, rvecs, batch, edges = _f32(a), _f32(kr_base), _f32(rvecs), _i64(batch), _i64(edges)
    gz, sumexp = _real(gz, dt), _real(sumexp, dt)
    N, H, E = a.shape[0], a.shape[1], edges.shape[1]
    start = row_starts(edges, N)
    ga = np.zeros((N, H), dt)
    getattr(lib(), f"cfo_reci_sum_bwd_{precision}")(
        _p(a), _p(kr_base), _p(rvecs), _p(batch), _p(start), _p(gz), _p(sumexp), c_longlong(N), c_longlong(H),
        c_longlong(E), c_int(lattice_range), c_int(int(nested)), _p(ga))
    return ga


def ref_reci_enc_fwd(a, kr_base, rvecs, vcell, batch, edges, K=64):
    """The reference's reci_enc_fwd.cu compiled for the CPU (LATTICE_RANGE = 2)."""
    a, kr_base, rvecs, vcell, batch, edges = _f32(a), _f32(kr_base), _f32(rvecs), _f32(vcell), _i64(batch), _i64(edges)
    N, H, E = a.shape[0], a.shape[1], edges.shape[1]
    z, s = np.zeros((E, H), np.float32), np.zeros((E, H), np.float32)
    ref_lib(K).cfref_reci_enc_fwd(c_longlong(E), c_int(H), _p(a), _p(kr_base), _p(rvecs), _p(vcell), _p(batch),
                                  _p(edges), c_longlong(N), c_longlong(H), c_longlong(E), _p(z), _p(s))
    return z, s


def ref_reci_enc_bwd(a, kr_base, rvecs, vcell, batch, edges, z, gz, sumexp, K=64):
    """The reference's reci_enc_bwd.cu compiled for the CPU (LATTICE_RANGE = 2)."""
    a, kr_base, rvecs, vcell, batch, edges = _f32(a), _f32(kr_base), _f32(rvecs), _f32(vcell), _i64(batch), _i64(edges)
    z, gz, sumexp = _f32(z), _f32(gz), _f32(sumexp)
    N, H, E = a.shape[0], a.shape[1], edges.shape[1]
    start = row_starts(edges, N)
    ga = np.zeros((N, H), np.float32)
    ref_lib(K).cfref_reci_enc_bwd(c_longlong(N), c_int(H), _p(a), _p(kr_base), _p(rvecs), _p(vcell), _p(batch),
                                  _p(edges), _p(start), _p(z), _p(gz), _p(sumexp), c_longlong(N), c_longlong(H),
                                  c_longlong(E), _p(ga))
    return ga
