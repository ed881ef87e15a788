"""ctypes binding of ``libcrystalformer_b200.so`` (the C ABI declared in include/crystalformer_b200.h).

There is no CPU or PyTorch fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_double, c_int, c_int64, c_void_p
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcrystalformer_b200.so")
_lib: Optional[ctypes.CDLL] = None

P, I64, I32, F64 = c_void_p, c_int64, c_int, c_double

# name -> argument types, in the order of include/crystalformer_b200.h
SIGNATURES = {
    "cf_crystal_offsets": [P, I64, P, P, P],
    "cf_batch_prepare": [P, P, P, P, P, I64, I64, I64, P, P, P, P, P, P, P, P],
    "cf_lattice_box": [P, I32, P, P, I64, I64, I64, P, F64, I32, I32, P, P],
    "cf_lattice_sum_fwd": [P, I32, P, P, P, P, I64, I64, I64, I64, F64, F64, P, I64, I64, P, F64, I32, I32, P, P, P],
    "cf_lattice_sum_bwd": [P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, F64, F64, P, F64, I32, I32, P, P, P, P],
    "cf_lattice_sum_bwd_static": [P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, F64, F64, P, F64, I32, I32, P, P, P],
    "cf_fused_attn_fwd": [P, P, P, P, P, P, P, I64, I64, I64, I64, P, P, P],
    "cf_fused_attn_bwd": [P, P, P, P, P, P, I64, I64, I64, I64, P, P, P, P, P, P, P, P, P],
    "cf_segment_mean_fwd": [P, P, I64, I64, P, P],
    "cf_infinite_attn_fwd": [P, P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, I64, F64, F64, P, F64, I32,
                             I32, P, P, P, P, P, P],
    "cf_infinite_attn_bwd": [P, P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, I64, F64, F64, P, F64, I32,
                             I32, P, P, P, P, P, P, P, P, P, P, P],
    "cf_pipe_probe": [I32, I32, I32, I64, P, P],
    "cf_model_forward": [P, P, I64, P, P, P, I64, I64, I64, I64, P, P, I32, P, P, I64, I64, F64, F64, I32, I32, P, P, I64, P,
                         P, I64, F64, P, P, P, P, P, P, P],
    "cf_peer_alloc": [I64, P, P],
    "cf_peer_open": [P, P],
    "cf_peer_close": [P],
    "cf_peer_free": [P],
    "cf_peer_gather_store": [P, I64, I64, P, P],
    "cf_peer_gather_collect": [P, ctypes.c_uint32, P, I64, I64, I64, P, P, F64, P],
    "cf_term_list_build": [P, P, P, P, P, P, P, I64, I64, I64, F64, I32, I32, F64, P, P],
    "cf_infinite_attn_fwd_listed": [P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, I64, F64, F64, P, F64, I32,
                                    I32, P, P, P, P, P, P, F64, P],
    "cf_infinite_attn_bwd_listed": [P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, I64, F64, F64, P, F64, I32,
                                    I32, P, P, P, P, P, P, P, P, P, P, P, F64, P],
    "cf_row_list_build": [P, P, P, P, P, P, P, I64, I64, I64, F64, I32, I32, F64, P, P],
    "cf_infinite_attn_fwd_sorted": [P, P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, I64, F64, F64, P, F64, I32,
                                    I32, P, P, P, P],
    "cf_serve_submit": [P, P, P, P, P, P, I64, I64, I64, I64, I32, P, P],
    "cf_row_cost": [P, P, I64, I64, F64, P, P],
    "cf_row_order": [P, P, I64, I64, F64, P, P],
    "cf_reci_phase": [P, P, P, P, I64, P, P],
    "cf_reci_sum_fwd": [P, P, P, P, P, P, I64, I64, I64, I32, P, P, P],
    "cf_reci_sum_bwd": [P, P, P, P, P, P, P, I64, I64, I64, I32, P, P],
    "cf_encoder_forward": [P, I32, P, P, P, P, P, P, P, P, P, I64, I64, I64, I64, I64, I64, F64, F64, I32, I32, P, P, P,
                           P],
}


MAX_PEERS = 16
PEER_HANDLE_BYTES = 64


class PeerGatherDescriptor(ctypes.Structure):
    """``cf_peer_gather`` of include/crystalformer_b200.h: one step of a peer gather as seen by one rank."""
    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("rows_per_rank", c_int64),
                ("step", ctypes.c_uint32), ("reserved", ctypes.c_uint32), ("cells", c_void_p * MAX_PEERS)]


class ModelDesc(ctypes.Structure):
    """``cf_model_desc`` of include/crystalformer_b200.h: the batch-independent arguments of cf_model_forward."""
    _fields_ = [("feature_dim", c_int64), ("W_embed", c_void_p), ("W_embed_packed", c_void_p),
                ("num_layers", ctypes.c_int32), ("lattice_range", ctypes.c_int32), ("minimum_range", ctypes.c_int32),
                ("dense_tile_rows", ctypes.c_int32), ("weights", c_void_p), ("scalars", c_void_p), ("K", c_int64),
                ("ff_dim", c_int64), ("wscale", c_double), ("cutoff_radius", c_double), ("W1", c_void_p), ("b1", c_void_p),
                ("hidden", c_int64), ("W2", c_void_p), ("b2", c_void_p), ("targets", c_int64), ("order_reach", c_double)]


class ServeSlot(ctypes.Structure):
    """``cf_serve_slot``: the streams, events and buffers of one batch in flight."""
    _fields_ = [("copy_stream", c_void_p), ("compute_stream", c_void_p), ("copied", c_void_p), ("inputs_free", c_void_p),
                ("done", c_void_p), ("x", c_void_p), ("pos", c_void_p), ("trans", c_void_p), ("sizes", c_void_p),
                ("workspace", c_void_p), ("y", c_void_p), ("y_host", c_void_p), ("max_atoms_total", c_int64),
                ("max_crystals", c_int64), ("max_edges", c_int64), ("species", c_void_p)]


class ServeGather(ctypes.Structure):
    """``cf_serve_gather``: the peer gather of one step of ``cf_serve_submit``."""
    _fields_ = [("store", c_void_p), ("collect_stream", c_void_p), ("store_after", c_void_p), ("stored", c_void_p),
                ("collected", c_void_p), ("own_cells", c_void_p), ("index", c_void_p), ("total_rows", c_int64),
                ("y_all", c_void_p), ("y_all_host", c_void_p), ("status", c_void_p), ("status_host", c_void_p),
                ("timeout_s", c_double)]


class CrystalformerB200Error(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, name: str, code: int, message: str):
        super().__init__(f"{name} failed with code {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    """Loads the shared library once; raises if it has not been built (python -m crystalformer_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m crystalformer_b200.build`; "
                "crystalformer_b200 has no CPU fallback")
        lib = ctypes.CDLL(LIB_PATH)
        lib.cf_version.restype = c_int
        lib.cf_last_error.restype = c_char_p
        lib.cf_set_weight_floor_log2.argtypes = [c_double]
        lib.cf_set_weight_floor_log2.restype = None
        lib.cf_get_weight_floor_log2.restype = c_double
        lib.cf_encoder_workspace_floats.argtypes = [I64, I64, I64]
        lib.cf_encoder_workspace_floats.restype = c_int64
        lib.cf_term_list_workspace_bytes.argtypes = [I64, I64]
        lib.cf_term_list_workspace_bytes.restype = c_int64
        lib.cf_row_list_workspace_bytes.argtypes = [I64, I64]
        lib.cf_row_list_workspace_bytes.restype = c_int64
        lib.cf_set_sorted_rows.argtypes = [c_int]
        lib.cf_set_sorted_rows.restype = None
        lib.cf_get_sorted_rows.restype = c_int
        lib.cf_set_chained_launches.argtypes = [c_int]
        lib.cf_set_chained_launches.restype = None
        lib.cf_set_row_stats.argtypes = [c_void_p]
        lib.cf_set_row_stats.restype = None
        lib.cf_model_workspace_bytes.argtypes = [I64, I64, I64, I64]
        lib.cf_model_workspace_bytes.restype = c_int64
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        _lib = lib
    return _lib


def call(name: str, *args) -> None:
    """Calls one entry point and raises CrystalformerB200Error on a negative status."""
    lib = load()
    code = getattr(lib, name)(*args)
    if code != 0:
        raise CrystalformerB200Error(name, code, lib.cf_last_error().decode())
