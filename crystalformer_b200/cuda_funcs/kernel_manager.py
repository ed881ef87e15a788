"""Kernel registry with the reference's interface (models/cuda_funcs/kernel_manager.py:15-134).

The reference reads every ``.cu`` file at import, substitutes constants into the text and JIT-compiles with NVRTC when
``compile_kernels`` is called.  Here the kernels are pre-compiled for sm_100a; ``compile_kernels`` records the same
constants (they are run-time arguments of the C ABI), checks that the shapes are among the compiled ones and makes
sure the library is loaded.
"""
from __future__ import annotations

import math
from typing import List

from .. import _lib


class Kernel:
    """Handle of one entry point of the library (the reference's object wraps a ``cupy.RawKernel``)."""

    def __init__(self, name: str, entry: str = None):
        self.name: str = name
        self.entry: str = entry  # C-ABI symbol that took over this kernel's work
        self.code: str = None
        self.raw_kernel = None

    def __call__(self, grid, block, args, **kwargs):
        raise RuntimeError(
            f"{self.name}: kernels are launched through the C ABI ({self.entry}); grid/block launches are not supported")


class KernelManager:
    real_enc_fwd: Kernel = None
    real_enc_bwd: Kernel = None
    real_enc_fwd_v2: Kernel = None
    real_enc_bwd_v2: Kernel = None
    real_enc_proj_fwd: Kernel = None
    real_enc_proj_bwd: Kernel = None
    real_enc_proj_fwd_v2: Kernel = None
    real_enc_proj_bwd_v2: Kernel = None
    fused_dpa_fwd: Kernel = None
    fused_dpa_fwd_v3: Kernel = None
    fused_dpa_bwd: Kernel = None
    fused_dpa_bwd_v3: Kernel = None
    fused_dpa_bwd_q: Kernel = None
    fused_dpa_bwd_q_v3: Kernel = None
    irregular_transpose: Kernel = None
    irregular_mean_fwd: Kernel = None

    # limits the reference exposes (kernel_manager.py:55-57); the attention kernels here have no 320-atom limit, the
    # value is kept for callers that read it
    MAX_SYSTEM_SIZE: int = 320
    MAX_SYSTEM_SIZE_POW2: int = int(2 ** math.ceil(math.log2(MAX_SYSTEM_SIZE)))
    RUNNING_SUM_LEN: int = 8

    # constants recorded by compile_kernels (text substitutions in the reference, kernel_manager.py:110-121)
    LATTICE_RANGE: int = 2
    MINIMUM_RANGE: int = 2
    HEAD_NUM: int = 8
    K_HEAD_DIM: int = 16
    V_HEAD_DIM: int = 16
    VPE_DIM: int = 64
    compiled: bool = False

    @staticmethod
    def get_kernel_names() -> List[str]:
        return [name for name, kind in KernelManager.__annotations__.items() if kind in (Kernel, "Kernel")]

    @staticmethod
    def get_kernel(name: str) -> Kernel:
        return getattr(KernelManager, name)

    @staticmethod
    def set_kernel(name: str, kernel: Kernel):
        setattr(KernelManager, name, kernel)


_ENTRY = {
    "real_enc_fwd": "cf_lattice_sum_fwd", "real_enc_fwd_v2": "cf_lattice_sum_fwd",
    "real_enc_proj_fwd": "cf_lattice_sum_fwd", "real_enc_proj_fwd_v2": "cf_lattice_sum_fwd",
    "real_enc_bwd": "cf_lattice_sum_bwd", "real_enc_bwd_v2": "cf_lattice_sum_bwd",
    "real_enc_proj_bwd": "cf_lattice_sum_bwd", "real_enc_proj_bwd_v2": "cf_lattice_sum_bwd",
    "fused_dpa_fwd": "cf_fused_attn_fwd", "fused_dpa_fwd_v3": "cf_fused_attn_fwd",
    "fused_dpa_bwd": "cf_fused_attn_bwd", "fused_dpa_bwd_v3": "cf_fused_attn_bwd",
    "fused_dpa_bwd_q": "cf_fused_attn_bwd", "fused_dpa_bwd_q_v3": "cf_fused_attn_bwd",
    "irregular_transpose": "cf_fused_attn_bwd", "irregular_mean_fwd": "cf_segment_mean_fwd",
}
for _name in KernelManager.get_kernel_names():
    KernelManager.set_kernel(_name, Kernel(_name, _ENTRY[_name]))


def compile_kernels(lattice_range: int, head_num: int, key_head_dim: int, value_pe_dim: int, value_head_dim: int,
                    set_minimum_range: bool):
    """Same signature as the reference (kernel_manager.py:109).  Nothing is compiled at run time; the call validates
    the configuration against the pre-compiled kernels and records the translation-box constants."""
    if head_num != 8 or key_head_dim != 16 or value_head_dim != 16 or value_pe_dim not in (0, 64):
        raise NotImplementedError(
            "crystalformer_b200 is compiled for head_num=8, head dims 16 and value_pe_dist_real in {0, 64}; got "
            f"head_num={head_num}, key_head_dim={key_head_dim}, value_head_dim={value_head_dim}, value_pe_dim={value_pe_dim}")
    if not 0 <= lattice_range <= 32:
        raise ValueError(f"lattice_range {lattice_range} outside [0, 32]")
    lib = _lib.load()
    KernelManager.LATTICE_RANGE = int(lattice_range)
    KernelManager.MINIMUM_RANGE = int(lattice_range) if set_minimum_range else 0
    KernelManager.HEAD_NUM = head_num
    KernelManager.K_HEAD_DIM = key_head_dim
    KernelManager.V_HEAD_DIM = value_head_dim
    KernelManager.VPE_DIM = value_pe_dim
    KernelManager.compiled = True
    for name in KernelManager.get_kernel_names():
        KernelManager.get_kernel(name).raw_kernel = getattr(lib, _ENTRY[name])
