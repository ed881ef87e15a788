"""Drop-in replacement of the reference's ``models/cuda_funcs`` package (models/cuda_funcs/__init__.py:19-29).

The names, call signatures, return conventions and error behaviour are the reference's, so its own host code
(``models/indexed_lattice_multi_head_attention_cuda.py``, ``models/pooling.py``, ``models/indexed_latticeformer_encoder.py``)
runs unchanged when this package is installed as ``models.cuda_funcs`` (``sys.modules['models.cuda_funcs'] = crystalformer_b200.cuda_funcs``
before the reference's modules are imported, with ``models.global_config.REPRODUCIBLITY_STATE = 3``).  Behind the names the
reference's CuPy ``RawKernel`` launches are replaced by calls into ``libcrystalformer_b200.so``.

``CUPY_AVAILABLE`` keeps its name because the reference reads it (models/latticeformer.py:139-143) to choose its CUDA
encoder; here it means "the sm_100a kernel library is loaded".  Importing this package without the built library raises.
"""
from .. import _lib as _lib

_lib.load()  # fail loudly at import time: there is no fallback implementation

CUPY_AVAILABLE = True

from .kernel_manager import Kernel, KernelManager, compile_kernels  # noqa: E402
from .real_space_enc import RealPeriodicEncodingFuncCUDA  # noqa: E402
from .real_space_enc_proj import RealPeriodicEncodingWithProjFuncCUDA  # noqa: E402
from .reci_space_enc import ReciPeriodicEncodingFuncCUDA  # noqa: E402
from .fused_dpa import FusedDotProductAttentionCUDA  # noqa: E402
from .irregular_mean import IrregularMeanCUDA  # noqa: E402

__all__ = [
    "KernelManager",
    "Kernel",
    "compile_kernels",
    "FusedDotProductAttentionCUDA",
    "RealPeriodicEncodingFuncCUDA",
    "RealPeriodicEncodingWithProjFuncCUDA",
    "ReciPeriodicEncodingFuncCUDA",
    "IrregularMeanCUDA",
    "CUPY_AVAILABLE",
]
