"""The reference project's own host code accepts this package as its ``models.cuda_funcs`` (the swap: the package is
put into ``sys.modules`` under that name before the reference's modules are imported).  Runs only where the reference tree is mounted; no GPU and no kernel launch are involved: the test
checks that the reference's modules import against the shim, pick their CUDA encoder, build with our kernels
"compiled", and that the state_dict keys of the reference model and of the mirror in this package coincide."""
import contextlib
import importlib
import io
import json
import os
import sys
import types

import pytest

REF = os.environ.get("CF_REFERENCE_ROOT", "/root/reference")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "models")), reason="reference tree not mounted")


@pytest.fixture()
def reference_with_shim():
    import crystalformer_b200.cuda_funcs as shim
    saved = {k: v for k, v in sys.modules.items() if k == "models" or k.startswith("models.")}
    for k in saved:
        del sys.modules[k]
    sys.dont_write_bytecode = True
    sys.path.insert(0, REF)
    sys.modules["models.cuda_funcs"] = shim
    try:
        yield shim
    finally:
        sys.path.remove(REF)
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            del sys.modules[k]
        sys.modules.update(saved)


def test_reference_host_code_runs_on_the_shim(reference_with_shim):
    shim = reference_with_shim
    config = importlib.import_module("models.global_config")
    config.REPRODUCIBLITY_STATE = 3
    attn = importlib.import_module("models.indexed_lattice_multi_head_attention_cuda")
    # the names the reference's attention module star-imports now come from this package
    assert attn.RealPeriodicEncodingWithProjFuncCUDA is shim.RealPeriodicEncodingWithProjFuncCUDA
    assert attn.FusedDotProductAttentionCUDA is shim.FusedDotProductAttentionCUDA
    assert attn.CUPY_AVAILABLE is True
    pooling = importlib.import_module("models.pooling")
    assert pooling.cuda_funcs is shim
    lat = importlib.import_module("models.latticeformer")
    P = json.load(open(os.path.join(REF, "params/latticeformer/default.json")))
    with contextlib.redirect_stdout(io.StringIO()):
        model = lat.Latticeformer(types.SimpleNamespace(**P))
    enc = importlib.import_module("models.indexed_latticeformer_encoder")
    assert isinstance(model.encoder, enc.CrystalformerEncoderCUDA)          # the CUDA path was chosen
    assert shim.KernelManager.compiled and shim.KernelManager.LATTICE_RANGE == 2 and shim.KernelManager.MINIMUM_RANGE == 2
    from crystalformer_b200.model import Latticeformer, default_params
    mine = Latticeformer(default_params())
    assert sorted(mine.state_dict().keys()) == sorted(model.state_dict().keys())
    for k, v in model.state_dict().items():
        assert tuple(mine.state_dict()[k].shape) == tuple(v.shape), k
