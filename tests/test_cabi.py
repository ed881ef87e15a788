"""The C-ABI shared library loads, exports every symbol the public header declares, and validates its arguments
before touching the device.  No GPU needed: only calls that fail validation are made."""
import ctypes
import os
import re

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from crystalformer_b200 import build
    build.build()
    from crystalformer_b200 import _lib
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(REPO, "include", "crystalformer_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cf_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_table_covers_the_header():
    from crystalformer_b200 import _lib
    bound = set(_lib.SIGNATURES) | {"cf_version", "cf_last_error", "cf_set_weight_floor_log2",
                                    "cf_get_weight_floor_log2", "cf_encoder_workspace_floats",
                                    "cf_model_workspace_bytes", "cf_term_list_workspace_bytes",
                                    "cf_row_list_workspace_bytes", "cf_set_sorted_rows", "cf_get_sorted_rows",
                                    "cf_set_row_stats", "cf_set_chained_launches"}
    assert set(declared_symbols()) <= bound


def test_version_and_knob(lib):
    assert lib.cf_version() >= 100
    lib.cf_set_weight_floor_log2(ctypes.c_double(-33.0))
    assert lib.cf_get_weight_floor_log2() == -33.0
    lib.cf_set_weight_floor_log2(ctypes.c_double(-30.0))


def test_validation_returns_codes_without_a_device(lib):
    from crystalformer_b200 import _lib
    null = ctypes.c_void_p(0)
    with pytest.raises(_lib.CrystalformerB200Error) as e:
        _lib.call("cf_lattice_sum_fwd", null, 0, null, null, null, null, 4, 4, 4, 64, 14.0, 1.0, null, 0, 0, null, 0.0,
                  2, 2, null, null, null)
    assert e.value.code == -2
    with pytest.raises(_lib.CrystalformerB200Error) as e:
        _lib.call("cf_lattice_sum_fwd", null, 0, null, null, null, null, 4, 8, 4, 32, 14.0, 1.0, null, 0, 0, null, 0.0,
                  2, 2, null, null, null)
    assert e.value.code == -2 and "K=32" in str(e.value)
    with pytest.raises(_lib.CrystalformerB200Error) as e:
        _lib.call("cf_lattice_sum_fwd", null, 0, null, null, null, null, 4, 8, 4, 64, 14.0, 1.0, null, 0, 0, null, 0.0,
                  2, 2, null, null, null)
    assert e.value.code == -1  # null pointers
    with pytest.raises(_lib.CrystalformerB200Error) as e:
        _lib.call("cf_lattice_sum_fwd", null, 0, null, null, null, null, 4, 8, 4, 64, 14.0, 1.0, null, 0, 0, null, 0.0,
                  99, 2, null, null, null)
    assert e.value.code == -4
    with pytest.raises(_lib.CrystalformerB200Error) as e:
        _lib.call("cf_fused_attn_fwd", null, null, null, null, null, null, null, 4, 8, 32, 4, null, null, null)
    assert e.value.code == -2
    with pytest.raises(_lib.CrystalformerB200Error) as e:
        _lib.call("cf_pipe_probe", 5, 1, 32, 1, null, null)
    assert e.value.code == -1


def test_package_refuses_cpu_tensors():
    import torch
    from crystalformer_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.segment_mean(torch.zeros((4, 8)), torch.tensor([0, 4]))


def test_peer_gather_descriptor_matches_the_header_layout():
    """cf_peer_gather of the header: two int32, one int64, two uint32, CF_MAX_PEERS pointers, naturally aligned."""
    from crystalformer_b200 import _lib
    header = open(os.path.join(REPO, "include", "crystalformer_b200.h")).read()
    peers = int(re.search(r"#define CF_MAX_PEERS (\d+)", header).group(1))
    handle = int(re.search(r"#define CF_PEER_HANDLE_BYTES (\d+)", header).group(1))
    assert peers == _lib.MAX_PEERS and handle == _lib.PEER_HANDLE_BYTES
    D = _lib.PeerGatherDescriptor
    assert ctypes.sizeof(D) == 24 + 8 * peers
    assert (D.world.offset, D.rank.offset, D.rows_per_rank.offset, D.step.offset, D.cells.offset) == (0, 4, 8, 16, 24)
