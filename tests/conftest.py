import os
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if REPO not in sys.path:
    sys.path.insert(0, REPO)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_ops():
    import numpy as np
    return dict(np.load(os.path.join(REPO, "tests", "golden", "golden_ops.npz")))


@pytest.fixture(scope="session")
def golden_model():
    import numpy as np
    return dict(np.load(os.path.join(REPO, "tests", "golden", "golden_model.npz")))


def rel_err(x, ref):
    """max |x - ref| / max |ref|: the per-tensor measure every fp32 parity bound in this suite uses."""
    import numpy as np
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.abs(ref).max() if ref.size else 1.0
    return float(np.abs(x - ref).max() / (den if den > 0 else 1.0)) if ref.size else 0.0
