import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "gaussian-mixture-convolution-networks_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 machine)")


def rel_inf(a, ref):
    """Parity metric for floating-point tensors: ||a - ref||_inf / max(||ref||_inf, 1e-30)."""
    import numpy as np
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.fixture(scope="session")
def golden_eval():
    import numpy as np
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "eval_inversed.npz")))
