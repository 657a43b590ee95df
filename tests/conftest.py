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


@pytest.fixture(scope="module", autouse=True)
def no_device_side_give_up(request):
    """After every GPU test module: no kernel of the library may have reported a give-up (a bounded wait that ran out,
    or a failed index check in a bounds-checked build). Modules that provoke one on purpose clear the word themselves."""
    yield
    module = request.module
    marks = getattr(module, "pytestmark", None)
    marks = marks if isinstance(marks, (list, tuple)) else [marks]
    if not any(getattr(m, "name", None) == "gpu" for m in marks if m is not None):
        return
    import torch
    if not torch.cuda.is_available():
        return
    from gmc import _native
    assert _native.device_check_word() == 0, f"a kernel reported a device-side give-up during {module.__name__}"
