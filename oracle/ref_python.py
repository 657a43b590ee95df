"""TEST INFRASTRUCTURE. Imports the reference's own Python (gmc.mixture, gmc.fitting, ...) on CPU.

Only usable where the reference checkout is present (environment variable GMC_REFERENCE_SRC, default: the directory
`reference/src` next to this repository): the golden
fixture generator under tests/golden/ uses it; nothing that runs on the GPU machine does. The reference's
Python builds its CUDA extensions at import time; those wrapper modules are replaced by stand-ins that
route to the reference's pure-PyTorch twins (gm.old_evaluate_inversed, torch.linalg.inv, torch.linalg.eigh)
before anything of the reference is imported.
"""
import os
import sys
import types

import torch

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE_SRC = os.environ.get("GMC_REFERENCE_SRC", os.path.join(os.path.dirname(_REPO), "reference", "src"))


def available() -> bool:
    return os.path.isdir(os.path.join(REFERENCE_SRC, "gmc"))


def load():
    """Returns the reference's (gmc.mixture, gmc.fitting, gmc.mat_tools) modules, CPU only."""
    if not available():
        raise RuntimeError(f"reference sources not found under {REFERENCE_SRC}")
    if "gmc" in sys.modules and not getattr(sys.modules["gmc"], "__file__", "").startswith(REFERENCE_SRC):
        raise RuntimeError("another 'gmc' package is already imported in this process; "
                           "run the reference oracle in a process of its own")

    def stub(name, **attrs):
        m = types.ModuleType(name)
        for k, v in attrs.items():
            setattr(m, k, v)
        sys.modules[name] = m
        return m

    class _Unavailable:
        @staticmethod
        def apply(*a, **k):
            raise RuntimeError("native extension of the reference is not built in this environment")

    stub("gmc.cpp.extensions.evaluate_inversed.evaluate_inversed", apply=None)
    stub("gmc.cpp.extensions.math.matrix_inverse", apply=torch.linalg.inv)
    stub("gmc.cpp.extensions.pieces.bindings", symeig_apply=torch.linalg.eigh,
         matrix_inverse_apply=torch.linalg.inv)
    stub("gmc.cpp.extensions.bvh_mhem_fit.binding", apply=_Unavailable.apply)
    if REFERENCE_SRC not in sys.path:
        sys.path.insert(0, REFERENCE_SRC)
    import gmc.mixture as gm
    import gmc.mat_tools as mat_tools
    sys.modules["gmc.cpp.extensions.evaluate_inversed.evaluate_inversed"].apply = gm.old_evaluate_inversed
    gm.evaluate_inversed = gm.old_evaluate_inversed
    import gmc.fitting as fitting
    return gm, fitting, mat_tools
