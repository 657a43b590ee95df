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


def load(native: bool = False):
    """Returns the reference's (gmc.mixture, gmc.fitting, gmc.mat_tools) modules, CPU only.

    native=True routes the reference's extension bindings to the reference's own native CPU code
    (oracle/_ref/libgmc_ref.so through oracle/ref_native.py; forward only, no autograd) and also makes
    gmc.modules / gmc.model importable (stand-ins for matplotlib, tensorboard and the OpenGL visualiser):
    use load_network() for those."""
    if not available():
        raise RuntimeError(f"reference sources not found under {REFERENCE_SRC}")
    if "gmc" in sys.modules and not getattr(sys.modules["gmc"], "__file__", "").startswith(REFERENCE_SRC):
        raise RuntimeError("another 'gmc' package is already imported in this process; "
                           "run the reference oracle in a process of its own")

    if REFERENCE_SRC not in sys.path:
        sys.path.insert(0, REFERENCE_SRC)

    def stub(name, **attrs):
        import importlib
        m = types.ModuleType(name)
        parent, _, leaf = name.rpartition(".")
        if parent.startswith("gmc"):
            # `import a.b.c as x` reads c as an attribute of a.b: import the (real) parent package and hang the stub on it
            try:
                setattr(importlib.import_module(parent), leaf, m)
            except ImportError:
                pass
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
    if native:
        from . import ref_native

        def fit_apply(mixture, n_components, reduction_n):
            shape = mixture.shape
            out = ref_native.mhem_fit_forward(mixture.detach().numpy(), int(n_components), int(reduction_n))
            return torch.from_numpy(out).view(shape[0], shape[1], int(n_components), shape[3])

        def convfit_apply(data, kernels, n_components):
            with ref_native.serial():      # the reference's mass pass is racy when its CPU threads run concurrently
                return torch.from_numpy(ref_native.convolution_fitting_forward(data.detach().numpy(), kernels.detach().numpy(),
                                                                               int(n_components))[0])

        sys.modules["gmc.cpp.extensions.bvh_mhem_fit.binding"].apply = fit_apply
        stub("gmc.cpp.extensions.convolution_fitting.binding", apply=convfit_apply)
        stub("gmc.cpp.extensions.convolution.binding", apply=_Unavailable.apply)
        stub("gmc.cpp.gm_vis")
        stub("gmc.cpp.gm_vis.gm_vis")
        stub("gmc.render")          # matplotlib / Qt debug pictures: not on the path
        stub("gmc.colourmap")
        for name in ("matplotlib", "matplotlib.cm", "matplotlib.pyplot", "matplotlib.colors", "matplotlib.image",
                     "pyrender"):
            if name not in sys.modules:
                stub(name)
        try:
            import importlib
            importlib.import_module("torch.utils.tensorboard")
        except Exception:
            stub("torch.utils.tensorboard", SummaryWriter=object)
    if REFERENCE_SRC not in sys.path:
        sys.path.insert(0, REFERENCE_SRC)
    import gmc.mixture as gm
    import gmc.mat_tools as mat_tools
    sys.modules["gmc.cpp.extensions.evaluate_inversed.evaluate_inversed"].apply = gm.old_evaluate_inversed
    gm.evaluate_inversed = gm.old_evaluate_inversed
    if native:
        from . import ref_native as _rn

        def native_eval(mixture, xes):
            return torch.from_numpy(_rn.eval_forward(mixture.detach().contiguous().numpy(), xes.detach().contiguous().numpy()))

        sys.modules["gmc.cpp.extensions.evaluate_inversed.evaluate_inversed"].apply = native_eval
        gm.evaluate_inversed = native_eval
    import gmc.fitting as fitting
    return gm, fitting, mat_tools


def load_network():
    """Returns the reference's (gmc.mixture, gmc.modules, gmc.model) with every extension routed to the reference's own
    native CPU code: the reference's network forward pass, runnable on CPU."""
    gm, fitting, mat_tools = load(native=True)
    import gmc.modules as modules
    import gmc.model as model
    return gm, modules, model
