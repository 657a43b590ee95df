"""GPU: the library compiled with device-side index checks (-DGMC_BOUNDS_CHECK, libgmc_b200_checked.so) runs the small
exhaustive cases of the fits without a single report, and its check does fire on an index that is out of range.

Stands in for a memory checker on the kernels whose indices come from data (tree children, object ids, sorted product
indices): a bad index sets bit 4 of the device check word and is replaced by 0, so nothing is read out of bounds. The
checked library is a second build of the same sources; a child process loads it through GMC_B200_LIB."""
import os
import subprocess
import sys

import pytest
import torch

from conftest import PKG, ROOT

pytestmark = pytest.mark.gpu

CHECKED = os.path.join(PKG, "gmc", "_lib", "libgmc_b200_checked.so")

CHILD = r'''
import sys
sys.path.insert(0, {root!r}); sys.path.insert(0, {pkg!r})
import numpy as np, torch
import synthetic_inputs as synthetic
from gmc import _native, lbvh
import gmc.cpp.extensions.bvh_mhem_fit.binding as fit
import gmc.cpp.extensions.convolution_fitting.binding as cf
assert _native._LIB_PATH.endswith("libgmc_b200_checked.so")
# the check itself: in range -> silent, out of range -> bit 4 and element 0
one, out = torch.full((1,), 3.5, device="cuda"), torch.zeros(1, device="cuda")
s = _native.stream_of(one)
assert _native.lib.gmc_debug_index_check(_native.ptr(one), _native.ptr(out), 0, 1, s) == 0
assert _native.device_check_word() == 0 and out.item() == 3.5
out.zero_()
assert _native.lib.gmc_debug_index_check(_native.ptr(one), _native.ptr(out), 70000, 1, s) == 0
assert _native.device_check_word() == 4 and out.item() == 3.5
assert _native.device_check_word() == 0
# the fits on small cases of every shape class: odd sizes, two Gaussians, duplicates, 2D and 3D, forward and backward
for D in (2, 3):
    for G, K, R in ((2, 4, 4), (3, 2, 2), (37, 8, 4), (64, 16, 2), (333, 32, 4)):
        g = torch.Generator().manual_seed(G)
        cov, _ = synthetic.covariances_and_inverses((2, 3, G), D, 0.03, 0.3, g)
        m = synthetic.pack(torch.rand(2, 3, G, generator=g) + 0.05, torch.rand(2, 3, G, D, generator=g) * 2 - 1, cov)
        if G > 5:
            m[0, 0, 3:5, 1:1 + D] = m[0, 0, 2:3, 1:1 + D]
        mt = m.cuda().requires_grad_(True)
        lbvh.build(mt.detach())
        out = fit.apply(mt, K, R)
        out.sum().backward()
        assert torch.isfinite(out).all() and torch.isfinite(mt.grad).all()
    for (B, Cin, Gd, Cout, Gk, K) in ((2, 3, 16, 4, 5, 16), (1, 1, 2, 1, 1, 4), (2, 2, 7, 2, 3, 42), (1, 8, 64, 2, 5, 32)):
        g = torch.Generator().manual_seed(Gd + K)
        cd, _ = synthetic.covariances_and_inverses((B, Cin, Gd), D, 0.03, 0.15, g)
        data = synthetic.pack(torch.randn(B, Cin, Gd, generator=g), torch.rand(B, Cin, Gd, D, generator=g) * 2 - 1, cd)
        ck, _ = synthetic.covariances_and_inverses((Cout, Cin, Gk), D, 0.02, 0.1, g)
        kern = synthetic.pack(torch.randn(Cout, Cin, Gk, generator=g) * 0.1, torch.randn(Cout, Cin, Gk, D, generator=g) * 0.1, ck)
        d, k = data.cuda().requires_grad_(True), kern.cuda().requires_grad_(True)
        out = cf.apply(d, k, K)
        out.sum().backward()
        assert torch.isfinite(out).all() and torch.isfinite(d.grad).all() and torch.isfinite(k.grad).all()
word = _native.device_check_word()
assert word == 0, f"an index check failed: word {{word}}"
print("checked build ok")
'''


def test_checked_build_reports_nothing_on_the_small_cases_and_its_check_fires():
    assert os.path.exists(CHECKED), "libgmc_b200_checked.so is not built (python build.py --checked)"
    env = dict(os.environ, GMC_B200_LIB=CHECKED)
    res = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT, pkg=PKG)], env=env, capture_output=True, text=True,
                         timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "checked build ok" in res.stdout


def test_regular_build_has_no_index_checks():
    from gmc import _native
    one = torch.zeros(1, device="cuda")
    assert _native.lib.gmc_debug_index_check(_native.ptr(one), _native.ptr(one), 0, 1, _native.stream_of(one)) == 4
