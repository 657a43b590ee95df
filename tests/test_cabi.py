"""CPU: the C-ABI library loads and exports every function that include/gmc_b200.h declares; host-side
argument checks answer with status codes (no GPU work is issued)."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "gmc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gmc_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    from gmc import _native
    names = _declared_functions()
    assert "gmc_eval_inversed_forward" in names and "gmc_eval_inversed_backward" in names
    for n in names:
        assert hasattr(_native.lib, n), f"{n} declared in gmc_b200.h but not exported"


def test_status_strings():
    from gmc import _native
    assert _native.lib.gmc_status_string(0) == b"ok"
    for s in range(1, 9):
        assert len(_native.lib.gmc_status_string(s)) > 0
    assert _native.lib.gmc_version().decode().count(".") == 1


def test_argument_checks_return_status_without_gpu():
    from gmc import _native
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)  # never dereferenced: argument checks come first
    f = _native.lib.gmc_eval_inversed_forward
    assert f(one, one, one, 1, 1, 1, 4, 1, 1, 1, null) == 1   # D = 4
    assert f(one, one, one, 2, 1, 1, 2, 3, 1, 1, null) == 2   # batch broadcast mismatch
    assert f(null, one, one, 1, 1, 1, 2, 1, 1, 1, null) == 3  # NULL mixture
    b = _native.lib.gmc_eval_inversed_backward
    assert b(one, one, one, one, one, 1, 1, 0, 2, 1, 1, 1, null) == 1
    assert b(null, one, one, one, one, 1, 1, 1, 2, 1, 1, 1, null) == 3


def test_argument_checks_of_the_added_entry_points():
    from gmc import _native
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)
    r = _native.lib.gmc_relu_fixed_point
    assert r(one, one, one, one, null, 1, 4, 5, null) == 1        # D = 5
    assert r(one, one, one, one, null, 1, 0, 2, null) == 1        # no components
    assert r(null, one, one, one, null, 1, 4, 2, null) == 3       # NULL mixtures
    assert r(one, one, one, one, null, 0, 4, 2, null) == 0        # nothing to do
    h = _native.lib.gmc_eval_inversed_host
    assert h(one, one, null, one, null, null, 1, 1, 1, 4, 1, 1, 1, 0) == 1          # D = 4
    assert h(one, one, null, one, null, null, 2, 1, 1, 2, 3, 1, 1, 0) == 2          # batch broadcast mismatch
    assert h(null, one, null, one, null, null, 1, 1, 1, 2, 1, 1, 1, 0) == 3         # NULL mixture
    assert h(one, one, null, null, null, null, 1, 1, 1, 2, 1, 1, 1, 0) == 3         # neither output nor gradient asked
    assert h(one, one, null, one, one, null, 1, 1, 1, 2, 1, 1, 1, 0) == 3           # gradient without grad_out


def test_argument_checks_of_the_lbvh_options_and_the_normalisation_entry_points():
    from gmc import _native
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)  # never dereferenced: argument checks come first
    f = _native.lib.gmc_lbvh_build_ex
    assert f(one, 1, 8, 4, 0, 0, 0.001, one, one, null, null) == 1               # D = 4
    assert f(one, 1, 8, 2, 5, 0, 0.001, one, one, null, null) == 4               # no such key layout
    assert f(one, 1, 8, 2, 2, 1, 0.001, one, one, one, null) == 4                # boxes need the component id in the key
    assert f(one, 1, 1, 2, 0, 0, 0.001, one, one, null, null) == 1               # a tree needs two leaves
    assert f(one, 1, 32769, 2, 0, 0, 0.001, one, one, null, null) == 1           # beyond the 16-bit node indices
    assert f(null, 1, 8, 2, 0, 0, 0.001, one, one, null, null) == 3              # NULL mixture
    assert f(one, 0, 8, 2, 1, 0, 0.001, one, one, null, null) == 0               # nothing to do
    t = _native.lib.gmc_trace_scale
    assert t(one, one, one, 1, 4, 5, null) == 1 and t(null, one, one, 1, 4, 2, null) == 3 and t(one, one, one, 0, 4, 2, null) == 0
    sc = _native.lib.gmc_spatial_scale
    assert sc(one, one, one, 1, 0, 2, null) == 1 and sc(one, null, one, 1, 4, 2, null) == 3 and sc(one, one, one, 0, 4, 3, null) == 0
    n = _native.lib.gmc_input_normalise
    assert n(one, one, null, null, 1, 8, 4, 1000, one, one, null) == 1            # D = 4
    assert n(one, one, null, null, 1, 8, 3, 1, one, one, null) == 1               # a standard deviation needs two samples
    assert n(one, null, null, null, 1, 8, 3, 1000, one, one, null) == 3           # neither seed nor uniform numbers
    assert n(one, one, null, null, 1, 8, 3, 1000, null, one, null) == 3           # NULL output
    assert n(one, one, null, null, 1, 20000, 3, 1000, one, one, null) == 1        # beyond the shared-memory size
    assert n(one, one, null, null, 0, 8, 3, 1000, one, one, null) == 0            # nothing to do


def test_argument_checks_of_the_no_allocation_entry_point():
    from gmc import _native
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)  # never dereferenced: argument checks come first
    f = _native.lib.gmc_mhem_fit_forward_noalloc
    assert f(one, 0, 8, 2, 8, 4, one, one, one, null) == 0            # nothing to do
    assert f(one, 1, 8, 2, 8, 4, null, one, one, null) == 3           # NULL output
    assert f(null, 1, 8, 2, 8, 4, one, one, one, null) == 3           # NULL input
    assert f(one, 1, 8, 4, 8, 4, one, one, one, null) == 1            # D = 4
    assert f(one, 1, 8, 2, 8, 3, one, one, one, null) == 4            # reduction_n = 3
    assert f(one, (1 << 20) // 8 + 1, 8, 2, 8, 4, one, one, one, null) == 9   # beyond the built-in scratch


def test_cpu_tensors_are_rejected_loudly():
    import gmc.cpp.extensions.evaluate_inversed.evaluate_inversed as ev
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        ev.apply(torch.zeros(1, 1, 1, 7), torch.zeros(1, 1, 1, 2))
    with pytest.raises(RuntimeError, match="last dimension"):
        ev.apply(torch.zeros(1, 1, 1, 8), torch.zeros(1, 1, 1, 2))
    with pytest.raises(RuntimeError, match="batch dimension"):
        ev.apply(torch.zeros(2, 1, 1, 7), torch.zeros(3, 1, 1, 2))
