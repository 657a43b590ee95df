"""GPU: the fit entry point that brings its own scratch (gmc_mhem_fit_forward_noalloc) against the regular one.

Some hosts of the library cannot allocate device memory when they call it (all of the GPU is already in their own
pools, or they only own input and output buffers), so this variant keeps its Morton-key scratch in an array built into
the library. It must give exactly what gmc_mhem_fit_forward gives, also on a second call that finds the previous call's
keys still in the shared array. Collected last on purpose: a run that stops at the first failure has then already run
every other test. Works in a fresh process too (its first call does the per-device set-up)."""
import numpy as np
import pytest
import torch

import synthetic_inputs as synthetic

pytestmark = pytest.mark.gpu


def _mixture(n_batch, n_layers, n_components, seed, n_dims=2):
    if n_dims == 2:
        m = synthetic.fit_target_2d(n_batch, n_layers, n_components, seed)
        m[..., 0] = m[..., 0].abs() + 0.01
    else:
        g = torch.Generator().manual_seed(seed)
        shape = (n_batch, n_layers, n_components)
        cov, _ = synthetic.covariances_and_inverses(shape, 3, 0.03, 0.15, g)
        m = synthetic.pack(torch.rand(shape, generator=g) * 0.8 + 0.2, torch.rand(*shape, 3, generator=g) * 2 - 1, cov)
    return m.cuda().contiguous()


def _call(name, mixture, K, R, with_scratch):
    from gmc import _native
    b, l, g, v = mixture.shape
    n_dims = {7: 2, 13: 3}[v]
    dev = mixture.device
    fitting = torch.full((b, l, K, v), float("nan"), device=dev)
    nodes = torch.full((b, l, 2 * g - 1, 4), -7, dtype=torch.int16, device=dev)
    attribs = torch.full((b * l, _native.lib.gmc_mhem_fit_attribute_floats(g, n_dims, R)), float("nan"), device=dev)
    args = [_native.ptr(mixture), b * l, g, n_dims, K, R, _native.ptr(fitting), _native.ptr(nodes), _native.ptr(attribs)]
    keys = None
    if with_scratch:
        keys = torch.empty((b * l, g), dtype=torch.int64, device=dev)
        args.append(_native.ptr(keys))
    args.append(_native.stream_of(mixture))
    status = getattr(_native.lib, name)(*args)
    torch.cuda.synchronize()
    return status, fitting, nodes, attribs


def test_noalloc_entry_point_matches_the_regular_one_on_two_calls_in_a_row():
    # second call: smaller problem, so stale keys of the first call sit behind and between the new ones
    for (b, l, g, K, R, seed, n_dims) in ((3, 4, 1024, 64, 4, 21, 2), (2, 3, 100, 32, 2, 22, 2), (2, 2, 64, 16, 2, 23, 3)):
        m = _mixture(b, l, g, seed, n_dims)
        s0, fit_ref, nodes_ref, attr_ref = _call("gmc_mhem_fit_forward", m, K, R, True)
        s1, fit_new, nodes_new, attr_new = _call("gmc_mhem_fit_forward_noalloc", m, K, R, False)
        assert s0 == 0 and s1 == 0
        assert torch.isfinite(fit_new).all()
        assert torch.equal(nodes_new, nodes_ref)
        # tolerance of the fit tests (relative 5e-3 per slot); the two paths run the same kernels, so in practice equal
        np.testing.assert_allclose(fit_new.cpu().numpy(), fit_ref.cpu().numpy(), rtol=5e-3, atol=1e-5)
        np.testing.assert_allclose(attr_new.cpu().numpy().view(np.int32), attr_ref.cpu().numpy().view(np.int32))


def test_noalloc_entry_point_refuses_problems_beyond_its_built_in_scratch():
    from gmc import _native
    cap = _native.lib.gmc_mhem_fit_forward_noalloc_capacity()
    assert cap == 1 << 20
    m = _mixture(1, 1, 8, 3)
    one = _native.ptr(m)
    # n_mixtures * n_components = cap + 8: refused by the size check, before any pointer is touched
    status = _native.lib.gmc_mhem_fit_forward_noalloc(one, cap // 8 + 1, 8, 2, 8, 4, one, one, one, _native.stream_of(m))
    assert status == 9
    assert b"built-in scratch" in _native.lib.gmc_status_string(status)
