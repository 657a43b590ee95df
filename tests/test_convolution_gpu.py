"""GPU parity of the exact convolution (forward bit-exact products, backward vs the fp64 oracle) and of the fused
convolution fit forward (bit-exact sort permutation and subtree ranges, values within tolerance, density 1e-3)."""
import numpy as np
import pytest
import torch

from conftest import rel_inf
from oracle import cpu_oracle
import synthetic_inputs as synthetic

pytestmark = pytest.mark.gpu


def _inputs(D, B, Cin, G, Cout, Gk, seed):
    if D == 2:
        data, kernels, _ = synthetic.config3(n_batch=B, seed=seed)
        if Cin <= data.shape[1] and G <= data.shape[2] and Cout <= kernels.shape[0] and Gk <= kernels.shape[2]:
            return data[:, :Cin, :G].contiguous(), kernels[:Cout, :Cin, :Gk].contiguous()
    g = torch.Generator().manual_seed(seed)
    cov_d, _ = synthetic.covariances_and_inverses((B, Cin, G), D, 0.03, 0.15, g)
    data = synthetic.pack(torch.randn(B, Cin, G, generator=g), torch.rand(B, Cin, G, D, generator=g) * 2 - 1, cov_d)
    cov_k, _ = synthetic.covariances_and_inverses((Cout, Cin, Gk), D, 0.02, 0.1, g)
    kernels = synthetic.pack(torch.randn(Cout, Cin, Gk, generator=g) * 0.1, torch.randn(Cout, Cin, Gk, D, generator=g) * 0.1, cov_k)
    return data, kernels


@pytest.mark.parametrize("D,B,Cin,G,Cout,Gk", [(2, 2, 3, 16, 4, 5), (2, 3, 8, 128, 2, 5), (3, 2, 2, 33, 3, 4), (2, 1, 1, 1, 1, 1)])
def test_exact_convolution_forward_and_backward(D, B, Cin, G, Cout, Gk):
    import gmc.cpp.extensions.convolution.binding as conv
    data, kernels = _inputs(D, B, Cin, G, Cout, Gk, 50 + G)
    d = data.cuda().requires_grad_(True)
    k = kernels.cuda().requires_grad_(True)
    out = conv.apply(d, k)
    ref = cpu_oracle.convolution_forward(data.numpy(), kernels.numpy())
    assert np.array_equal(out.detach().cpu().numpy(), ref)              # one multiply or one add per value: exact
    g = torch.randn(out.shape, generator=torch.Generator().manual_seed(1))
    out.backward(g.cuda())
    gd, gk = cpu_oracle.convolution_backward(g.numpy(), data.numpy(), kernels.numpy())
    assert rel_inf(d.grad.cpu().numpy(), gd) < 1e-4
    assert rel_inf(k.grad.cpu().numpy(), gk) < 1e-4


@pytest.mark.parametrize("D,B,Cin,G,Cout,Gk,K", [(2, 2, 3, 16, 4, 5, 16), (2, 4, 8, 128, 3, 5, 128), (3, 2, 1, 64, 8, 5, 64),
                                                 (3, 2, 8, 64, 2, 5, 32), (2, 2, 2, 7, 2, 3, 42), (2, 1, 1, 2, 1, 1, 4),
                                                 (3, 2, 2, 3, 2, 2, 6),          # inputs too many to stage beside the keys
                                                 (2, 1, 4, 1000, 1, 2, 16),      # inputs too large to stage for the sums
                                                 (3, 1, 32, 16, 3, 5, 8), (3, 2, 8, 64, 2, 5, 70)])
def test_convolution_fitting_forward_matches_oracle(D, B, Cin, G, Cout, Gk, K):
    import gmc.cpp.extensions.convolution_fitting.binding as cf
    data, kernels = _inputs(D, B, Cin, G, Cout, Gk, 70 + G + K)
    fitting, cached, nodesobjs, subtrees = cf.forward(data.cuda(), kernels.cuda(), K)
    ref, ref_cached, ref_objs, ref_sub = cpu_oracle.convolution_fitting_forward(data.numpy(), kernels.numpy(), K)
    assert np.array_equal(nodesobjs.cpu().numpy(), ref_objs)            # sort permutation
    assert np.array_equal(subtrees.cpu().numpy(), ref_sub)              # tree topology + mass-driven selection
    out = fitting.cpu().numpy()
    assert np.isfinite(out).all()
    used = ref_sub[..., 0::2] >= 0
    for name, sl in (("weight", slice(0, 1)), ("position", slice(1, 1 + D)), ("covariance", slice(1 + D, None))):
        assert rel_inf(out[..., sl], ref[..., sl]) < 1e-4, name
    assert rel_inf(cached.cpu().numpy()[used], ref_cached[used]) < 1e-3
    T = Cin * G * Gk
    target = cpu_oracle.convolution_forward(data.numpy(), kernels.numpy()).reshape(B * Cout, T, -1)
    err = cpu_oracle.density_rel_l2(out.reshape(B * Cout, K, -1), ref.reshape(B * Cout, K, -1), target, res=64 if D == 2 else 24)
    assert err.max() <= 1e-3


@pytest.mark.parametrize("D,B,Cin,G,Cout,Gk,K", [(2, 2, 8, 1024, 2, 5, 128),      # T = 40960
                                                 (3, 1, 4, 512, 3, 5, 64),        # T = 10240
                                                 (2, 1, 1, 8193, 1, 1, 16)])      # just above the shared-memory size
def test_convolution_fitting_of_large_trees_matches_oracle(D, B, Cin, G, Cout, Gk, K):
    """More than 8192 products per tree: the tree is built in global scratch (gmc_convolution_fitting_forward_large).
    Same permutation, same subtree ranges, same values; the backward runs on the same outputs."""
    import gmc.cpp.extensions.convolution_fitting.binding as cf
    from oracle import autograd_oracles
    data, kernels = _inputs(D, B, Cin, G, Cout, Gk, 1000 + G + K)
    data[0, 0, 10:20, 1:1 + D] = data[0, 0, 9:10, 1:1 + D]          # equal Morton codes: ties keep ascending product index
    d = data.cuda().requires_grad_(True)
    k = kernels.cuda().requires_grad_(True)
    fitting, cached, nodesobjs, subtrees = cf.forward(d.detach(), k.detach(), K)
    ref, ref_cached, ref_objs, ref_sub = cpu_oracle.convolution_fitting_forward(data.numpy(), kernels.numpy(), K)
    assert np.array_equal(nodesobjs.cpu().numpy(), ref_objs)
    assert np.array_equal(subtrees.cpu().numpy(), ref_sub)
    out = fitting.cpu().numpy()
    for name, sl in (("weight", slice(0, 1)), ("position", slice(1, 1 + D)), ("covariance", slice(1 + D, None))):
        assert rel_inf(out[..., sl], ref[..., sl]) < 1e-4, name
    res = cf.apply(d, k, K)
    g = torch.randn(res.shape, generator=torch.Generator().manual_seed(4))
    res.backward(g.cuda())
    gd, gk, _ = autograd_oracles.convolution_fitting_backward(g.numpy(), data.numpy(), kernels.numpy(), ref_objs, ref_sub)
    for a, r in ((d.grad.cpu().numpy(), gd), (k.grad.cpu().numpy(), gk)):
        scale = max(np.abs(r).max(), 1e-30)
        assert float(np.abs(a - r).max() / scale) < 1e-4
    with pytest.raises(RuntimeError):
        cf.forward(torch.zeros(1, 1, 65536, 1 + D + D * D).cuda(), torch.zeros(1, 1, 1, 1 + D + D * D).cuda(), 4)


def test_convolution_fitting_with_k_equal_t_is_the_exact_convolution():
    # the reference's own criterion (src/gmc/test_cpp_convolution_fitting.py:60-68, test_modules.py:89-108)
    import gmc.cpp.extensions.convolution_fitting.binding as cf
    import gmc.cpp.extensions.convolution.binding as conv
    data, kernels = _inputs(2, 2, 3, 10, 2, 4, 5)
    T = 3 * 10 * 4
    fitting, _, _, _ = cf.forward(data.cuda(), kernels.cuda(), T)
    exact = conv.forward(data.cuda(), kernels.cuda())
    a, e = fitting.cpu().numpy(), exact.cpu().numpy()
    for b in range(2):
        for o in range(2):
            sa = a[b, o][np.lexsort(a[b, o].T[::-1])]
            se = e[b, o][np.lexsort(e[b, o].T[::-1])]
            assert np.abs(sa - se).max() < 1e-4


@pytest.mark.parametrize("D,B,Cin,G,Cout,Gk,K", [(2, 2, 3, 16, 4, 5, 16), (2, 3, 8, 64, 3, 5, 32), (3, 2, 2, 20, 3, 5, 24),
                                                 (2, 2, 2, 7, 2, 3, 60)])
def test_convolution_fitting_backward_matches_autograd_oracle(D, B, Cin, G, Cout, Gk, K):
    """Analytic CUDA backward against fp64 autograd through the restated forward with the tree frozen."""
    import gmc.cpp.extensions.convolution_fitting.binding as cf
    from oracle import autograd_oracles
    data, kernels = _inputs(D, B, Cin, G, Cout, Gk, 90 + G + K)
    d = data.cuda().requires_grad_(True)
    k = kernels.cuda().requires_grad_(True)
    out = cf.apply(d, k, K)
    g = torch.randn(out.shape, generator=torch.Generator().manual_seed(3))
    out.backward(g.cuda())
    _, _, objs, sub = cf.forward(data.cuda(), kernels.cuda(), K)
    gd, gk, _ = autograd_oracles.convolution_fitting_backward(g.numpy(), data.numpy(), kernels.numpy(),
                                                               objs.cpu().numpy(), sub.cpu().numpy())
    for name, a, r in (("grad_data", d.grad.cpu().numpy(), gd), ("grad_kernels", k.grad.cpu().numpy(), gk)):
        assert np.isfinite(a).all()
        scale = max(np.abs(r).max(), 1e-30)
        for field, sl in (("weight", slice(0, 1)), ("position", slice(1, 1 + D)), ("covariance", slice(1 + D, None))):
            err = float(np.abs(a[..., sl] - r[..., sl]).max() / scale)
            print(f"conv-fit backward {name} {field}: rel(tensor) {err:.2e}, rel(field) {rel_inf(a[..., sl], r[..., sl]):.2e}")
            assert err < 1e-4, f"{name} {field}: {err:.2e}"
