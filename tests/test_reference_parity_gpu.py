"""GPU: the CUDA kernels against the REFERENCE ITSELF.

* tests/golden/reference_native.npz: outputs of the reference's native code on the inline mixtures / gradient sets of its
  unit tests (src/gmc/cpp/extensions/unittests/support.h:228-1020) and on seeded cases.
* tests/golden/gmcn3d_forward.npz: the reference's network (src/gmc/model.py:179-218) of benchmark configuration 4, run on
  CPU with its native code, layer by layer.
* tests/golden/relu_tree_hem.npz: the reference's fixed_point_and_tree_hem (src/gmc/fitting.py:162-201) at the shape of
  benchmark configuration 2.
* the reference library itself (oracle/_ref/libgmc_ref.so) where it travelled with the repository.

Bars: Morton keys, sort permutations, node arrays, subtree ranges bit-exact; values and gradients relative 1e-4
(per tensor / per field, ||a-b||inf / ||ref||inf); fitted mixtures relative L2 density error <= 1e-3.
"""
import os

import numpy as np
import pytest
import torch

from conftest import ROOT, rel_inf
from oracle import cpu_oracle, ref_native
import synthetic_inputs as synthetic

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(ROOT, "tests", "golden")


def _fields(D):
    return (("weight", slice(0, 1)), ("position", slice(1, 1 + D)), ("covariance", slice(1 + D, None)))


def _extent_source(mixtures):
    """Copy of [n, K, V] mixtures in which unused slots (weight 0, identity covariance) repeat the first slot, so that
    the density grid spans the Gaussians that carry weight."""
    m = mixtures.copy()
    unused = m[..., 0] == 0
    m[unused] = np.broadcast_to(m[:, :1], m.shape)[unused]
    return m


@pytest.fixture(scope="module")
def native():
    return dict(np.load(os.path.join(GOLDEN, "reference_native.npz")))


def test_fit_on_the_reference_unit_test_mixtures(native):
    """LBVH + BVH-MHEM fit forward and backward of the CUDA path on every golden case. Mixtures of the reference's unit
    tests include zero weights, repeated centres and exactly equal distances."""
    import gmc.cpp.extensions.bvh_mhem_fit.binding as fit
    from gmc import lbvh
    n = int(native["n_mhem"])
    worst_fwd = worst_bwd = 0.0
    for i in range(n):
        key = f"mhem{i:03d}"
        m = torch.from_numpy(native[key + "_mixture"])
        K, R = (int(v) for v in native[key + "_kr"])
        G, V = m.shape[-2:]
        D = {7: 2, 13: 3}[V]
        keys, nodes = lbvh.build(m.cuda())
        assert np.array_equal(keys.cpu().numpy().view(np.uint64).reshape(-1, G), native[key + "_keys"]), key
        assert np.array_equal(nodes.cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4), native[key + "_nodes"]), key
        mt = m.cuda().requires_grad_(True)
        out = fit.apply(mt, K, R)
        ref = native[key + "_fitting"]
        err = rel_inf(out.detach().cpu().numpy().reshape(ref.shape), ref)
        worst_fwd = max(worst_fwd, err)
        assert err <= 2e-3, f"{key} ({native[key + '_source']}): fitting rel {err:.2e}"
        flat = native[key + "_mixture"].reshape(-1, G, V)
        dens = cpu_oracle.density_rel_l2(out.detach().cpu().numpy().reshape(ref.shape), ref, flat)
        assert dens.max() <= 1e-3, f"{key}: density {dens.max():.2e}"
        out.backward(torch.from_numpy(native[key + "_grad"]).cuda())
        gref = native[key + "_grad_target"]
        scale = max(np.abs(gref).max(), 1e-30)
        got = mt.grad.cpu().numpy().reshape(gref.shape)
        for field, sl in _fields(D):
            err = float(np.abs(got[..., sl] - gref[..., sl]).max() / scale)
            worst_bwd = max(worst_bwd, err)
            assert err <= 1e-4, f"{key} ({native[key + '_source']}) grad {field}: rel {err:.2e}"
    print(f"\nCUDA fit vs reference native on {n} cases: worst forward rel {worst_fwd:.2e}, worst gradient rel {worst_bwd:.2e}")


def test_convolution_fitting_on_the_reference_golden_cases(native):
    import gmc.cpp.extensions.convolution_fitting.binding as cf
    for i in range(int(native["n_cf"])):
        key = f"cf{i}"
        data, kernels, K = native[key + "_data"], native[key + "_kernels"], int(native[key + "_k"])
        D = {7: 2, 13: 3}[data.shape[-1]]
        d = torch.from_numpy(data).cuda().requires_grad_(True)
        k = torch.from_numpy(kernels).cuda().requires_grad_(True)
        fitting, cached, objs, sub = cf.forward(d.detach(), k.detach(), K)
        assert np.array_equal(objs.cpu().numpy(), native[key + "_nodesobjs"]), key
        assert np.array_equal(sub.cpu().numpy(), native[key + "_subtrees"]), key
        for field, sl in _fields(D):
            assert rel_inf(fitting.cpu().numpy()[..., sl], native[key + "_fitting"][..., sl]) <= 1e-4, (key, field)
        out = cf.apply(d, k, K)
        out.backward(torch.from_numpy(native[key + "_grad"]).cuda())
        for name, a, r in (("grad_data", d.grad, native[key + "_grad_data"]), ("grad_kernels", k.grad, native[key + "_grad_kernels"])):
            scale = max(np.abs(r).max(), 1e-30)
            for field, sl in _fields(D):
                err = float(np.abs(a.cpu().numpy()[..., sl] - r[..., sl]).max() / scale)
                print(f"{key} {name} {field}: rel {err:.2e}")
                assert err <= 1e-4, f"{key} {name} {field}: rel {err:.2e}"


def test_network_forward_layer_by_layer_against_the_reference_network():
    """Net.features of this package on the CUDA kernels against the reference's own network run on CPU with its native
    code: same seeded parameters (asserted through checksums), every layer's output mixture by density (<= 1e-3) and
    slot by slot, and the integrated features at 1e-3."""
    import gmc.model as model
    import gmc.mixture as gm
    golden = dict(np.load(os.path.join(GOLDEN, "gmcn3d_forward.npz")))
    cfg = model.Config(n_dims=3)
    cfg.n_classes = 64
    cfg.layers = [model.Layer(8, 1, 64, 64), model.Layer(16, 1, 32, 32), model.Layer(32, 1, 16, 16), model.Layer(64, 1, 8, 8)]
    torch.manual_seed(4)
    net = model.Net(config=cfg).eval()
    sd = net.state_dict()
    names = sorted(sd.keys())
    assert names == [str(n) for n in golden["param_names"]]
    sums = np.array([[float(sd[n].double().sum()), float(sd[n].double().abs().sum())] for n in names])
    assert np.allclose(sums, golden["param_checksums"], rtol=1e-12, atol=1e-12), "seeded parameters differ from the reference's"
    net = net.cuda()

    class StoredInputNorm(torch.nn.Module):
        """The input normalisation scales by a standard deviation estimated from random sample points; its output for
        the reference's random stream is part of the fixture and is fed to the layers as it is."""

        def forward(self, x):
            return torch.from_numpy(golden["norm0"]).cuda(), torch.from_numpy(golden["norm0_constant"]).cuda()

    net.norm0 = StoredInputNorm()
    acts, convs = [], []
    for i in range(4):
        net.norms[i].register_forward_hook(lambda mod, inp, out: acts.append(out[0].detach()))
        net.gmcs[i].register_forward_hook(lambda mod, inp, out: convs.append(out[0].detach()))
    x_in = torch.from_numpy(golden["input"]).cuda()
    with torch.no_grad():
        fused = net.features(x_in)                       # per layer: convolution fit + one fused kernel
        assert not acts, "the fused inference path does not call the layer modules"
        net._fused_inference_layers = lambda x: False    # module by module, so that the hooks see every layer
        feats = net.features(x_in)
    assert rel_inf(fused.cpu().numpy(), feats.cpu().numpy()) <= 1e-6
    for i in range(4):
        for what, got, ref in (("conv", convs[i], golden[f"conv{i}"]), ("layer", acts[i], golden[f"layer{i}"])):
            got = got.cpu().numpy()
            assert got.shape == ref.shape
            B, C, K, V = ref.shape
            target = ref.reshape(B * C, K, V)
            dens = cpu_oracle.density_rel_l2(got.reshape(B * C, K, V), target, _extent_source(target), res=24)
            print(f"{what}{i}: density rel L2 max {dens.max():.2e}, values rel {rel_inf(got, ref):.2e}")
            assert dens.max() <= 1e-3, f"{what}{i}: density {dens.max():.2e}"
    err = rel_inf(feats.cpu().numpy(), golden["features"])
    print(f"features: rel {err:.2e}")
    assert err <= 1e-3


def test_fixed_point_and_tree_hem_at_the_benchmark_shape():
    """fixed_point_and_tree_hem (ReLU fixed point, rescale, LBVH, BVH-MHEM 1024 -> 64 with R = 4, scale back) against the
    reference's Python + native code on two mixtures of benchmark configuration 2, and 3D with R = 4 and R = 2."""
    import gmc.fitting as fitting
    golden = dict(np.load(os.path.join(GOLDEN, "relu_tree_hem.npz")))
    target, constant = torch.from_numpy(golden["c2_target"]).cuda(), torch.from_numpy(golden["c2_constant"]).cuda()
    with torch.no_grad():
        out, ret_const, steps = fitting.fixed_point_and_tree_hem(target, constant, 64, fitting.Config(n_reduction=4))
    assert rel_inf(steps[1].cpu().numpy(), golden["c2_fixed_point"]) <= 1e-4
    ref = golden["c2_fitting"].reshape(-1, 64, 7)
    got = out.cpu().numpy().reshape(-1, 64, 7)
    dens = cpu_oracle.density_rel_l2(got, ref, golden["c2_fixed_point"].reshape(-1, 1024, 7))
    print(f"\nconfig-2 pipeline: density rel L2 {dens.max():.2e}, values rel {rel_inf(got, ref):.2e}")
    assert dens.max() <= 1e-3
    assert rel_inf(ret_const.cpu().numpy(), golden["c2_ret_const"]) <= 1e-6
    t3, c3 = torch.from_numpy(golden["d3_target"]).cuda(), torch.from_numpy(golden["d3_constant"]).cuda()
    for R in (4, 2):
        with torch.no_grad():
            out, _, steps = fitting.fixed_point_and_tree_hem(t3, c3, 16, fitting.Config(n_reduction=R))
        ref = golden[f"d3r{R}_fitting"].reshape(-1, 16, 13)
        dens = cpu_oracle.density_rel_l2(out.cpu().numpy().reshape(-1, 16, 13), ref, steps[1].cpu().numpy().reshape(-1, 64, 13), res=24)
        assert dens.max() <= 1e-3, f"3D R={R}: {dens.max():.2e}"


@pytest.fixture(scope="module")
def reference_library():
    if not ref_native.available():
        pytest.skip("oracle/_ref/libgmc_ref.so did not travel with the repository")
    return ref_native


@pytest.mark.parametrize("D,G,K,R", [(2, 1024, 64, 4), (3, 64, 16, 4), (2, 300, 32, 2)])
def test_fit_against_the_reference_library(reference_library, D, G, K, R):
    """Kernel against the reference library directly (not through the restatement), benchmark shapes."""
    import gmc.cpp.extensions.bvh_mhem_fit.binding as fit
    if D == 2:
        m = synthetic.fit_target_2d(2, 3, G, 31).numpy()
        m[..., 0] = np.abs(m[..., 0]) + 1e-3
    else:
        m = np.ascontiguousarray(synthetic.config4_input(6, 32).numpy().reshape(2, 3, 64, 13)[:, :, :G])
    V = m.shape[-1]
    ref_fit, dump = reference_library.mhem_fit_forward(m, K, R, dump=True)
    mt = torch.from_numpy(m).cuda().requires_grad_(True)
    out = fit.apply(mt, K, R)
    nodes = fit.forward(mt.detach(), K, R)[1]
    assert np.array_equal(nodes.cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4), dump["nodes"])
    dens = cpu_oracle.density_rel_l2(out.detach().cpu().numpy().reshape(-1, K, V), ref_fit, m.reshape(-1, G, V), res=64 if D == 2 else 24)
    assert dens.max() <= 1e-3
    grad = np.random.default_rng(G).standard_normal((2, 3, K, V)).astype(np.float32)
    out.backward(torch.from_numpy(grad).cuda())
    gref = reference_library.mhem_fit_backward(grad, m, K, R)
    got = mt.grad.cpu().numpy().reshape(gref.shape)
    scale = max(np.abs(gref).max(), 1e-30)
    for field, sl in _fields(D):
        err = float(np.abs(got[..., sl] - gref[..., sl]).max() / scale)
        print(f"fit backward D={D} G={G} K={K} R={R} {field}: rel {err:.2e}")
        assert err <= 1e-4, f"{field}: {err:.2e}"


@pytest.mark.parametrize("D,B,Cin,G,Cout,Gk,K", [(2, 2, 8, 128, 3, 5, 128), (3, 2, 1, 64, 4, 5, 64), (3, 2, 8, 64, 3, 5, 32),
                                                 (3, 2, 16, 32, 3, 5, 16), (3, 2, 32, 16, 3, 5, 8)])
def test_convolution_fitting_against_the_reference_library(reference_library, D, B, Cin, G, Cout, Gk, K):
    """Config 3 and the four layer shapes of config 4, forward and backward, kernel against the reference library."""
    import gmc.cpp.extensions.convolution_fitting.binding as cf
    if D == 2:
        data = synthetic.fit_target_2d(B, Cin, G, 1003).numpy()
    else:
        data = np.ascontiguousarray(synthetic.config4_input(B * Cin, 1004).numpy().reshape(B, Cin, 64, 13)[:, :, :G])
        data[..., 0] *= np.where(np.arange(G) % 5 == 0, -1.0, 1.0)
    g = torch.Generator().manual_seed(5 + Cin)
    w = torch.randn(Cout, Cin, Gk, generator=g) * 0.3
    p = torch.randn(Cout, Cin, Gk, D, generator=g) * 0.1
    cov, _ = synthetic.covariances_and_inverses((Cout, Cin, Gk), D, 0.02, 0.1, g)
    kernels = synthetic.pack(w, p, cov).numpy()
    d = torch.from_numpy(data).cuda().requires_grad_(True)
    k = torch.from_numpy(kernels).cuda().requires_grad_(True)
    fitting, cached, objs, sub = cf.forward(d.detach(), k.detach(), K)
    grad = np.random.default_rng(K).standard_normal(fitting.shape).astype(np.float32)
    out = cf.apply(d, k, K)
    out.backward(torch.from_numpy(grad).cuda())

    def forward():
        out_r, cached_r, objs_r, sub_r = reference_library.convolution_fitting_forward(data, kernels, K)
        assert np.array_equal(objs.cpu().numpy(), objs_r) and np.array_equal(sub.cpu().numpy(), sub_r)
        for field, sl in _fields(D):
            assert rel_inf(fitting.cpu().numpy()[..., sl], out_r[..., sl]) <= 1e-4, field

    def backward():
        gd_r, gk_r = reference_library.convolution_fitting_backward(grad, data, kernels, K)
        for name, a, r in (("grad_data", d.grad, gd_r), ("grad_kernels", k.grad, gk_r)):
            scale = max(np.abs(r).max(), 1e-30)
            for field, sl in _fields(D):
                err = float(np.abs(a.cpu().numpy()[..., sl] - r[..., sl]).max() / scale)
                assert err <= 1e-4, f"{name} {field}: {err:.2e}"

    # serial: the reference's mass pass is racy when its CPU threads run concurrently (two independent atomics,
    # src/gmc/cpp/extensions/convolution_fitting/Tree.cu:289-294); one thread at a time is race-free
    with reference_library.serial():
        forward()
        backward()
