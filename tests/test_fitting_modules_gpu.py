"""GPU: the Python layer above the kernels (gmc.fitting, gmc.modules, gmc.model) against golden vectors from the
reference's Python and against the CPU oracle."""
import math
import os

import numpy as np
import pytest
import torch

from conftest import ROOT, rel_inf
from oracle import cpu_oracle
import synthetic_inputs as synthetic

pytestmark = pytest.mark.gpu


def test_relu_fixed_point_matches_reference_python():
    import gmc.fitting as fitting
    golden = dict(np.load(os.path.join(ROOT, "tests", "golden", "relu_fit.npz")))
    for idx in (0, 1):
        m = torch.from_numpy(golden[f"relu{idx}_mixture"]).cuda()
        c = torch.from_numpy(golden[f"relu{idx}_constant"]).cuda()
        initial = fitting.initial_approx_to_relu(m, c)
        assert rel_inf(initial.cpu().numpy(), golden[f"relu{idx}_initial"]) < 1e-6
        fp, ret_const = fitting.fixed_point_iteration_to_relu(m, c, initial)
        assert rel_inf(fp.cpu().numpy(), golden[f"relu{idx}_fixed_point"]) < 1e-4
        assert rel_inf(ret_const.cpu().numpy(), golden[f"relu{idx}_ret_const"]) < 1e-6
        # the strategy takes the fused kernel when no gradient is needed: pinned to the same golden vectors
        out, const, steps = fitting.fixed_point_only(m, c, -1)
        assert len(steps) == 1 and rel_inf(steps[0].cpu().numpy(), golden[f"relu{idx}_initial"]) < 1e-6
        assert rel_inf(out.cpu().numpy(), golden[f"relu{idx}_fixed_point"]) < 1e-4
        assert rel_inf(const.cpu().numpy(), golden[f"relu{idx}_ret_const"]) < 1e-6
        out_g = fitting.fixed_point_only(m.clone().requires_grad_(True), c, -1)[0]
        assert torch.equal(out_g.detach(), fp)


def test_evaluate_covariance_form_and_integrate(golden_eval):
    import gmc.mixture as gm
    c = "eval04_d2"
    m_inv = torch.from_numpy(golden_eval[c + "_mixture"])
    x = torch.from_numpy(golden_eval[c + "_xes"]).cuda()
    cov = torch.linalg.inv(gm.covariances(m_inv).double()).float()
    m_cov = gm.pack_mixture(gm.weights(m_inv), gm.positions(m_inv), cov).cuda().requires_grad_(True)
    out = gm.evaluate(m_cov, x)
    assert rel_inf(out.detach().cpu().numpy(), golden_eval[c + "_out"]) < 1e-3     # two fp32 inversions in the chain
    out.sum().backward()
    assert torch.isfinite(m_cov.grad).all()
    integ = gm.integrate(m_cov)
    assert rel_inf(integ.detach().cpu().numpy(), m_inv[..., 0].double().sum(-1).numpy()) < 1e-5
    g = torch.autograd.grad(integ.sum(), m_cov)[0]
    assert torch.equal(g[..., 0], torch.ones_like(g[..., 0])) and g[..., 1:].abs().max().item() == 0


def test_matrix_inverse_against_torch():
    import gmc.mat_tools as mat_tools
    for d in (2, 3):
        m = torch.rand(1000, d, d)
        m = (m @ m.transpose(-1, -2) + torch.eye(d) * 0.01).cuda().requires_grad_(True)
        mine = mat_tools.inverse(m)
        ref = torch.linalg.inv(m.detach().double())
        assert ((mine.detach().double() - ref) ** 2).mean().item() < 1e-5     # src/gmc/test_mat_tools.py criterion
        assert rel_inf(mine.detach().cpu().numpy(), ref.cpu().numpy()) < 1e-3
        g = torch.randn(mine.shape, generator=torch.Generator().manual_seed(d)).cuda()
        g = g + g.transpose(-1, -2)            # symmetric incoming gradient: the case the operator is written for
        mine.backward(g)
        m64 = m.detach().double().requires_grad_(True)
        torch.linalg.inv(m64).backward(g.double())
        assert rel_inf(m.grad.cpu().numpy(), m64.grad.cpu().numpy()) < 1e-3


def test_tree_hem_against_oracle_pipeline():
    import gmc.fitting as fitting
    m = synthetic.fit_target_2d(2, 3, 256, 31)
    m[..., 0] = m[..., 0].abs() + 0.01
    out = fitting.tree_hem(m.cuda(), 32, 4).cpu().numpy().reshape(-1, 32, 7)
    # the same pipeline on the CPU: scale to mean trace D, oracle fit, scale back (src/gmc/fitting.py:342-358)
    flat = m.numpy().reshape(-1, 256, 7).astype(np.float64)
    scale = (flat[..., 3] + flat[..., 6]).mean(-1) / 2
    back = np.sqrt(scale)
    scaled = flat.copy()
    scaled[..., 1:3] /= back[:, None, None]
    scaled[..., 3:] /= scale[:, None, None]
    ref = cpu_oracle.mhem_fit_forward(scaled.astype(np.float32), 32, 4).astype(np.float64)
    ref[..., 1:3] *= back[:, None, None]
    ref[..., 3:] *= scale[:, None, None]
    err = cpu_oracle.density_rel_l2(out, ref, flat)
    assert err.max() <= 1e-3, err


def test_convolution_module_constant_path_and_exact_mode():
    import gmc.modules as modules
    import gmc.mixture as gm
    torch.manual_seed(0)
    conv = modules.Convolution(modules.ConvolutionConfig(), n_layers_in=3, n_layers_out=4, n_kernel_components=5, n_dims=2).cuda()
    x = synthetic.fit_target_2d(2, 3, 10, 4).cuda()
    const = torch.rand(2, 3).cuda()
    y, y_const = conv(x, const)
    assert y.shape == (2, 4, 3 * 10 * 5, 7)
    k = conv.kernels().detach()
    expected = (const.view(2, 1, 3) * k[..., 0].sum(-1).view(1, 4, 3)).sum(2)
    assert rel_inf(y_const.detach().cpu().numpy(), expected.cpu().numpy()) < 1e-5
    conv.n_fitting_components = 150
    y_fit, _ = conv(x, const)
    # K = T: same integral per channel as the exact convolution
    assert rel_inf(gm.integrate(y_fit.detach()).cpu().numpy(), gm.integrate(y.detach()).cpu().numpy()) < 1e-4
    y.sum().backward()
    assert conv.weights.grad is not None and torch.isfinite(conv.weights.grad).all()


def test_cov_scale_norm_makes_mean_trace_equal_d():
    # property checked by the reference's src/gmc/test_modules.py:153-172
    import gmc.modules as modules
    import gmc.mixture as gm
    import gmc.mat_tools as mat_tools
    x = synthetic.fit_target_2d(3, 4, 20, 9).cuda()
    norm = modules.CovScaleNorm(4, batch_norm=False).cuda()
    y, c = norm((x, None))
    traces = mat_tools.trace(gm.covariances(y)).mean(-1)
    assert torch.allclose(traces, torch.full_like(traces, 2.0), rtol=1e-4)
    assert c.shape == (3, 4) and c.abs().max().item() == 0


def test_net_forward_3d_is_finite_and_repeatable():
    import gmc.model as model
    cfg = model.Config(n_dims=3)
    cfg.layers = [model.Layer(8, 1, 32, 32), model.Layer(16, 1, 16, 16), model.Layer(10, 1, 8, 8)]
    torch.manual_seed(5)
    net = model.Net(config=cfg).cuda().eval()
    x = synthetic.config4_input(n_batch=6).cuda()
    with torch.no_grad():
        torch.manual_seed(1)
        a = net(x)
        torch.manual_seed(1)
        b = net(x)
    assert a.shape == (6, 10) and torch.isfinite(a).all()
    assert torch.allclose(a.exp().sum(1), torch.ones(6, device=a.device), atol=1e-4)
    assert torch.allclose(a, b, atol=1e-5)


@pytest.mark.parametrize("d", [2, 3])
def test_symeig_criteria_of_the_reference_test(d):
    # src/gmc/cpp/extensions/math/test_symeig.py: unit length, orthogonality, A v = lambda v, all within 1.5e-3 (fp32)
    import gmc.mat_tools as mat_tools
    precision = 1.5e-3
    t = torch.rand(10, 5, 100, d, d, generator=torch.Generator().manual_seed(d))
    t = (t @ t.transpose(-1, -2) + torch.eye(d) * 0.000001).cuda().requires_grad_(True)
    values, vectors = mat_tools.symeig(t)
    ref_values = torch.linalg.eigvalsh(t.detach().double())
    assert (values.detach().double() - ref_values).abs().max().item() < precision
    assert ((vectors.norm(dim=-2) - 1) ** 2).max().item() < precision
    for i in range(d):
        for j in range(i + 1, d):
            assert (vectors[..., i] * vectors[..., j]).sum(-1).abs().max().item() < precision
    errors = (t @ vectors) - vectors * values.unsqueeze(-2)
    assert errors.abs().max().item() < precision
    # backward: gradient of sum(eigenvalues) = trace -> identity
    values.sum().backward()
    eye = torch.eye(d, device=t.device).expand_as(t.grad)
    assert (t.grad - eye).abs().max().item() < 1e-3


def test_splitter_keeps_the_integral_and_reaches_the_target_count():
    import gmc.fitting as fitting
    import gmc.mixture as gm
    m = synthetic.fit_target_2d(2, 3, 12, 77, s_lo=0.02, s_hi=0.2).cuda()
    out = fitting.splitter(m, [16, 20])
    assert out.shape == (2, 3, 20, 7)
    assert rel_inf(gm.integrate(out).cpu().numpy(), gm.integrate(m).cpu().numpy()) < 1e-5
    assert torch.all(gm.covariances(out).det() > 0)


def test_render_grid_matches_direct_evaluation():
    import gmc.render as render
    import gmc.mixture as gm
    m = synthetic.fit_target_2d(2, 3, 9, 3).cuda()
    const = torch.rand(2, 3).cuda()
    img = render.render(m, const, x_low=-1, y_low=-1, x_high=1, y_high=1, width=8, height=6)
    assert img.shape == (2, 3, 8, 6)
    x = torch.tensor([[[[-1.0, -1.0], [1.0, 1.0]]]]).cuda()
    direct = gm.evaluate(m, x) + const.unsqueeze(-1)
    assert torch.allclose(img[:, :, 0, 0], direct[:, :, 0], rtol=1e-4, atol=1e-5)
    assert torch.allclose(img[:, :, -1, -1], direct[:, :, 1], rtol=1e-4, atol=1e-5)
    assert (render.render_with_relu(m, const, width=4, height=4) >= 0).all()


@pytest.mark.parametrize("method", ["fixed_point_only", "fixed_point_and_tree_hem"])
def test_net_training_step_runs_every_backward_kernel(method):
    """Forward + backward + optimiser step through Net on the GPU: convolution-fitting backward, evaluation backward
    (ReLU fixed point), matrix-inverse backward and, with the tree reduction, the BVH-MHEM backward."""
    import gmc.model as model
    import gmc.fitting as fitting
    cfg = model.Config(n_dims=2)
    cfg.layers = [model.Layer(4, 1, 24, 12), model.Layer(10, 1, 16, 8)]
    cfg.relu_config.fitting_method = getattr(fitting, method)
    torch.manual_seed(11)
    net = model.Net(config=cfg).cuda().train()
    x = synthetic.fit_target_2d(6, 1, 20, 5)
    x[..., 0] = x[..., 0].abs() + 0.1
    x = x.cuda()
    target = torch.randint(0, 10, (6,), generator=torch.Generator().manual_seed(1)).cuda()
    opt = torch.optim.Adam(net.parameters(), lr=1e-3)
    losses = []
    for _ in range(3):
        opt.zero_grad()
        torch.manual_seed(2)           # BatchNorm samples random positions
        loss = torch.nn.functional.nll_loss(net(x), target)
        loss.backward()
        grads = [p.grad for p in net.parameters() if p.grad is not None]
        assert grads and all(torch.isfinite(g).all() for g in grads)
        assert any(g.abs().max().item() > 0 for g in grads)
        opt.step()
        losses.append(loss.item())
    assert all(l == l for l in losses)
    for g in net.gmcs:
        assert g.weights.grad is not None and g.positions.grad is not None and g.covariance_factors.grad is not None


def test_graphed_forward_equals_eager_forward(monkeypatch):
    """The GMCN forward captured as a CUDA graph returns the eager result, also for a second input. The normalisation
    layers sample random positions, so the samplers (torch.rand of the module path, the seed that the fused input
    normalisation draws with torch.randint) are replaced by fixed values for the comparison."""
    import math
    import gmc.model as model
    from gmc.cuda_graph import GraphedForward

    def fixed_rand(*shape, device=None, **kwargs):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = tuple(shape[0])
        n = math.prod(shape)
        return ((torch.arange(n, device=device, dtype=torch.float32) * 0.6180339887) % 1.0).view(*shape)

    cfg = model.Config(n_dims=3)
    cfg.layers = [model.Layer(4, 1, 16, 16), model.Layer(10, 1, 8, 8)]
    torch.manual_seed(5)
    net = model.Net(config=cfg).cuda().eval()
    xs = [synthetic.config4_input(n_batch=3, seed=s).cuda() for s in (1, 2)]
    monkeypatch.setattr(torch, "rand", fixed_rand)
    monkeypatch.setattr(torch, "randint", lambda low, high, size, **kw: torch.full(tuple(size), 12345, dtype=kw.get("dtype"),
                                                                                   device=kw.get("device")))

    def fn(x):
        return net.features(x)

    graph = GraphedForward(fn, xs[0])
    for x in xs:
        with torch.no_grad():
            ref = fn(x)
        out = graph(x).clone()
        assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        graph(xs[0][:2])


@pytest.mark.parametrize("D,B,L,G", [(2, 3, 4, 16), (3, 2, 5, 8), (3, 2, 3, 64), (2, 2, 2, 48), (3, 1, 2, 300), (2, 1, 1, 1100), (2, 2, 1, 200), (3, 1, 1, 129),
                                     (3, 1, 1, 1)])
def test_fused_relu_fixed_point_equals_the_composite_path(D, B, L, G):
    """gmc_relu_fixed_point against initial_approx_to_relu + fixed_point_iteration_to_relu built from the evaluation
    kernel: several mixtures per CTA, one mixture per CTA, more components than one shared-memory chunk."""
    import gmc.fitting as fitting
    import gmc.mixture as gm
    m = (synthetic.fit_target_2d(B, L, G, 7 + G) if D == 2 else
         synthetic.config4_input(n_batch=B * L * max(1, (G + 63) // 64), seed=G).reshape(B, L, -1, 13)[:, :, :G].contiguous()).cuda()
    m[..., 0] = torch.randn(m.shape[:-1], generator=torch.Generator().manual_seed(G)).cuda()     # both signs
    c = torch.randn(B, L, generator=torch.Generator().manual_seed(1)).cuda() * 0.3
    initial_ref = fitting.initial_approx_to_relu(m, c)
    fp_ref, const_ref = fitting.fixed_point_iteration_to_relu(m, c, initial_ref)
    initial, fp, const = fitting.fused_relu_fixed_point(m, c)
    assert torch.equal(initial, initial_ref) and torch.equal(const, const_ref)
    assert torch.equal(fp[..., 1:], fp_ref[..., 1:])
    assert torch.allclose(gm.weights(fp), gm.weights(fp_ref), rtol=1e-4, atol=1e-6)
    # the strategy uses the fused kernel without autograd and the composite path with it
    with torch.no_grad():
        a = fitting.fixed_point_only(m, c, G)[0]
    b = fitting.fixed_point_only(m.clone().requires_grad_(True), c, G)[0]
    assert torch.allclose(a, b.detach(), rtol=1e-4, atol=1e-6)


def _sorted_rows(a):
    """Rows of every [.., n, V] mixture sorted lexicographically (strategies may order equal sets differently)."""
    flat = a.reshape(-1, a.shape[-2], a.shape[-1])
    return np.stack([m[np.lexsort(m.T[::-1])] for m in flat])


def test_other_relu_fit_strategies_match_reference_python():
    """fixed_point_and_max, fixed_point_and_mhem (dense EM), solver (pseudo inverse) and splitter against outputs of
    the reference's own Python (tests/golden/strategies.npz; fp64 there, fp32 kernels here)."""
    import gmc.fitting as fitting
    import gmc.mixture as gm
    golden = dict(np.load(os.path.join(ROOT, "tests", "golden", "strategies.npz")))
    for idx in (0, 1):
        m = torch.from_numpy(golden[f"s{idx}_mixture"]).cuda()
        c = torch.from_numpy(golden[f"s{idx}_constant"]).cuda()
        K = int(golden[f"s{idx}_k"])
        G = m.shape[2]
        out, const, steps = fitting.fixed_point_and_max(m, c, K)
        assert rel_inf(out.cpu().numpy(), golden[f"s{idx}_max"]) < 1e-4
        assert rel_inf(const.cpu().numpy(), golden[f"s{idx}_max_const"]) < 1e-6 and len(steps) == 2
        out, const, steps = fitting.fixed_point_and_mhem(m, c, K)
        assert len(steps) == 3 and rel_inf(steps[2].cpu().numpy(), golden[f"s{idx}_mhem_selected"]) < 1e-4
        assert rel_inf(out.cpu().numpy(), golden[f"s{idx}_mhem_f32"]) < 1e-4      # the reference's own fp32 run
        assert rel_inf(out.cpu().numpy(), golden[f"s{idx}_mhem"]) < 1e-2          # fp64: powers of about 20 |w| amplify rounding
        out, const, steps = fitting.solver(m, c, K)
        # the pseudo inverse of a badly conditioned G x G system in fp32: compare what the weights are solved for,
        # the values of the fitted mixture at the centres
        ref = torch.from_numpy(golden[f"s{idx}_solver"]).cuda().float()
        centres = gm.positions(m)
        assert rel_inf(gm.evaluate(out, centres).cpu().numpy(), gm.evaluate(ref, centres).cpu().numpy()) < 2e-2
        positive = gm.pack_mixture(gm.weights(m).abs() + 0.1, gm.positions(m), gm.covariances(m))
        split = fitting.splitter(positive, [G + 3, G + 5])
        ref_split = golden[f"s{idx}_split"]
        assert split.shape == ref_split.shape
        # The displacement of the two halves is built from a ROW of the eigenvector matrix (reference fitting.py:265),
        # i.e. it mixes components of eigenvectors whose signs are the eigen-solver's choice: the centres of the halves
        # are not pinned. Pinned: the set of (weight, covariance) rows and the weighted mean of the centres.
        D = gm.n_dimensions(m)
        mine, ref = split.cpu().numpy(), ref_split
        keep = [0] + list(range(1 + D, mine.shape[-1]))
        assert np.abs(_sorted_rows(mine[..., keep]) - _sorted_rows(ref[..., keep])).max() < 1e-3
        centre = lambda a: (a[..., :1] * a[..., 1:1 + D]).sum(-2)
        assert np.abs(centre(mine) - centre(ref)).max() < 1e-3


def test_dropout_batchnorm_and_the_two_optimiser_step():
    """Dropout drops whole channels only in training; BatchNorm (per-sample mode) makes the sampled standard deviation
    one; the training step of the reference's runners (loss optimiser + weight-decay optimiser,
    src/modelnet_classification/main.py:111-124) runs through Net."""
    import gmc.mixture as gm
    import gmc.model as model
    import gmc.modules as modules
    m = synthetic.fit_target_2d(8, 16, 10, 21).cuda()
    m[..., 0] = m[..., 0].abs() + 0.1
    const = torch.zeros(8, 16).cuda()
    drop = modules.Dropout(0.5).cuda()
    drop.eval()
    assert torch.equal(drop((m, const))[0], m)
    drop.train()
    torch.manual_seed(0)
    out, _ = drop((m, const))
    dropped = gm.weights(out).abs().sum(-1) == 0
    assert 0 < dropped.sum().item() < dropped.numel()
    assert torch.equal(gm.positions(out)[dropped], torch.zeros_like(gm.positions(out)[dropped]))
    assert torch.allclose(gm.weights(out)[~dropped], 2.0 * gm.weights(m)[~dropped])
    eye = torch.eye(2).cuda().expand_as(gm.covariances(out)[dropped])
    assert torch.equal(gm.covariances(out)[dropped], eye)

    norm = modules.BatchNorm(16, batch_norm=False).cuda()
    torch.manual_seed(1)
    y, y_const = norm((m, const))
    lo = gm.positions(y).reshape(8, -1, 2).min(1)[0].view(8, 1, 1, 2)
    hi = gm.positions(y).reshape(8, -1, 2).max(1)[0].view(8, 1, 1, 2)
    torch.manual_seed(1)                               # the layer's own 1000 sample points
    pts = (torch.rand(8, 16, 1000, 2, device="cuda") * 1.3 - 0.15) * (hi - lo) + lo
    values = (gm.evaluate(y, pts) + y_const.unsqueeze(-1)).detach()
    assert (values.std(dim=2) - 1).abs().max().item() < 1e-3
    # the constant is shifted by the mean of the UNSCALED samples, as in the reference (modules.py:425)
    unscaled_mean = (gm.evaluate(m, pts) + const.unsqueeze(-1)).mean(dim=2)
    assert torch.allclose(y_const, const - unscaled_mean, atol=1e-5)

    cfg = model.Config(n_dims=2)
    cfg.layers = [model.Layer(4, 1, 16, 8), model.Layer(10, 1, 8, 4)]
    torch.manual_seed(3)
    net = model.Net(config=cfg).cuda().train()
    kernel_optimiser = torch.optim.Adam(net.parameters(), lr=1e-3)
    weight_decay_optimiser = torch.optim.SGD(net.parameters(), lr=1e-2)
    x = synthetic.fit_target_2d(4, 1, 12, 5)
    x[..., 0] = x[..., 0].abs() + 0.1
    target = torch.tensor([1, 3, 5, 7]).cuda()
    before = net.weight_decay_loss().item()
    for _ in range(2):
        loss = torch.nn.functional.nll_loss(net(x.cuda()), target)
        kernel_optimiser.zero_grad()
        loss.backward()
        kernel_optimiser.step()
        weight_decay_optimiser.zero_grad()
        net.weight_decay_loss().backward()
        weight_decay_optimiser.step()
    assert math.isfinite(loss.item()) and net.weight_decay_loss().item() < before + 1e-3


def test_convolution_kernel_cache_follows_the_parameters():
    """In inference the kernel mixture is built once and rebuilt when a parameter changes; training never caches."""
    import gmc.modules as modules
    conv = modules.Convolution(modules.ConvolutionConfig(), 2, 3, n_kernel_components=4, n_dims=2).cuda().eval()
    with torch.no_grad():
        a = conv.kernels()
        assert conv.kernels() is a
        conv.weights.add_(1.0)
        b = conv.kernels()
        assert b is not a and not torch.equal(a, b)
    assert conv.kernels().requires_grad            # autograd on: built fresh, differentiable
    conv.train()
    with torch.no_grad():
        assert conv.kernels() is not conv.kernels()


@pytest.mark.parametrize("D", [2, 3])
def test_fused_inference_layers_equal_the_module_path(D):
    """Net.features in evaluation mode runs each layer as convolution fit + one fused kernel (weights / n_in, ReLU
    fixed-point fit, covariance-scale normalisation); it must return what the module-by-module path returns, also with
    normalisation buffers that are not all one."""
    import gmc.model as model
    cfg = model.Config(n_dims=D)
    cfg.layers = [model.Layer(6, 1, 12, 12), model.Layer(5, 1, 8, 8), model.Layer(7, 1, 4, 4)]
    torch.manual_seed(3)
    net = model.Net(config=cfg).cuda().eval()
    for i, norm in enumerate(net.norms):
        norm.averaged_cov_trace.copy_(torch.rand_like(norm.averaged_cov_trace) + 0.5 + i)
    g = torch.Generator().manual_seed(5)
    cov, _ = synthetic.covariances_and_inverses((3, 1, 20), D, 0.05, 0.3, g)
    x = synthetic.pack(torch.rand(3, 1, 20, generator=g) + 0.2, torch.rand(3, 1, 20, D, generator=g) * 2 - 1, cov).cuda()
    # the input normalisation draws sample points, by different samplers on the two paths (it has its own test):
    # both paths get its module-path result, computed once
    torch.manual_seed(11)
    with torch.no_grad():
        stored = net.norm0((x, None))

    class StoredInputNorm(torch.nn.Module):
        def forward(self, _):
            return stored

    net.norm0 = StoredInputNorm()
    with torch.no_grad():
        assert net._fused_inference_layers(x)
        fused = net.features(x)
    net._fused_inference_layers = lambda t: False
    with torch.no_grad():
        plain = net.features(x)
    assert torch.isfinite(fused).all()
    assert rel_inf(fused.cpu().numpy(), plain.cpu().numpy()) <= 1e-6
    # with autograd on, the general path is taken
    del net._fused_inference_layers
    xg = x.clone().requires_grad_(True)
    assert not net._fused_inference_layers(xg) or not torch.is_grad_enabled()


@pytest.mark.parametrize("D", [2, 3])
def test_tree_hem_scaling_kernels_equal_the_tensor_path(D):
    """tree_hem without a gradient scales through gmc_trace_scale / gmc_spatial_scale; with a gradient through the
    tensor operations of the reference (src/gmc/fitting.py:342-358). Same result up to the rounding of the mean."""
    import gmc.fitting as fitting
    import synthetic_inputs as synthetic
    g = torch.Generator().manual_seed(40 + D)
    cov, _ = synthetic.covariances_and_inverses((3, 4, 96), D, 0.02, 0.3, g)
    w = torch.rand(3, 4, 96, generator=g) + 0.05
    p = torch.rand(3, 4, 96, D, generator=g) * 4 - 2
    m = synthetic.pack(w, p, cov).cuda()
    fused = fitting.tree_hem(m, 16, 4)
    tensor_path = fitting.tree_hem(m.clone().requires_grad_(True), 16, 4).detach()
    assert fused.shape == tensor_path.shape == (3, 4, 16, 1 + D + D * D)
    assert torch.allclose(fused, tensor_path, rtol=2e-5, atol=1e-6)


@pytest.mark.parametrize("D", [2, 3])
def test_fused_input_normalisation_equals_the_two_modules(D):
    """gmc_input_normalise against CovScaleNorm(1, batch_norm=False) + BatchNorm(1, batch_norm=False) fed with the same
    uniform numbers (torch.rand patched), and the seeded path: repeatable, statistics near the sampled ones."""
    import gmc.modules as modules
    import gmc.mixture as gm
    g = torch.Generator().manual_seed(60 + D)
    B, G, n = 5, 64, 1000
    cov, _ = synthetic.covariances_and_inverses((B, 1, G), D, 0.03, 0.15, g)
    w = torch.rand(B, 1, G, generator=g) * 0.8 + 0.2
    p = torch.rand(B, 1, G, D, generator=g) * 2 - 1
    m = synthetic.pack(w, p, cov).cuda()
    uniforms = torch.rand(B, n, D, generator=g).cuda()
    norm = torch.nn.Sequential(modules.CovScaleNorm(1, batch_norm=False), modules.BatchNorm(1, batch_norm=False)).cuda().eval()
    with torch.no_grad():
        norm[1].learnable_scaling.fill_(1.7)
        real_rand = torch.rand
        torch.rand = lambda *shape, **kw: uniforms.view(B, 1, n, D)
        try:
            ref_m, ref_c = norm((m, None))
        finally:
            torch.rand = real_rand
        out_m, out_c = modules.fused_input_normalisation(m, norm[1].learnable_scaling, uniforms=uniforms)
    assert torch.allclose(out_m, ref_m, rtol=2e-4, atol=1e-6), float((out_m - ref_m).abs().max())
    assert torch.allclose(out_c, ref_c, rtol=2e-4, atol=1e-5)
    torch.manual_seed(3)
    a_m, a_c = modules.fused_input_normalisation(m, None)
    torch.manual_seed(3)
    b_m, b_c = modules.fused_input_normalisation(m, None)
    assert torch.equal(a_m, b_m) and torch.equal(a_c, b_c)
    # another thousand sample points give the same statistics up to the sampling error (large for narrow Gaussians in 3D)
    ratio = gm.weights(a_m) * 1.7 / gm.weights(out_m)
    assert (ratio > 0.5).all() and (ratio < 2.0).all()
    assert torch.equal(gm.positions(a_m), gm.positions(out_m)) and torch.equal(gm.covariances(a_m), gm.covariances(out_m))
