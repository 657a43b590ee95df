"""Fitting a mixture to ReLU(mixture + constant) and reducing the number of components.

Counterpart of the reference's src/gmc/fitting.py: the same strategy functions
`f(mixture, constant, n_components, config, tensorboard_epoch, convolution_layer) -> (fitting, constant, steps)`
(`fixed_point_only` is the default of ReLUFitting), built on gm.evaluate (CUDA) and the BVH-MHEM kernel.
"""
import typing

import torch
from torch import Tensor

import gmc.mixture as gm
import gmc.mat_tools as mat_tools
from gmc.cpp.extensions.bvh_mhem_fit import binding as cppBvhMhemFit


class Config:
    def __init__(self, n_reduction: int = 4):
        self.n_reduction = n_reduction
        self.KL_divergence_threshold = 2.0


# ---------------------------------------------------------------------------------------------
# ReLU approximation by one fixed-point step (reference fitting.py:279-312)
# ---------------------------------------------------------------------------------------------
def initial_approx_to_relu(mixture: Tensor, constant: Tensor) -> Tensor:
    """Components whose weight plus the constant is not positive get the weight -max(constant, 0)."""
    relu_const = constant.clamp_min(0)
    w = gm.weights(mixture)
    new_w = torch.where(w + constant.unsqueeze(-1) > 0, w, -relu_const.unsqueeze(-1).expand_as(w))
    return gm.pack_mixture(new_w, gm.positions(mixture), gm.covariances(mixture))


def fixed_point_iteration_to_relu(target_mixture: Tensor, target_constant: Tensor, fitting_mixture: Tensor,
                                  n_iter: int = 1) -> typing.Tuple[Tensor, Tensor]:
    """Weights x of the fitting mixture are moved towards ReLU(target) at the component centres:
    x <- x (b + 0.05) / (fit(x)(centres) + 0.05), starting from |w| + 0.1."""
    assert gm.n_batch(target_mixture) == gm.n_batch(fitting_mixture)
    assert gm.n_layers(target_mixture) == gm.n_layers(fitting_mixture)
    assert gm.n_dimensions(target_mixture) == gm.n_dimensions(fitting_mixture)
    assert target_mixture.device == fitting_mixture.device

    positions = gm.positions(fitting_mixture)
    covariances = gm.covariances(fitting_mixture)
    ret_const = target_constant.clamp_min(0)
    b = gm.evaluate(target_mixture, positions) + target_constant.unsqueeze(-1)
    b = b.clamp_min(0) - ret_const.unsqueeze(-1)

    x = gm.weights(fitting_mixture).abs() + 0.1
    for _ in range(n_iter):
        x = x.abs()
        x = x * (b + 0.05) / (gm.evaluate(gm.pack_mixture(x, positions, covariances), positions) + 0.05)
    return gm.pack_mixture(x, positions, covariances), ret_const


def generate_random_sampling(m: Tensor, n: int) -> Tensor:
    """n uniform points per (batch, layer) inside the box of the centres grown by one standard deviation."""
    md = m.detach()
    sd = torch.sqrt(torch.diagonal(gm.covariances(md), dim1=-2, dim2=-1))
    hi = (gm.positions(md) + sd).max(dim=2, keepdim=True)[0]
    lo = (gm.positions(md) - sd).min(dim=2, keepdim=True)[0]
    return torch.rand(gm.n_batch(m), gm.n_layers(m), n, gm.n_dimensions(m), device=m.device) * (hi - lo) + lo


def mse(target_mixture: Tensor, target_constant: Tensor, fitting_mixture: Tensor, fitting_constant: Tensor,
        test_points: Tensor = None, with_activation: bool = True) -> float:
    if test_points is None:
        test_points = generate_random_sampling(target_mixture, 500)
    if with_activation:
        truth = gm.evaluate_with_activation_fun(target_mixture, target_constant, test_points)
    else:
        truth = gm.evaluate(target_mixture, test_points)
    mean, sd = truth.mean(), truth.std()
    truth = (truth - mean) / sd
    fit = (gm.evaluate(fitting_mixture, test_points) + fitting_constant.unsqueeze(-1) - mean) / sd
    return ((fit - truth) ** 2).mean().item()


class _Log:
    """Optional scalar logging to a (writer, epoch) pair with an add_scalar method."""

    def __init__(self, tensorboard_epoch, mixture, layer):
        self.on = tensorboard_epoch is not None
        if self.on:
            self.writer, self.epoch = tensorboard_epoch
            self.points = generate_random_sampling(mixture, 1000)
            self.layer = layer

    def scalar(self, name, fun):
        if self.on:
            self.writer.add_scalar(name.format(self.layer), fun(self.points), self.epoch)


FUSED_FIXED_POINT_MAX_COMPONENTS = 4096


def fused_relu_fixed_point(mixture: Tensor, constant: Tensor) -> typing.Tuple[Tensor, Tensor, Tensor]:
    """(initial, fixed point, constant) of `initial_approx_to_relu` + `fixed_point_iteration_to_relu(n_iter=1)` in one
    kernel (gmc_relu_fixed_point); no gradient is recorded."""
    from gmc import _native
    m = mixture.detach().contiguous()
    c = constant.detach().contiguous()
    _native.require_cuda_f32(m, "mixture")
    _native.require_cuda_f32(c, "constant")
    fp = torch.empty_like(m)
    initial = torch.empty_like(m)
    ret_const = torch.empty_like(c)
    if m.numel() > 0:
        with torch.cuda.device_of(m):
            _native.check(_native.lib.gmc_relu_fixed_point(
                _native.ptr(m), _native.ptr(c), _native.ptr(fp), _native.ptr(ret_const), _native.ptr(initial),
                gm.n_batch(m) * gm.n_layers(m), gm.n_components(m), gm.n_dimensions(m), _native.stream_of(m)),
                "relu fixed point")
    return initial, fp, ret_const


def fused_relu_layer(mixture: Tensor, constant: typing.Optional[Tensor], weight_divisor: float = 1.0,
                     channel_scale: typing.Optional[Tensor] = None) -> typing.Tuple[Tensor, Tensor]:
    """The middle of a network layer in evaluation mode, one kernel (gmc_relu_fixed_point_layer):
    (mixture with weights / weight_divisor, constant or zero) -> ReLU fixed-point fit -> centres * f and covariances * f^2
    with f = channel_scale[layer] -> (mixture, constant). No gradient is recorded."""
    from gmc import _native
    m = mixture.detach().contiguous()
    _native.require_cuda_f32(m, "mixture")
    c = None
    if constant is not None:
        c = constant.detach().contiguous()
        _native.require_cuda_f32(c, "constant")
    f = None
    if channel_scale is not None:
        f = channel_scale.detach().contiguous()
        _native.require_cuda_f32(f, "channel_scale")
        if f.numel() != gm.n_layers(m):
            raise RuntimeError("channel_scale needs one factor per layer")
    out = torch.empty_like(m)
    ret_const = torch.empty((gm.n_batch(m), gm.n_layers(m)), dtype=torch.float32, device=m.device)
    if m.numel() > 0:
        with torch.cuda.device_of(m):
            _native.check(_native.lib.gmc_relu_fixed_point_layer(
                _native.ptr(m), _native.ptr(c), _native.ptr(out), _native.ptr(ret_const), _native.ptr(None),
                gm.n_batch(m) * gm.n_layers(m), gm.n_components(m), gm.n_dimensions(m), float(weight_divisor),
                _native.ptr(f), gm.n_layers(m), _native.stream_of(m)), "relu fixed point (layer)")
    return out, ret_const


def _fixed_point_stage(mixture, constant, log, target=None):
    needs_grad = torch.is_grad_enabled() and (mixture.requires_grad or constant.requires_grad)
    if (target is None and not needs_grad and mixture.is_cuda and mixture.dtype == torch.float32
            and 0 < gm.n_components(mixture) <= FUSED_FIXED_POINT_MAX_COMPONENTS):
        initial, fp, ret_const = fused_relu_fixed_point(mixture, constant)
        log.scalar("51.1 fitting {} fixed point iteration mse =", lambda p: mse(mixture, constant, fp, ret_const, p))
        return initial, fp, ret_const
    start = mixture if target is None else target
    initial = initial_approx_to_relu(start, constant)
    fp, ret_const = fixed_point_iteration_to_relu(mixture, constant, initial)
    log.scalar("51.1 fitting {} fixed point iteration mse =", lambda p: mse(mixture, constant, fp, ret_const, p))
    return initial, fp, ret_const


# ---------------------------------------------------------------------------------------------
# strategies (reference fitting.py:19-240)
# ---------------------------------------------------------------------------------------------
def fixed_point_only(mixture: Tensor, constant: Tensor, n_components: int, config: Config = Config(),
                     tensorboard_epoch=None, convolution_layer: str = None):
    log = _Log(tensorboard_epoch, mixture, convolution_layer)
    initial, fp, ret_const = _fixed_point_stage(mixture, constant, log)
    return fp, ret_const, [initial]


def splitter_and_fixed_point(mixture: Tensor, constant: Tensor, n_components, config: Config = Config(),
                             tensorboard_epoch=None, convolution_layer: str = None):
    log = _Log(tensorboard_epoch, mixture, convolution_layer)
    if isinstance(n_components, (list, tuple)):
        split = splitter(mixture, n_components)
    elif n_components != -1:
        split = splitter(mixture, [n_components])
    else:
        split = mixture
    initial, fp, ret_const = _fixed_point_stage(mixture, constant, log, target=split)
    return fp, ret_const, [split, initial]


def _log_reduction(log, mixture, constant, fp, fitting, ret_const):
    log.scalar("51.0 fitting {} all mse =", lambda p: mse(mixture, constant, fitting, ret_const, p))
    log.scalar("51.2 fitting {} reduction mse =", lambda p: mse(fp, ret_const, fitting, ret_const, p, with_activation=False))


def fixed_point_and_max(mixture: Tensor, constant: Tensor, n_components: int, config: Config = Config(),
                        tensorboard_epoch=None, convolution_layer: str = None):
    """Keeps the n_components components with the largest weights after the fixed-point step."""
    log = _Log(tensorboard_epoch, mixture, convolution_layer)
    initial, fp, ret_const = _fixed_point_stage(mixture, constant, log)
    if n_components < 0:
        return fp, ret_const, [initial]
    idx = torch.topk(fp[..., 0], n_components)[1].unsqueeze(-1).expand(-1, -1, -1, mixture.shape[-1])
    fitting = torch.gather(fp, -2, idx)
    _log_reduction(log, mixture, constant, fp, fitting, ret_const)
    return fitting, ret_const, [initial, fp]


def fixed_point_and_tree_hem(mixture: Tensor, constant: Tensor, n_components: int, config: Config = Config(),
                             tensorboard_epoch=None, convolution_layer: str = None):
    """Fixed-point step, then BVH-MHEM reduction to n_components."""
    log = _Log(tensorboard_epoch, mixture, convolution_layer)
    initial, fp, ret_const = _fixed_point_stage(mixture, constant, log)
    if n_components < 0:
        return fp, ret_const, [initial]
    fitting = tree_hem(fp, max(config.n_reduction, n_components), config.n_reduction)
    _log_reduction(log, mixture, constant, fp, fitting, ret_const)
    if n_components < config.n_reduction:
        reduced = representative_select_for_relu(fitting, n_components, config)
        fitting = mhem_fit_a_to_b(reduced, fitting, config)
    return fitting, ret_const, [initial, fp]


def fixed_point_and_tree_hem2(mixture: Tensor, constant: Tensor, n_components: int, config: Config = Config(),
                              tensorboard_epoch=None, convolution_layer: str = None):
    config.n_reduction = 2
    return fixed_point_and_tree_hem(mixture, constant, n_components, config, tensorboard_epoch, convolution_layer)


def fixed_point_and_mhem(mixture: Tensor, constant: Tensor, n_components: int, config: Config = Config(),
                         tensorboard_epoch=None, convolution_layer: str = None):
    """Fixed-point step, then one dense hierarchical-EM step onto the n_components heaviest components."""
    log = _Log(tensorboard_epoch, mixture, convolution_layer)
    initial, fp, ret_const = _fixed_point_stage(mixture, constant, log)
    if n_components < 0:
        return fp, ret_const, [initial]
    reduced = representative_select_for_relu(fp, n_components, config)
    fitting = mhem_fit_a_to_b(reduced, fp, config)
    _log_reduction(log, mixture, constant, fp, fitting, ret_const)
    return fitting, ret_const, [initial, fp, reduced]


def solver(mixture: Tensor, constant: Tensor, n_components: int, config: Config = Config(), tensorboard_epoch=None,
           convolution_layer: str = None, solver_n_samples=0):
    """Least-squares weights (pseudo inverse) so that the mixture matches ReLU(mixture + constant) at its centres
    (plus / or at random samples)."""
    log = _Log(tensorboard_epoch, mixture, convolution_layer)
    w, p, c = gm.weights(mixture), gm.positions(mixture), gm.covariances(mixture)
    points = p
    if solver_n_samples > 0:
        points = torch.cat((p, generate_random_sampling(mixture, gm.n_components(mixture) * solver_n_samples)), dim=2)
    elif solver_n_samples < 0:
        points = generate_random_sampling(mixture, gm.n_components(mixture) * (-solver_n_samples))
    ret_const = constant.clamp_min(0)
    target = (gm.evaluate(mixture, points) + constant.unsqueeze(-1)).clamp_min(0) - ret_const.unsqueeze(-1)
    A = gm.evaluate_componentwise(gm.pack_mixture(torch.ones_like(w), p, c), points)
    new_w = (torch.linalg.pinv(A) @ target.unsqueeze(-1)).squeeze(-1)
    fitting = gm.pack_mixture(new_w, p, c)
    log.scalar("51.1 fitting {} solver mse (centroids) =", lambda pts: mse(mixture, constant, fitting, ret_const, p))
    log.scalar("51.2 fitting {} solver mse (rand pos) =", lambda pts: mse(mixture, constant, fitting, ret_const, pts))
    return fitting, ret_const, []


# ---------------------------------------------------------------------------------------------
# reductions (reference fitting.py:243-276, 342-530)
# ---------------------------------------------------------------------------------------------
def _fused_tree_hem_scaling(m: Tensor) -> bool:
    return m.is_cuda and m.dtype == torch.float32 and not (torch.is_grad_enabled() and m.requires_grad)


def tree_hem(m: Tensor, n_components: int, n_reduction: int, check_inputs: bool = False) -> Tensor:
    """BVH-MHEM reduction; the mixture is scaled per (batch, layer) to a mean covariance trace of D first
    (the reference's src/gmc/fitting.py:342-358). Without a gradient the scaling runs as two small kernels of the
    library (gmc_trace_scale, gmc_spatial_scale) instead of a chain of tensor operations."""
    if _fused_tree_hem_scaling(m) and not check_inputs:
        from gmc import _native
        m = m.contiguous()
        b, l, g, v = m.shape
        d = gm.n_dimensions(m)
        forth = torch.empty((b, l), dtype=torch.float32, device=m.device)
        back = torch.empty_like(forth)
        scaled = torch.empty_like(m)
        with torch.cuda.device_of(m):
            st = _native.stream_of(m)
            _native.check(_native.lib.gmc_trace_scale(_native.ptr(m), _native.ptr(forth), _native.ptr(back), b * l, g, d, st),
                          "trace scale")
            _native.check(_native.lib.gmc_spatial_scale(_native.ptr(m), _native.ptr(forth), _native.ptr(scaled), b * l, g, d, st),
                          "spatial scale")
            fitted = cppBvhMhemFit.apply(scaled, n_components, n_reduction).contiguous()
            _native.check(_native.lib.gmc_spatial_scale(_native.ptr(fitted), _native.ptr(back), _native.ptr(fitted), b * l,
                                                        fitted.shape[2], d, st), "spatial scale")
        return fitted
    scale = mat_tools.trace(gm.covariances(m)).mean(-1, keepdim=True) / gm.n_dimensions(m)
    back = torch.sqrt(scale)
    forth = 1 / back
    if check_inputs:       # host synchronisation: off by default so that a forward pass can be captured in a CUDA graph
        assert (scale > 0).all().item()
        assert not torch.any(torch.isnan(forth)) and not torch.any(torch.isinf(forth))
    m = gm.spatial_scale(m, forth)
    m = cppBvhMhemFit.apply(m, n_components, n_reduction)
    return gm.spatial_scale(m, back)


def splitter(mixture: Tensor, iteration_targets: typing.List[int], displacement: float = 0.5,
             resize: float = 0.25) -> Tensor:
    """Splits the most elongated components along their major axis until each target count is reached."""
    d = gm.n_dimensions(mixture)
    resize_vec = torch.ones(d, device=mixture.device)
    resize_vec[-1] = resize
    for target in iteration_targets:
        k = target - gm.n_components(mixture)
        assert k > 0
        eigenvalues, eigenvectors = mat_tools.symeig(gm.covariances(mixture))
        rating = eigenvalues[..., -1]
        rating = torch.where(eigenvalues[..., -1] / eigenvalues[..., -2] > 1.04, rating, torch.zeros_like(rating))
        if d > 2:
            rating = torch.where(eigenvalues[..., 1] / eigenvalues[..., 0] > 1.04, rating, torch.zeros_like(rating))
        selected, selection = torch.topk(rating, k, dim=2)
        assert (selected > 0.00000000001).all().item()
        sel_g = selection.unsqueeze(-1).expand(-1, -1, -1, mixture.shape[-1])
        n = mixture.gather(2, sel_g)
        vals = eigenvalues.gather(2, selection.unsqueeze(-1).expand(-1, -1, -1, d))
        vecs = eigenvectors.gather(2, selection.unsqueeze(-1).unsqueeze(-1).expand(-1, -1, -1, d, d))
        shift = torch.sqrt(vals[..., -1].unsqueeze(-1)) * displacement * vecs[..., -1, :]
        w = gm.weights(n) / 2
        c = vecs @ torch.diag_embed(vals * resize_vec) @ vecs.transpose(-1, -2)
        first = gm.pack_mixture(w, gm.positions(n) + shift, c)
        second = gm.pack_mixture(w, gm.positions(n) - shift, c)
        mixture = torch.cat((mixture.scatter(2, sel_g, first), second), dim=2)
    return mixture


def mixture_to_double_gmm(mixture: Tensor) -> typing.Tuple[Tensor, Tensor, Tensor]:
    integrals = gm.weights(mixture)
    abs_integrals = integrals.abs().sum(dim=2, keepdim=True).clamp_min(0.05)
    return gm.pack_mixture(integrals / abs_integrals, gm.positions(mixture), gm.covariances(mixture)), integrals, abs_integrals


def calc_likelihoods(target: Tensor, fitting: Tensor) -> Tensor:
    """[B, L, n_target, n_fitting] likelihoods with 20 virtual points (Preiner et al., equation 9)."""
    b, l, nt, d = gm.n_batch(target), gm.n_layers(target), gm.n_components(target), gm.n_dimensions(target)
    nf = gm.n_components(fitting)
    unit = gm.pack_mixture(torch.ones_like(gm.weights(fitting)), gm.positions(fitting), gm.covariances(fitting))
    values = gm.evaluate_componentwise(unit, gm.positions(target))
    c = mat_tools.inverse(gm.covariances(fitting)).view(b, l, 1, nf, d, d) @ gm.covariances(target).view(b, l, nt, 1, d, d)
    almost = values * torch.exp(-0.5 * mat_tools.trace(c))
    return torch.pow(almost, (20 * gm.weights(target).abs()).unsqueeze(-1))


def calc_KL_divergence(target: Tensor, fitting: Tensor) -> Tensor:
    tp, tc = gm.positions(target).unsqueeze(3), gm.covariances(target).unsqueeze(3)
    fp, fc = gm.positions(fitting).unsqueeze(2), gm.covariances(fitting).unsqueeze(2)
    fci = mat_tools.inverse(fc.contiguous())
    diff = tp - fp
    maha = (diff.unsqueeze(-2) @ fci @ diff.unsqueeze(-1)).squeeze(-1).squeeze(-1)
    return 0.5 * (maha + mat_tools.trace(fci @ tc) - gm.n_dimensions(target) - torch.log(tc.det() / fc.det()))


def representative_select_for_relu(mixture: Tensor, n_components: int, config: Config = Config()) -> Tensor:
    """The n_components components with the largest |weight|."""
    assert n_components > 0
    _, order = torch.sort(gm.weights(mixture.detach()).abs(), descending=True)
    return mat_tools.my_index_select(mixture, order)[:, :, :n_components, :]


def mhem_fit_a_to_b(fitting_mixture: Tensor, target_mixture: Tensor, config: Config = Config(), tensorboard=None) -> Tensor:
    """One dense hierarchical-EM step that moves fitting_mixture towards target_mixture."""
    assert gm.n_batch(target_mixture) == gm.n_batch(fitting_mixture)
    assert gm.n_layers(target_mixture) == gm.n_layers(fitting_mixture)
    assert gm.n_dimensions(target_mixture) == gm.n_dimensions(fitting_mixture)
    b, l = gm.n_batch(target_mixture), gm.n_layers(target_mixture)
    nt, nf, d = gm.n_components(target_mixture), gm.n_components(fitting_mixture), gm.n_dimensions(target_mixture)
    dev = target_mixture.device
    target, _, abs_integrals = mixture_to_double_gmm(target_mixture)
    fitting, _, _ = mixture_to_double_gmm(fitting_mixture)

    lik = calc_likelihoods(target.detach(), fitting.detach()) * gm.weights(fitting).abs().view(b, l, 1, nf)
    resp = lik / lik.sum(3, keepdim=True).clamp_min(0.00001)
    resp = resp * gm.weights(target).abs().unsqueeze(-1)
    new_w = resp.sum(2)
    resp = resp / new_w.clamp_min(0.00001).view(b, l, 1, nf)
    new_p = (resp.unsqueeze(-1) * gm.positions(target).view(b, l, nt, 1, d)).sum(2)
    diff = gm.positions(target).view(b, l, nt, 1, d, 1) - new_p.view(b, l, 1, nf, d, 1)
    new_c = (resp.unsqueeze(-1).unsqueeze(-1) * (gm.covariances(target).view(b, l, nt, 1, d, d) + diff @ diff.transpose(-1, -2))).sum(2)
    new_c = new_c + (new_w < 0.0001).unsqueeze(-1).unsqueeze(-1) * torch.eye(d, device=dev).view(1, 1, 1, d, d) * 0.0001
    out_w = new_w.contiguous() * gm.weights(fitting).sign() * abs_integrals
    return gm.pack_mixture(out_w, new_p.contiguous(), new_c.contiguous())
