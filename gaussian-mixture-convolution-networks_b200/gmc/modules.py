"""Network modules on Gaussian mixtures: convolution with learnable mixture kernels, ReLU fitting, normalisations.

Counterpart of the reference's src/gmc/modules.py (forward paths and parameters; the debug renderers of the
reference need matplotlib and an OpenGL visualiser and are not part of this package). Module and parameter names are
kept, so a state_dict of the reference's Convolution / BatchNorm / CovScaleNorm loads unchanged.
"""
import math
import typing

import torch
from torch import Tensor

import gmc.mixture as gm
import gmc.fitting
import gmc.mat_tools as mat_tools
import gmc.cpp.extensions.convolution.binding as cpp_convolution
import gmc.cpp.extensions.convolution_fitting.binding as cpp_convolution_fitting


class ConvolutionConfig:
    def __init__(self, learnable_radius=False):
        self.learnable_radius = learnable_radius


class Convolution(torch.nn.modules.Module):
    """Convolution of an n_layers_in-channel mixture with n_layers_out x n_layers_in kernel mixtures of
    n_kernel_components Gaussians each. n_fitting_components < 0: exact convolution (Cin * G * Gk output components
    per channel); otherwise the fused convolution + fit to n_fitting_components."""

    def __init__(self, config: ConvolutionConfig, n_layers_in: int, n_layers_out: int, n_kernel_components: int = 4,
                 n_dims: int = 2, position_range: float = 1, covariance_range: float = 0.25, weight_sd=0.1,
                 weight_mean=0.0, learn_positions: bool = True, learn_covariances: bool = True,
                 covariance_epsilon: float = 0.05, n_fitting_components: int = -1):
        super(Convolution, self).__init__()
        self.config = config
        self.n_channels_in = n_layers_in
        self.n_channels_out = n_layers_out
        self.n_kernel_components = n_kernel_components
        self.n_dims = n_dims
        if config.learnable_radius:
            self.position_range = torch.nn.Parameter(torch.tensor([position_range], dtype=torch.float32))
            self.covariance_range = torch.nn.Parameter(torch.tensor([covariance_range], dtype=torch.float32))
        else:
            self.position_range = position_range
            self.covariance_range = covariance_range
        self.weight_sd = weight_sd
        self.weight_mean = weight_mean
        self.covariance_epsilon = covariance_epsilon
        self.learn_positions = learn_positions
        self.learn_covariances = learn_covariances
        self.last_in = None
        self.n_fitting_components = n_fitting_components

        shape = (n_layers_out, n_layers_in, n_kernel_components)
        self.weights = torch.nn.Parameter(torch.randn(*shape, 1, dtype=torch.float32))
        if n_dims == 2:
            # one component in the centre, the others on the unit circle
            angles = torch.arange(0, 2 * math.pi, 2 * math.pi / (n_kernel_components - 1))
            xs = torch.cat((torch.zeros(1), torch.sin(angles)))
            ys = torch.cat((torch.zeros(1), torch.cos(angles)))
            positions = torch.stack((xs, ys), dim=1).view(1, 1, n_kernel_components, 2).repeat(n_layers_out, n_layers_in, 1, 1)
        else:
            assert n_dims == 3
            # one component in the centre, the others uniform on the unit sphere
            z = torch.rand(*shape, 1, dtype=torch.float32) * 2 - 1
            theta = torch.rand(*shape, 1, dtype=torch.float32) * 2 * math.pi - math.pi
            r = torch.sqrt(1 - z * z)
            positions = torch.cat((torch.sin(theta) * r, torch.cos(theta) * r, z), dim=3)
            positions[:, :, 0, :] = 0
        self.positions = torch.nn.Parameter(positions)
        # covariances are A A^T + epsilon I with a learnable, initially near-identity A
        factors = (torch.rand(*shape, n_dims, n_dims, dtype=torch.float32) * 2 - 1) * 0.05 + torch.eye(n_dims)
        self.covariance_factors = torch.nn.Parameter(factors)
        self.set_requires_grad(True)

    def set_requires_grad(self, flag: bool):
        self.weights.requires_grad = flag
        self.positions.requires_grad = self.learn_positions and flag
        self.covariance_factors.requires_grad = self.learn_covariances and flag

    def kernels(self) -> Tensor:
        if not (self.training or torch.is_grad_enabled()):
            # inference: the kernel mixture only changes when a parameter does
            def stamp(v):     # parameters by storage and version, plain numbers by value
                return (v.data_ptr(), v._version) if isinstance(v, torch.Tensor) else v
            key = tuple(stamp(v) for v in (self.weights, self.positions, self.covariance_factors, self.position_range,
                                           self.covariance_range, self.weight_sd, self.weight_mean,
                                           self.covariance_epsilon))
            cached = getattr(self, "_kernels_cache", None)
            if cached is None or cached[0] != key:
                cached = (key, self._build_kernels().detach())
                self._kernels_cache = cached
            return cached[1]
        return self._build_kernels()

    def _build_kernels(self) -> Tensor:
        weights = self.weights * self.weight_sd + self.weight_mean
        A = self.covariance_factors
        cov = A @ A.transpose(-1, -2)
        eps = self.covariance_epsilon * torch.clamp(cov.detach().abs().max(), min=1.0)    # stays on the device
        cov = cov + torch.eye(self.n_dims, dtype=torch.float32, device=A.device) * eps
        return gm.pack_mixture(weights, self.positions * self.position_range, cov * self.covariance_range)

    def weight_decay_loss(self) -> Tensor:
        """Decays the weights towards 0 and A A^T towards the identity (positions are left alone)."""
        eye = torch.eye(self.n_dims, device=self.weights.device, dtype=self.weights.dtype)
        A = self.covariance_factors
        off = A @ A.transpose(-1, -2) - eye
        return (off * off).mean() + (self.weights * self.weights).mean()

    def forward(self, x: Tensor, x_constant: Tensor) -> typing.Tuple[Tensor, Tensor]:
        self.last_in = (x.detach(), x_constant.detach())
        kernels = self.kernels()
        if self.n_fitting_components < 0:
            out_mixtures = cpp_convolution.apply(x, kernels)
        else:
            out_mixtures = cpp_convolution_fitting.apply(x, kernels, self.n_fitting_components)
        # a constant convolved with a kernel is the constant times the kernel's integral
        n_batch = x_constant.shape[0]
        a = x_constant.view(n_batch, 1, gm.n_layers(x))
        b = gm.integrate(kernels).view(1, self.n_channels_out, gm.n_layers(x))
        return out_mixtures, (a * b).sum(dim=2)


class ReLUFittingConfig:
    def __init__(self):
        self.fitting_method = gmc.fitting.fixed_point_only
        self.fitting_config = gmc.fitting.Config()


class ReLUFitting(torch.nn.modules.Module):
    """Approximates ReLU(mixture + constant) by a mixture with n_output_gaussians components (+ a constant)."""

    def __init__(self, config: ReLUFittingConfig, n_layers: int, n_output_gaussians: int, n_input_gaussians: int = -1,
                 convolution_layer: str = ""):
        super(ReLUFitting, self).__init__()
        self.config = config
        self.n_layers = n_layers
        self.n_input_gaussians = n_input_gaussians
        self.n_output_gaussians = n_output_gaussians
        self.convolution_layer = convolution_layer
        self.last_in = None
        self.last_out = None
        self.last_steps = None

    def forward(self, x_m: Tensor, x_constant: Tensor, tensorboard=None) -> typing.Tuple[Tensor, Tensor]:
        y_m, y_constant, steps = self.config.fitting_method(x_m, x_constant, self.n_output_gaussians,
                                                            self.config.fitting_config, tensorboard,
                                                            convolution_layer=self.convolution_layer)
        self.last_in = (x_m.detach(), x_constant.detach())
        self.last_out = (y_m.detach(), y_constant.detach())
        self.last_steps = [s.detach() for s in steps]
        return y_m, y_constant


class Dropout(torch.nn.modules.Module):
    """Drops whole feature channels in training: weight 0, position 0, identity covariance; the rest is rescaled."""

    def __init__(self, drop_percentage: float):
        super(Dropout, self).__init__()
        self.drop_percentage = drop_percentage

    def forward(self, x: typing.Tuple[Tensor, typing.Optional[Tensor]]) -> typing.Tuple[Tensor, Tensor]:
        x_gm, x_constant = x
        if not self.training:
            return x_gm, x_constant
        d = gm.n_dimensions(x_gm)
        drop = (torch.rand(gm.n_batch(x_gm), gm.n_layers(x_gm), device=x_gm.device) < self.drop_percentage).unsqueeze(-1)
        zero = torch.zeros((), dtype=torch.float32, device=x_gm.device)
        w = torch.where(drop, zero, gm.weights(x_gm) * (1.0 / (1 - self.drop_percentage)))
        p = torch.where(drop.unsqueeze(-1), zero, gm.positions(x_gm))
        c = torch.where(drop.unsqueeze(-1).unsqueeze(-1), torch.eye(d, device=x_gm.device).view(1, 1, 1, d, d),
                        gm.covariances(x_gm))
        return gm.pack_mixture(w, p, c), x_constant


class CovScaleNorm(torch.nn.modules.Module):
    """Uniform spatial scaling so that the average covariance trace becomes n_dimensions; per channel over the batch
    (running average, batch_norm=True) or per sample (batch_norm=False)."""

    def __init__(self, n_layers: int, batch_norm: bool = True):
        super(CovScaleNorm, self).__init__()
        self.batch_norm = batch_norm
        self.register_buffer("averaged_cov_trace", torch.ones(n_layers))

    def inference_scale(self, n_dims: int) -> Tensor:
        """Per-channel factor of the batch variant in evaluation mode, sqrt(n_dims / averaged_cov_trace): the value
        forward() multiplies centres with (covariances get its square). Cached until the buffer changes."""
        key = (self.averaged_cov_trace.data_ptr(), self.averaged_cov_trace._version, n_dims)
        cached = getattr(self, "_scale_cache", None)
        if cached is None or cached[0] != key:
            cached = (key, torch.sqrt(n_dims / self.averaged_cov_trace.detach()).contiguous())
            self._scale_cache = cached
        return cached[1]

    def forward(self, x: typing.Tuple[Tensor, typing.Optional[Tensor]]) -> typing.Tuple[Tensor, Tensor]:
        x_gm, x_constant = x
        n_batch = gm.n_batch(x_gm)
        if self.batch_norm:
            if self.training:
                traces = mat_tools.trace(gm.covariances(x_gm))
                alpha = min(n_batch / 1000, 0.2)
                self.averaged_cov_trace = ((1.0 - alpha) * self.averaged_cov_trace + alpha * traces.mean(dim=(0, 2))).detach()
            n_batch = 1
            avg_trace = self.averaged_cov_trace.detach()
        else:
            avg_trace = mat_tools.trace(gm.covariances(x_gm)).mean(dim=2)
        factor = torch.sqrt(gm.n_dimensions(x_gm) / avg_trace).view(n_batch, gm.n_layers(x_gm), 1)
        y_gm = gm.spatial_scale(x_gm, factor)
        if x_constant is None:
            x_constant = torch.zeros(n_batch, gm.n_layers(x_gm), device=x_gm.device)
        return y_gm, x_constant


def fused_input_normalisation(x_gm: Tensor, scaling: typing.Optional[Tensor] = None, n_samples: int = 1000,
                              uniforms: typing.Optional[Tensor] = None) -> typing.Tuple[Tensor, Tensor]:
    """CovScaleNorm(1, batch_norm=False) followed by BatchNorm(1, batch_norm=False) on a one-channel mixture
    [B, 1, G, V] in one kernel (gmc_input_normalise), without autograd. `scaling` is the BatchNorm's learnable factor
    (a one-element CUDA tensor) or None. The sample positions come from `uniforms`
    ([B, n_samples, D] in [0, 1)) or from a hash of a seed drawn from torch's generator of the device."""
    from gmc import _native
    _native.require_cuda_f32(x_gm, "mixture")
    b, l, g, v = x_gm.shape
    if l != 1:
        raise RuntimeError("fused_input_normalisation handles one-channel mixtures")
    d = gm.n_dimensions(x_gm)
    x_gm = x_gm.contiguous()
    out = torch.empty_like(x_gm)
    constants = torch.empty((b, 1), dtype=torch.float32, device=x_gm.device)
    if scaling is not None:
        scaling = scaling.detach().reshape(1).contiguous()
        _native.require_cuda_f32(scaling, "scaling")
    seed = None
    if uniforms is None:
        seed = torch.randint(0, 2 ** 62, (1,), dtype=torch.int64, device=x_gm.device)
    else:
        uniforms = uniforms.contiguous()
        _native.require_cuda_f32(uniforms, "uniforms")
        n_samples = uniforms.shape[1]
    with torch.cuda.device_of(x_gm):
        _native.check(_native.lib.gmc_input_normalise(
            _native.ptr(x_gm), _native.ptr(seed), _native.ptr(uniforms), _native.ptr(scaling), b, g, d, int(n_samples),
            _native.ptr(out), _native.ptr(constants), _native.stream_of(x_gm)), "input normalisation")
    return out, constants


class BatchNorm(torch.nn.modules.Module):
    """Scales the weights so that the standard deviation of the mixture's values, sampled at random positions inside
    the box of the centres, becomes one; the sampled mean is subtracted from the constant."""

    def __init__(self, n_layers: int, batch_norm: bool = True, learn_scaling: bool = True):
        super(BatchNorm, self).__init__()
        self.batch_norm = batch_norm
        self.learnable_scaling = torch.nn.Parameter(torch.ones(n_layers)) if learn_scaling else None
        self.register_buffer("averaged_channel_sd", torch.ones(n_layers))
        self.register_buffer("averaged_channel_mean", torch.ones(n_layers))

    def forward(self, x: typing.Tuple[Tensor, typing.Optional[Tensor]]) -> typing.Tuple[Tensor, Tensor]:
        x_gm, x_constant = x
        n_batch, n_channels, d = gm.n_batch(x_gm), gm.n_layers(x_gm), gm.n_dimensions(x_gm)
        if x_constant is None:
            x_constant = torch.zeros(n_batch, n_channels, device=x_gm.device)
        if self.batch_norm and not self.training:
            # evaluation with batch statistics: only the running averages are used, so nothing is sampled
            # (the reference samples and evaluates here as well and then discards the result, modules.py:396-410)
            sd, mean = self.averaged_channel_sd.detach(), self.averaged_channel_mean.detach()
            return self._scaled(x_gm, x_constant, sd, mean, n_channels)
        n_samples = 10000 // n_batch if self.batch_norm else 1000
        centres = gm.positions(x_gm).reshape(n_batch, -1, d).detach()
        lo = centres.min(dim=1)[0].view(n_batch, 1, 1, d)
        hi = centres.max(dim=1)[0].view(n_batch, 1, 1, d)
        points = torch.rand(n_batch, n_channels, n_samples, d, device=x_gm.device)
        if d == 2:
            points = points * 1.3 - 0.15
        points = points * (hi - lo) + lo
        values = (gm.evaluate(x_gm, points) + x_constant.unsqueeze(-1)).detach()
        if self.batch_norm:
            sd, mean = torch.std_mean(values, dim=(0, 2))
            if self.training:
                alpha = min(n_batch / 1000, 0.1)
                self.averaged_channel_sd = ((1.0 - alpha) * self.averaged_channel_sd + alpha * sd).detach()
                self.averaged_channel_mean = ((1.0 - alpha) * self.averaged_channel_mean + alpha * mean).detach()
            sd, mean = self.averaged_channel_sd.detach(), self.averaged_channel_mean.detach()
        else:
            sd, mean = torch.std_mean(values, dim=2)
        return self._scaled(x_gm, x_constant, sd, mean, n_channels)

    def _scaled(self, x_gm, x_constant, sd, mean, n_channels):
        factor = 1 / sd.clamp_min(0.001)
        if self.learnable_scaling is not None:
            factor = factor * self.learnable_scaling
        factor = factor.view(-1, n_channels, 1)
        return gm.pack_mixture(gm.weights(x_gm) * factor, gm.positions(x_gm), gm.covariances(x_gm)), x_constant - mean
