"""Packed Gaussian mixtures and their functional operators.

Counterpart of the reference's src/gmc/mixture.py. A mixture is a float32 tensor
[n_batch, n_layers, n_components, 1 + D + D*D] = [weight | position | covariance (row-major DxD)], D in {2, 3};
"layers" are feature channels; weights are integrals ("priors"), not amplitudes.
Evaluation, matrix inversion and integration run as CUDA kernels of libgmc_b200.so.
"""
import math

import torch
from torch import Tensor

from . import _native
from . import mat_tools
from . import config
from .cpp.extensions.evaluate_inversed import evaluate_inversed as cppExtensionsEvaluateInversed


# ---------------------------------------------------------------------------------------------
# shape accessors and packing (reference mixture.py:11-67)
# ---------------------------------------------------------------------------------------------
def n_dimensions(mixture: Tensor) -> int:
    vector_length = mixture.shape[-1]
    if vector_length == 7:
        return 2
    if vector_length == 13:
        return 3
    raise AssertionError(f"Invalid mixture with shape {mixture.shape}: last dimension must be 7 (2d) or 13 (3d)")


def n_batch(mixture: Tensor) -> int:
    return mixture.shape[0]


def n_layers(mixture: Tensor) -> int:
    """Number of feature channels."""
    return mixture.shape[1]


def n_components(mixture: Tensor) -> int:
    return mixture.shape[2]


def weights(mixture: Tensor) -> Tensor:
    return mixture[:, :, :, 0]


def positions(mixture: Tensor) -> Tensor:
    return mixture[:, :, :, 1:(n_dimensions(mixture) + 1)]


def covariances(mixture: Tensor) -> Tensor:
    d = n_dimensions(mixture)
    return mixture[:, :, :, (d + 1):].view(*mixture.shape[:-1], d, d)


def pack_mixture(weights: Tensor, positions: Tensor, covariances: Tensor) -> Tensor:
    assert weights.shape[0] == positions.shape[0] == covariances.shape[0]
    assert weights.shape[1] == positions.shape[1] == covariances.shape[1]
    assert weights.shape[2] == positions.shape[2] == covariances.shape[2]
    d = positions.shape[-1]
    assert d == 2 or d == 3
    lead = positions.shape[:-1]
    return torch.cat((weights.reshape(*lead, 1), positions, covariances.reshape(*lead, d * d)), dim=-1)


def is_valid_mixture(mixture: Tensor) -> bool:
    assert not torch.any(torch.isnan(mixture))
    assert not torch.any(torch.isinf(mixture))
    assert len(mixture.shape) == 4
    assert n_dimensions(mixture) in (2, 3)
    assert torch.all(covariances(mixture).det() > 0)
    return True


def is_valid_mixture_and_constant(mixture: Tensor, constant: Tensor) -> bool:
    assert is_valid_mixture(mixture)
    assert len(constant.shape) == 2
    assert constant.shape[0] == 1 or constant.shape[0] == mixture.shape[0]
    assert constant.shape[1] == 1 or constant.shape[1] == mixture.shape[1]
    assert mixture.device == constant.device
    return True


# ---------------------------------------------------------------------------------------------
# integration (reference mixture.py:87-91)
# ---------------------------------------------------------------------------------------------
class _Integrate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mixture: Tensor):
        mixture = mixture.contiguous()
        _native.require_cuda_f32(mixture, "mixture")
        b, l, g, _ = mixture.shape
        out = torch.empty((b, l), dtype=torch.float32, device=mixture.device)
        ctx.mixture_shape = mixture.shape
        if g == 0 or b * l == 0:
            return out.zero_()
        with torch.cuda.device_of(mixture):
            _native.check(_native.lib.gmc_integrate(_native.ptr(mixture), _native.ptr(out), b * l, g,
                                                    n_dimensions(mixture), _native.stream_of(mixture)), "integrate")
        return out

    @staticmethod
    def backward(ctx, grad_output):
        grad = torch.zeros(ctx.mixture_shape, dtype=grad_output.dtype, device=grad_output.device)
        grad[..., 0] = grad_output.unsqueeze(-1)
        return grad


def integrate(mixture: Tensor) -> Tensor:
    """Integral of every mixture = sum of its weights, [n_batch, n_layers]."""
    return _Integrate.apply(mixture)


# ---------------------------------------------------------------------------------------------
# evaluation (reference mixture.py:94-149)
# ---------------------------------------------------------------------------------------------
def evaluate_inversed(mixture: Tensor, xes: Tensor) -> Tensor:
    """Mixture whose matrix slot holds INVERSE covariances, evaluated at xes [1|B, 1|L, N, D] -> [B, L, N]."""
    return cppExtensionsEvaluateInversed.apply(mixture, xes)


def evaluate_inversed_with_amplitude_mixture(mixture: Tensor, xes: Tensor) -> Tensor:
    return cppExtensionsEvaluateInversed.apply(convert_amplitudes_to_priors(mixture), xes)


def evaluate(mixture: Tensor, xes: Tensor) -> Tensor:
    """Covariance-form mixture evaluated at xes -> [n_batch, n_layers, n_xes]."""
    inv = mat_tools.inverse(covariances(mixture))
    return evaluate_inversed(pack_mixture(weights(mixture), positions(mixture), inv), xes)


def _componentwise_inversed_dense(gaussians: Tensor, xes: Tensor, component_axis_first: bool) -> Tensor:
    b, l, g, _ = gaussians.shape
    d = n_dimensions(gaussians)
    assert len(xes.shape) == 4
    assert xes.shape[0] in (1, b) and xes.shape[1] in (1, l) and xes.shape[3] == d
    n = xes.shape[2]
    diff = xes.view(xes.shape[0], xes.shape[1], n, 1, d) - positions(gaussians).view(b, l, 1, g, d)
    s = covariances(gaussians).view(b, l, 1, g, d, d)
    quad = (diff.unsqueeze(-2) @ s @ diff.unsqueeze(-1)).view(b, l, n, g)
    norm = torch.sqrt(torch.det(s) / ((2.0 * math.pi) ** d))
    values = weights(gaussians).view(b, l, 1, g) * norm * torch.exp(-0.5 * quad)
    return values.transpose(2, 3) if component_axis_first else values


def old_evaluate_inversed(mixture: Tensor, xes: Tensor) -> Tensor:
    """Dense PyTorch formulation (memory hungry); kept for API compatibility and as a cross-check."""
    return _componentwise_inversed_dense(mixture, xes, False).sum(-1)


def evaluate_componentwise_inversed(gaussians: Tensor, xes: Tensor) -> Tensor:
    """Value of every component at every x: [n_batch, n_layers, n_xes, n_components]."""
    return _componentwise_inversed_dense(gaussians, xes, False)


def evaluate_componentwise(mixture: Tensor, xes: Tensor) -> Tensor:
    inv = mat_tools.inverse(covariances(mixture))
    return evaluate_componentwise_inversed(pack_mixture(weights(mixture), positions(mixture), inv), xes)


def evaluate_with_activation_fun(mixture: Tensor, bias: Tensor, xes: Tensor) -> Tensor:
    assert is_valid_mixture_and_constant(mixture, bias)
    values = evaluate(mixture, xes) + bias.unsqueeze(-1)
    return torch.clamp_min(values, 0.00001)


# ---------------------------------------------------------------------------------------------
# construction and algebra (reference mixture.py:203-317)
# ---------------------------------------------------------------------------------------------
def generate_random_mixtures(n_batch: int = 1, n_layers: int = 1, n_components: int = 1, n_dims: int = 2,
                             pos_radius: float = 10, cov_radius: float = 10,
                             weight_min: float = -1, weight_max: float = 1,
                             device: torch.device = 'cpu') -> Tensor:
    assert n_batch > 0 and n_layers > 0 and n_components > 0
    assert n_dims == 2 or n_dims == 3
    assert weight_min < weight_max
    w = torch.rand(n_batch, n_layers, n_components, dtype=torch.float32, device=device) * (weight_max - weight_min) + weight_min
    p = torch.rand(n_batch, n_layers, n_components, n_dims, dtype=torch.float32, device=device) * 2 * pos_radius - pos_radius
    c = mat_tools.gen_random_positive_definite((n_batch, n_layers, n_components, n_dims, n_dims), device=device) * cov_radius
    return pack_mixture(w, p, c)


def _polynomial_mul_repeat(A: Tensor, B: Tensor) -> (Tensor, Tensor):
    """All pairs of components of A and B: A is tiled, B's components are each repeated n_components(A) times."""
    reps = [1] * A.dim()
    reps[2] = B.shape[2]
    return A.repeat(reps), B.repeat_interleave(A.shape[2], dim=2)


def convolve(m1: Tensor, m2: Tensor) -> Tensor:
    """Exact convolution of two mixtures with equal layer counts: every pair gives (w1 w2, mu1 + mu2, C1 + C2)."""
    assert n_batch(m1) == 1 or n_batch(m2) == 1 or n_batch(m1) == n_batch(m2)
    assert n_layers(m1) == n_layers(m2)
    assert n_dimensions(m1) == n_dimensions(m2)
    assert is_valid_mixture(m1)
    assert is_valid_mixture(m2)
    m1, m2 = _polynomial_mul_repeat(m1, m2)
    summed = m1 + m2
    assert (torch.det(covariances(summed)) > 0).all()
    w = (weights(m1) * weights(m2)).unsqueeze(-1)
    result = torch.cat((w, summed[:, :, :, 1:]), dim=-1)
    assert is_valid_mixture(result)
    return result


def spatial_scale(m: Tensor, scaling_factors: Tensor) -> Tensor:
    """Scales positions and covariances; weights (integrals) are unchanged. scaling_factors: [B, L, 1 or D]."""
    assert len(scaling_factors.shape) == 3
    sf = scaling_factors.unsqueeze(-2)
    p = positions(m) * sf
    if sf.shape[-1] == n_dimensions(m):
        cs = torch.diag_embed(sf)
        c = cs @ covariances(m) @ cs
    else:
        cs = sf.unsqueeze(-1)
        c = cs * cs * covariances(m)
    return pack_mixture(weights(m), p, c)


def convert_priors_to_amplitudes2(weights: torch.Tensor, covariances: torch.Tensor) -> torch.Tensor:
    d = covariances.shape[-1]
    return weights / (covariances.det().sqrt() * math.sqrt((2 * math.pi) ** d))


def convert_priors_to_amplitudes(gm: torch.Tensor) -> torch.Tensor:
    c = covariances(gm)
    return pack_mixture(convert_priors_to_amplitudes2(weights(gm), c), positions(gm), c)


def convert_amplitudes_to_priors(gm: torch.Tensor) -> torch.Tensor:
    d = n_dimensions(gm)
    c = covariances(gm)
    return pack_mixture(weights(gm) * (c.det().sqrt() * math.sqrt((2 * math.pi) ** d)), positions(gm), c)
