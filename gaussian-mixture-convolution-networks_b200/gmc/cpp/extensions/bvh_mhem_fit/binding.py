"""BVH-MHEM reduction of a mixture to fewer components as a differentiable operator.

Same import path, class name and `apply(target_mixture, n_components_fitting, reduction_n)` as the reference's
src/gmc/cpp/extensions/bvh_mhem_fit/binding.py:23-61; forward runs gmc_mhem_fit_forward of libgmc_b200.so.
"""
import torch
import torch.autograd

from gmc import _native


def _dims(mixture: torch.Tensor):
    if mixture.dim() != 4 or mixture.shape[-1] not in (7, 13):
        raise RuntimeError("mixture must be [batch, layers, components, 7 or 13]")
    return mixture.shape[0], mixture.shape[1], mixture.shape[2], 2 if mixture.shape[-1] == 7 else 3


def forward(mixture: torch.Tensor, n_components_fitting: int, reduction_n: int):
    """-> (fitting [B, L, K, V], bvh_nodes int16 [B, L, 2G-1, 4], bvh_attributes float32 [B*L, A])."""
    n_batch, n_layers, n_components, n_dims = _dims(mixture)
    _native.require_cuda_f32(mixture, "mixture")
    if n_components <= 1:
        raise RuntimeError("number of components must be greater 1 for this implementation")
    if n_components >= 65535:
        raise RuntimeError("number of components must be smaller than 65535 for morton code computation")
    if reduction_n not in (2, 4):
        raise RuntimeError("reduction_n must be 2 or 4")
    if n_components_fitting % reduction_n != 0:
        raise RuntimeError("n_components_fitting must be a multiple of reduction_n")
    dev = mixture.device
    n_mix = n_batch * n_layers
    fitting = torch.empty((n_batch, n_layers, n_components_fitting, mixture.shape[-1]), dtype=torch.float32, device=dev)
    nodes = torch.empty((n_batch, n_layers, 2 * n_components - 1, 4), dtype=torch.int16, device=dev)
    a = _native.lib.gmc_mhem_fit_attribute_floats(n_components, n_dims, reduction_n)
    attribs = torch.empty((n_mix, a), dtype=torch.float32, device=dev)
    keys = torch.empty((n_mix, n_components), dtype=torch.int64, device=dev)
    with torch.cuda.device_of(mixture):
        _native.check(_native.lib.gmc_mhem_fit_forward(
            _native.ptr(mixture), n_mix, n_components, n_dims, n_components_fitting, reduction_n,
            _native.ptr(fitting), _native.ptr(nodes), _native.ptr(attribs), _native.ptr(keys),
            _native.stream_of(mixture)), "bvh_mhem_fit forward")
    return fitting, nodes, attribs


def backward(grad: torch.Tensor, fitting_mixture: torch.Tensor, target_mixture: torch.Tensor, bvh_nodes: torch.Tensor,
             bvh_attribs: torch.Tensor, n_components_fitting: int, reduction_n: int) -> torch.Tensor:
    """Gradient w.r.t. the target mixture. The saved forward tensors are left untouched."""
    n_batch, n_layers, n_components, n_dims = _dims(target_mixture)
    _native.require_cuda_f32(grad, "grad")
    _native.require_cuda_f32(target_mixture, "target_mixture")
    if tuple(grad.shape) != (n_batch, n_layers, n_components_fitting, target_mixture.shape[-1]):
        raise RuntimeError("grad has the wrong shape")
    n_mix = n_batch * n_layers
    grad_target = torch.empty_like(target_mixture)
    extra = 2 * n_components if n_components > 8192 else 0      # per-node bookkeeping of large mixtures (see gmc_b200.h)
    scratch = torch.empty((n_mix, (n_components - 1) * reduction_n * target_mixture.shape[-1] + extra), dtype=torch.float32,
                          device=target_mixture.device)
    with torch.cuda.device_of(target_mixture):
        _native.check(_native.lib.gmc_mhem_fit_backward(
            _native.ptr(grad), _native.ptr(target_mixture), n_mix, n_components, n_dims, n_components_fitting,
            reduction_n, _native.ptr(bvh_nodes), _native.ptr(bvh_attribs), _native.ptr(scratch),
            _native.ptr(grad_target), _native.stream_of(target_mixture)), "bvh_mhem_fit backward")
    return grad_target


class BvhMhemFit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, target_mixture: torch.Tensor, n_components_fitting: int, reduction_n: int):
        if not target_mixture.is_contiguous():
            target_mixture = target_mixture.contiguous()
        fitting_mixture, bvh_nodes, bvh_attribs = forward(target_mixture, n_components_fitting, reduction_n)
        ctx.save_for_backward(fitting_mixture, target_mixture, bvh_nodes, bvh_attribs)
        ctx.n_components_fitting = n_components_fitting
        ctx.reduction_n = reduction_n
        return fitting_mixture

    @staticmethod
    def backward(ctx, grad_output):
        fitting_mixture, target_mixture, bvh_nodes, bvh_attribs = ctx.saved_tensors
        grad_target = backward(grad_output.contiguous(), fitting_mixture, target_mixture, bvh_nodes, bvh_attribs,
                               ctx.n_components_fitting, ctx.reduction_n)
        if torch.any(torch.isnan(grad_target)):
            raise RuntimeError("bvh_mhem_fit backward produced NaNs "
                               f"(target has NaNs: {torch.any(torch.isnan(target_mixture)).item()}, "
                               f"grad_output has NaNs: {torch.any(torch.isnan(grad_output)).item()})")
        return grad_target, None, None


apply = BvhMhemFit.apply
