"""Fused convolution + reduction to n_components_fitting Gaussians as a differentiable operator.

Same import path and `apply(data, kernels, n_components_fitting)` as the reference's
src/gmc/cpp/extensions/convolution_fitting/binding.py:22-45; forward runs gmc_convolution_fitting_forward.
"""
import torch
import torch.autograd

from gmc import _native
from gmc.cpp.extensions.convolution.binding import _dims


SHARED_MEMORY_TREE_MAX = 8192      # products per tree that gmc_convolution_fitting_forward builds in shared memory


def forward(data: torch.Tensor, kernels: torch.Tensor, n_components_fitting: int):
    """-> (fitting [B, Cout, K, V], cached_pos_covs [B, Cout, K, D*D], nodesobjs int32 [B, Cout, T],
    fitting_subtrees int32 [B, Cout, 2K])."""
    dims = _dims(data, kernels)
    _native.require_cuda_f32(data, "data")
    _native.require_cuda_f32(kernels, "kernels")
    n_batch, n_in, n_comp, n_out, n_kcomp, n_dims = dims
    T = n_in * n_comp * n_kcomp
    K = int(n_components_fitting)
    dev = data.device
    fitting = torch.empty((n_batch, n_out, K, data.shape[-1]), dtype=torch.float32, device=dev)
    cached = torch.empty((n_batch, n_out, K, n_dims * n_dims), dtype=torch.float32, device=dev)
    nodesobjs = torch.empty((n_batch, n_out, T), dtype=torch.int32, device=dev)
    subtrees = torch.empty((n_batch, n_out, 2 * K), dtype=torch.int32, device=dev)
    with torch.cuda.device_of(data):
        if T > SHARED_MEMORY_TREE_MAX:
            # trees too large for shared memory are built in global scratch
            n_bytes = _native.lib.gmc_convolution_fitting_large_scratch_bytes(n_batch, n_in, n_comp, n_out, n_kcomp)
            if n_bytes == 0:
                raise _native.GmcError(f"convolution_fitting: {T} products per tree are beyond the limit of 65535")
            scratch = torch.empty((n_bytes + 15) // 16 * 2, dtype=torch.int64, device=dev)
            _native.check(_native.lib.gmc_convolution_fitting_forward_large(
                _native.ptr(data), _native.ptr(kernels), *dims, K, _native.ptr(fitting), _native.ptr(cached),
                _native.ptr(nodesobjs), _native.ptr(subtrees), _native.ptr(scratch), scratch.numel() * 8,
                _native.stream_of(data)), "convolution_fitting forward (large trees)")
        else:
            _native.check(_native.lib.gmc_convolution_fitting_forward(
                _native.ptr(data), _native.ptr(kernels), *dims, K, _native.ptr(fitting), _native.ptr(cached),
                _native.ptr(nodesobjs), _native.ptr(subtrees), _native.stream_of(data)), "convolution_fitting forward")
    return fitting, cached, nodesobjs, subtrees


def backward(grad: torch.Tensor, data: torch.Tensor, kernels: torch.Tensor, n_components_fitting: int,
             fitting: torch.Tensor, cached_pos_covs: torch.Tensor, nodesobjs: torch.Tensor, fitting_subtrees: torch.Tensor,
             needs_data: bool = True, needs_kernels: bool = True):
    """-> (grad_data, grad_kernels); a gradient that is not needed comes back as None."""
    dims = _dims(data, kernels)
    _native.require_cuda_f32(grad, "grad")
    grad_data = torch.empty_like(data) if needs_data else None
    grad_kernels = torch.empty_like(kernels) if needs_kernels else None
    with torch.cuda.device_of(data):
        _native.check(_native.lib.gmc_convolution_fitting_backward(
            _native.ptr(grad), _native.ptr(data), _native.ptr(kernels), *dims, int(n_components_fitting),
            _native.ptr(fitting), _native.ptr(cached_pos_covs), _native.ptr(nodesobjs), _native.ptr(fitting_subtrees),
            _native.ptr(grad_data), _native.ptr(grad_kernels), _native.stream_of(data)), "convolution_fitting backward")
    return grad_data, grad_kernels


class ConvolutionFitting(torch.autograd.Function):
    @staticmethod
    def forward(ctx, data: torch.Tensor, kernels: torch.Tensor, n_components_fitting: int):
        data = data.contiguous()
        kernels = kernels.contiguous()
        fitting, cached_pos_cov, nodesobjs, fitting_subtrees = forward(data, kernels, n_components_fitting)
        ctx.save_for_backward(data, kernels, fitting, cached_pos_cov, nodesobjs, fitting_subtrees)
        ctx.n_components_fitting = n_components_fitting
        return fitting

    @staticmethod
    def backward(ctx, grad_output):
        data, kernels, fitting, cached_pos_cov, nodesobjs, fitting_subtrees = ctx.saved_tensors
        grad_data, grad_kernels = backward(grad_output.contiguous(), data, kernels, ctx.n_components_fitting, fitting,
                                           cached_pos_cov, nodesobjs, fitting_subtrees,
                                           ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return grad_data, grad_kernels, None


apply = ConvolutionFitting.apply
