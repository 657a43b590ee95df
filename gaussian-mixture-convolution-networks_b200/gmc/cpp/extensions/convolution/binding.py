"""Exact convolution of Gaussian mixtures as a differentiable operator.

Same import path and `apply(data, kernels)` as the reference's src/gmc/cpp/extensions/convolution/binding.py:21-44
(the reference names this class ConvolutionFitting as well); runs gmc_convolution_forward / _backward.
"""
import torch
import torch.autograd

from gmc import _native


def _dims(data: torch.Tensor, kernels: torch.Tensor):
    if data.dim() != 4 or kernels.dim() != 4 or data.shape[-1] not in (7, 13):
        raise RuntimeError("data and kernels must be [., ., ., 7 or 13]")
    if data.shape[-1] != kernels.shape[-1]:
        raise RuntimeError("number of dimensions of data and kernel must agree")
    if data.shape[1] != kernels.shape[1]:
        raise RuntimeError("number of input feature maps must agree with the second kernel dimension")
    if data.dtype != kernels.dtype:
        raise RuntimeError("kernel and data dtypes must agree")
    if data.device != kernels.device:
        raise RuntimeError("data and kernel devices must agree")
    n_dims = 2 if data.shape[-1] == 7 else 3
    return data.shape[0], data.shape[1], data.shape[2], kernels.shape[0], kernels.shape[2], n_dims


def forward(data: torch.Tensor, kernels: torch.Tensor) -> torch.Tensor:
    dims = _dims(data, kernels)
    _native.require_cuda_f32(data, "data")
    _native.require_cuda_f32(kernels, "kernels")
    n_batch, n_in, n_comp, n_out, n_kcomp, _ = dims
    out = torch.empty((n_batch, n_out, n_in * n_comp * n_kcomp, data.shape[-1]), dtype=torch.float32, device=data.device)
    with torch.cuda.device_of(data):
        _native.check(_native.lib.gmc_convolution_forward(_native.ptr(data), _native.ptr(kernels), _native.ptr(out),
                                                          *dims, _native.stream_of(data)), "convolution forward")
    return out


def backward(grad: torch.Tensor, data: torch.Tensor, kernels: torch.Tensor):
    dims = _dims(data, kernels)
    _native.require_cuda_f32(grad, "grad")
    grad_data = torch.empty_like(data)
    grad_kernels = torch.empty_like(kernels)
    with torch.cuda.device_of(data):
        _native.check(_native.lib.gmc_convolution_backward(_native.ptr(grad), _native.ptr(data), _native.ptr(kernels),
                                                           _native.ptr(grad_data), _native.ptr(grad_kernels), *dims,
                                                           _native.stream_of(data)), "convolution backward")
    return grad_data, grad_kernels


class ConvolutionFitting(torch.autograd.Function):
    @staticmethod
    def forward(ctx, data: torch.Tensor, kernels: torch.Tensor):
        data = data.contiguous()
        kernels = kernels.contiguous()
        result = forward(data, kernels)
        ctx.save_for_backward(data, kernels)
        return result

    @staticmethod
    def backward(ctx, grad_output):
        data, kernels = ctx.saved_tensors
        return backward(grad_output.contiguous(), data, kernels)


apply = ConvolutionFitting.apply
