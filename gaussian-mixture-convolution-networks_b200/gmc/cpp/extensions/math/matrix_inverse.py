"""Batched 2x2 / 3x3 matrix inverse as a differentiable operator.

Same import path, class name and `apply` as the reference's src/gmc/cpp/extensions/math/matrix_inverse.py:14-36.
Forward runs gmc_matrix_inverse of libgmc_b200.so; backward is the reference's -A^-1 g A^-1 (transposes dropped
because the operator is meant for symmetric matrices, matrix_inverse.py:31-33) in gmc_matrix_inverse_backward.
"""
import torch
import torch.autograd

from gmc import _native


def forward(matrices: torch.Tensor) -> torch.Tensor:
    if matrices.dim() < 2 or matrices.shape[-1] != matrices.shape[-2] or matrices.shape[-1] not in (2, 3):
        raise RuntimeError("matrix inverse needs [..., 2, 2] or [..., 3, 3] input")
    _native.require_cuda_f32(matrices, "matrices")
    out = torch.empty_like(matrices)
    n_dims = matrices.shape[-1]
    n = matrices.numel() // (n_dims * n_dims)
    with torch.cuda.device_of(matrices):
        _native.check(_native.lib.gmc_matrix_inverse(_native.ptr(matrices), _native.ptr(out), n, n_dims,
                                                     _native.stream_of(matrices)), "matrix_inverse")
    return out


class MatrixInverse(torch.autograd.Function):
    @staticmethod
    def forward(ctx, matrices: torch.Tensor):
        if not matrices.is_contiguous():
            matrices = matrices.contiguous()
        output = forward(matrices)
        ctx.save_for_backward(output)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (matrices_inverse,) = ctx.saved_tensors
        if not grad_output.is_contiguous():
            grad_output = grad_output.contiguous()
        _native.require_cuda_f32(grad_output, "grad_output")
        out = torch.empty_like(matrices_inverse)
        n_dims = matrices_inverse.shape[-1]
        n = matrices_inverse.numel() // (n_dims * n_dims)
        with torch.cuda.device_of(matrices_inverse):
            _native.check(_native.lib.gmc_matrix_inverse_backward(
                _native.ptr(matrices_inverse), _native.ptr(grad_output), _native.ptr(out), n, n_dims,
                _native.stream_of(matrices_inverse)), "matrix_inverse backward")
        return out


apply = MatrixInverse.apply
