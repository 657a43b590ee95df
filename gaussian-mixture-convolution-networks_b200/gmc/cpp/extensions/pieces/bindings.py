"""Matrix inverse and symmetric eigen-decomposition of 2x2 / 3x3 matrices as differentiable operators.

Counterpart of the reference's src/gmc/cpp/extensions/pieces/bindings.py:18-44 (`matrix_inverse_apply`,
`symeig_apply`). The eigen-decomposition runs gmc_symeig of libgmc_b200.so; its backward is the standard eigh adjoint
`V (diag(gL) + (V^T gV - gV^T V) / 2 / E) V^T` with E_ij = L_j - L_i, which the reference also evaluates with tensor
operations (src/gmc/cpp/extensions/pieces/symeig.cu:23-108).
"""
import torch
import torch.autograd

from gmc import _native
from gmc.cpp.extensions.math import matrix_inverse as _matrix_inverse

matrix_inverse_apply = _matrix_inverse.apply


def symeig(matrices: torch.Tensor):
    if matrices.dim() < 2 or matrices.shape[-1] != matrices.shape[-2] or matrices.shape[-1] not in (2, 3):
        raise RuntimeError("symeig needs [..., 2, 2] or [..., 3, 3] input")
    _native.require_cuda_f32(matrices, "matrices")
    d = matrices.shape[-1]
    n = matrices.numel() // (d * d)
    values = torch.empty(matrices.shape[:-1], dtype=torch.float32, device=matrices.device)
    vectors = torch.empty_like(matrices)
    with torch.cuda.device_of(matrices):
        _native.check(_native.lib.gmc_symeig(_native.ptr(matrices), _native.ptr(values), _native.ptr(vectors), n, d,
                                             _native.stream_of(matrices)), "symeig")
    return values, vectors


def symeig_backward(matrices, eigvals, eigvecs, grad_eigvals, grad_eigvecs):
    vh = eigvecs.transpose(-2, -1)
    if grad_eigvecs is None:
        if grad_eigvals is None:
            return torch.zeros_like(matrices)
        return (eigvecs * grad_eigvals.unsqueeze(-2)) @ vh
    e = eigvals.unsqueeze(-2) - eigvals.unsqueeze(-1)
    e = e + torch.eye(e.shape[-1], dtype=e.dtype, device=e.device)      # any non-zero value: the diagonal is replaced
    inner = vh @ grad_eigvecs
    inner = (inner - inner.transpose(-2, -1)) * 0.5 / e
    diag = grad_eigvals if grad_eigvals is not None else torch.zeros_like(eigvals)
    inner = inner - torch.diag_embed(torch.diagonal(inner, dim1=-2, dim2=-1)) + torch.diag_embed(diag)
    return eigvecs @ inner @ vh


class SymEig(torch.autograd.Function):
    @staticmethod
    def forward(ctx, matrices: torch.Tensor):
        matrices = matrices.contiguous()
        eigvals, eigvecs = symeig(matrices)
        ctx.save_for_backward(matrices, eigvals, eigvecs)
        return eigvals, eigvecs

    @staticmethod
    def backward(ctx, grad_eigvals, grad_eigvecs):
        matrices, eigvals, eigvecs = ctx.saved_tensors
        grad = symeig_backward(matrices, eigvals, eigvecs, grad_eigvals, grad_eigvecs)
        # degenerate spectra (for example the identity covariance of zero Gaussians) give NaN here while the incoming
        # gradient is zero; the reference zeroes those entries as well
        return torch.where(torch.isnan(grad), torch.zeros_like(grad), grad)


symeig_apply = SymEig.apply
