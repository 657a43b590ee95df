"""Small tensor helpers of the mixture library (counterpart of the reference's src/gmc/mat_tools.py:12-65)."""
import typing

import torch
from torch import Tensor

from .cpp.extensions.math import matrix_inverse as _matrix_inverse
from .cpp.extensions.pieces import bindings as _pieces


def batched_index_select(tensor: Tensor, dim: int, index: Tensor) -> Tensor:
    """Per-batch gather: out[b, ..., j, ...] = tensor[b, ..., index[b, j], ...] along `dim`."""
    shape = [-1 if i in (0, dim) else s for i, s in enumerate(tensor.shape)]
    for i in range(1, tensor.dim()):
        if i != dim:
            index = index.unsqueeze(i)
    return torch.gather(tensor, dim, index.expand(shape))


def my_index_select(tensor: Tensor, index: Tensor) -> Tensor:
    """Gather along the last axis of `index`; leading axes of extent one in `index` are broadcast."""
    dim = index.dim() - 1
    shape = [(-1 if index.shape[i] > 1 else tensor.shape[i]) if i < index.dim() else tensor.shape[i]
             for i in range(tensor.dim())]
    for i in range(index.dim(), tensor.dim()):
        index = index.unsqueeze(i)
    return torch.gather(tensor, dim, index.expand(shape))


def inverse(tensor: Tensor) -> Tensor:
    """Inverse of [..., 2, 2] / [..., 3, 3] matrices on the GPU (one thread per matrix)."""
    return _matrix_inverse.apply(tensor)


def symeig(tensor: Tensor):
    """Eigen-decomposition of symmetric 2x2 / 3x3 matrices -> (eigenvalues ascending, eigenvectors)."""
    return _pieces.symeig_apply(tensor)


def flatten_index(tensor: Tensor, shape: torch.Size) -> Tensor:
    """Row-major linear index of the coordinates in the last axis of `tensor` for an array of `shape`."""
    assert tensor.shape[-1] == len(shape)
    strides = []
    acc = 1
    for s in reversed(list(shape)):
        strides.append(acc)
        acc *= s
    strides = torch.tensor(list(reversed(strides)), dtype=torch.long, device=tensor.device)
    return (tensor * strides).sum(dim=-1)


def gen_random_positive_definite(dims: typing.List, epsilon: float = 0.01, device: torch.device = 'cpu') -> Tensor:
    assert dims[-1] == dims[-2]
    a = torch.rand(dims, dtype=torch.float32, device=device) * 2 - 1
    return a @ a.transpose(-1, -2) + torch.eye(dims[-1], dtype=torch.float32, device=device) * epsilon


def trace(matrices: Tensor) -> Tensor:
    return torch.diagonal(matrices, dim1=-2, dim2=-1).sum(-1)
