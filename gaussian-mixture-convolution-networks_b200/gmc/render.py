"""Headless 2D density images of mixtures: the mixture (plus constant) evaluated on a regular grid with the CUDA
evaluation kernel, returned as a tensor. Counterpart of the grid part of the reference's src/gmc/render.py:45-61;
colour mapping, matplotlib figures and the OpenGL 3D renderer of the reference are not part of this package."""
import typing

import torch
from torch import Tensor

import gmc.mixture as gm


def _grid(x_low, y_low, x_high, y_high, width, height, device) -> Tensor:
    xs = torch.linspace(x_low, x_high, width, device=device)
    ys = torch.linspace(y_low, y_high, height, device=device)
    gx, gy = torch.meshgrid(xs, ys, indexing="ij")
    return torch.stack((gx, gy), dim=-1).reshape(1, 1, -1, 2)


def render(mixture: Tensor, constant: Tensor, batches: typing.Tuple[int, int] = (0, None),
           layers: typing.Tuple[int, int] = (0, None), x_low: float = -22, y_low: float = -22, x_high: float = 22,
           y_high: float = 22, width: int = 100, height: int = 100) -> Tensor:
    """[n_batch, n_layers, width, height] values of mixture + constant on the grid (2D mixtures only)."""
    assert gm.n_dimensions(mixture) == 2
    m = mixture.detach()[batches[0]:batches[1], layers[0]:layers[1]]
    c = constant.detach()[batches[0]:batches[1], layers[0]:layers[1]]
    xes = _grid(x_low, y_low, x_high, y_high, width, height, m.device)
    values = gm.evaluate(m.contiguous(), xes) + c.unsqueeze(-1)
    return values.view(m.shape[0], m.shape[1], width, height)


def render_with_relu(mixture: Tensor, constant: Tensor, **kwargs) -> Tensor:
    return torch.clamp_min(render(mixture, constant, **kwargs), 0)
