"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

All tensors are generated on the CPU with a seeded torch.Generator (so a CPU checker and the GPU see the same
bits) and returned as fp32 CPU tensors. They stand in for the MNIST / ModelNet10 mixtures the reference trains
on, which are produced by its own pre-fitting scripts and are not redistributable with this package.
"""
import math

import torch


def _log_uniform(shape, lo, hi, g):
    return torch.exp(torch.rand(shape, generator=g) * (math.log(hi) - math.log(lo)) + math.log(lo))


def random_rotations(shape, n_dims, g):
    """2D: rotation by theta ~ U(0, pi). 3D: Haar-distributed rotation (QR of a normal matrix, sign fixed, det +1)."""
    if n_dims == 2:
        theta = torch.rand(shape, generator=g) * math.pi
        c, s = torch.cos(theta), torch.sin(theta)
        return torch.stack((torch.stack((c, -s), -1), torch.stack((s, c), -1)), -2)
    a = torch.randn(*shape, 3, 3, generator=g)
    q, r = torch.linalg.qr(a)
    q = q * torch.sign(torch.diagonal(r, dim1=-2, dim2=-1)).unsqueeze(-2)
    det = torch.linalg.det(q)
    q[..., :, 0] = q[..., :, 0] * det.unsqueeze(-1)
    return q


def covariances_and_inverses(shape, n_dims, s_lo, s_hi, g):
    """Sigma = Q diag(s^2) Q^T and its closed-form inverse Q diag(s^-2) Q^T (both symmetrised), s ~ logU(s_lo, s_hi)."""
    q = random_rotations(shape, n_dims, g)
    s = _log_uniform((*shape, n_dims), s_lo, s_hi, g)
    cov = q @ torch.diag_embed(s * s) @ q.transpose(-1, -2)
    inv = q @ torch.diag_embed(1.0 / (s * s)) @ q.transpose(-1, -2)
    cov = 0.5 * (cov + cov.transpose(-1, -2))
    inv = 0.5 * (inv + inv.transpose(-1, -2))
    return cov, inv


def pack(weights, positions, matrices):
    n_dims = positions.shape[-1]
    return torch.cat((weights.unsqueeze(-1), positions, matrices.reshape(*positions.shape[:-1], n_dims * n_dims)),
                     dim=-1).contiguous()


def eval_config(n_batch, n_layers, n_components, n_xes, n_dims, s_lo, s_hi, seed, broadcast_xes=False):
    """(mixture in inverse-covariance form, xes, grad_out) for an evaluate_inversed forward + backward."""
    g = torch.Generator().manual_seed(seed)
    shape = (n_batch, n_layers, n_components)
    w = torch.rand(shape, generator=g) * 2 - 1
    p = torch.rand(*shape, n_dims, generator=g) * 2 - 1
    _, inv = covariances_and_inverses(shape, n_dims, s_lo, s_hi, g)
    xs = (1, 1) if broadcast_xes else (n_batch, n_layers)
    xes = torch.rand(*xs, n_xes, n_dims, generator=g) * 2.4 - 1.2
    grad_out = torch.randn(n_batch, n_layers, n_xes, generator=g)
    return pack(w, p, inv), xes.contiguous(), grad_out.contiguous()


def config0(seed=1000):
    """2D evaluation, B=2, L=4, G=64, N=4096, s ~ logU(0.05, 0.3)."""
    return eval_config(2, 4, 64, 4096, 2, 0.05, 0.3, seed)


def config1(n_batch=32, seed=1001, broadcast_xes=False):
    """3D evaluation at scale, B=32 (or a batch slice), L=16, G=512, N=16384, s ~ logU(0.03, 0.25)."""
    return eval_config(n_batch, 16, 512, 16384, 3, 0.03, 0.25, seed, broadcast_xes)


def fit_target_2d(n_batch, n_layers, n_components, seed, s_lo=0.02, s_hi=0.2):
    """Covariance-form 2D mixture with weights ~ N(0,1), means ~ U(-1,1)^2 (the input of the ReLU fit)."""
    g = torch.Generator().manual_seed(seed)
    shape = (n_batch, n_layers, n_components)
    w = torch.randn(shape, generator=g)
    p = torch.rand(*shape, 2, generator=g) * 2 - 1
    cov, _ = covariances_and_inverses(shape, 2, s_lo, s_hi, g)
    return pack(w, p, cov)


def config2(n_batch=32, n_layers=32, seed=1002):
    """2D BVH-MHEM fit input: [B, 32, 1024, 7] and a zero constant."""
    return fit_target_2d(n_batch, n_layers, 1024, seed), torch.zeros(n_batch, n_layers)


def config3(n_batch=64, seed=1003):
    """2D convolution-fitting layer: data [B, 8, 128, 7], kernels [16, 8, 5, 7], K = 128."""
    data = fit_target_2d(n_batch, 8, 128, seed)
    g = torch.Generator().manual_seed(seed + 7919)
    shape = (16, 8, 5)
    w = torch.randn(shape, generator=g) * 0.1
    p = torch.randn(*shape, 2, generator=g) * 0.1
    cov, _ = covariances_and_inverses(shape, 2, 0.02, 0.1, g)
    return data, pack(w, p, cov), 128


def config4_input(n_batch=256, seed=1004):
    """3D network input: [B, 1, 64, 13], weights ~ U(0.2, 1), s ~ logU(0.03, 0.15)."""
    g = torch.Generator().manual_seed(seed)
    shape = (n_batch, 1, 64)
    w = torch.rand(shape, generator=g) * 0.8 + 0.2
    p = torch.rand(*shape, 3, generator=g) * 2 - 1
    cov, _ = covariances_and_inverses(shape, 3, 0.03, 0.15, g)
    return pack(w, p, cov)
