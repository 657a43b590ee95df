"""TEST INFRASTRUCTURE, NOT PRODUCT CODE. Gradient oracles for the two fitting operators.

The reference's backward passes are hand-written reverse-mode derivatives of its own forward passes with the discrete
decisions of the forward (tree, selected subtrees, initial representatives, KL gate) held fixed:
  convolution_fitting  src/gmc/cpp/extensions/convolution_fitting/implementation_backward.h:22-159
                       (util/grad/welford.h:14-97 = derivative of the weighted mean / covariance sums)
  bvh_mhem_fit         src/gmc/cpp/extensions/bvh_mhem_fit/implementation_backward.h:41-305 (grad_em, the forward of
                       implementation_forward.h:188-323 walked back line by line), :307-519 (which nodes receive which
                       gradient)
Here the same forward formulas are restated in PyTorch fp64 on CPU, with the decisions taken from the forward
oracle, and torch.autograd walks them back. This is also the method of the reference's own unit tests, which compare
the analytic backward with numeric / automatic differentiation of the forward with a frozen tree
(unittests/convolution_fitting.cpp:20-119, unittests/bvh_mhem_fit_alpha_vs_ad.cpp).
"""
import math

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------
# convolution fitting
# ---------------------------------------------------------------------------------------------
def convolution_fitting_given_tree(data: torch.Tensor, kernels: torch.Tensor, nodesobjs: np.ndarray,
                                   subtrees: np.ndarray) -> torch.Tensor:
    """Forward of convolution_fitting with the tree frozen (implementation_forward.h:19-124):
    out[b, o, k] = (sum w, weighted mean of mu_d + mu_k, weighted mean of C_d + C_k + weighted scatter of the centres)
    over the leaves start..end-1 of output k."""
    B, Cin, G, RF = data.shape
    Cout, _, Gk, _ = kernels.shape
    D = {7: 2, 13: 3}[RF]
    T = Cin * G * Gk
    K = subtrees.shape[-1] // 2
    n_internal = T - 1
    out = []
    for b in range(B):
        for o in range(Cout):
            obj = torch.from_numpy(nodesobjs[b, o].astype(np.int64))
            comp_k = obj // (G * Cin)
            rem = obj - comp_k * (G * Cin)
            ch_in = rem // G
            comp_in = rem - ch_in * G
            dg = data[b, ch_in, comp_in]          # [T, RF] in sorted leaf order
            kg = kernels[o, ch_in, comp_k]
            w = dg[:, 0] * kg[:, 0]
            p = dg[:, 1:1 + D] + kg[:, 1:1 + D]
            C = (dg[:, 1 + D:] + kg[:, 1 + D:]).view(T, D, D)
            slot = torch.full((T,), K, dtype=torch.int64)
            for k in range(K):
                s, e = int(subtrees[b, o, 2 * k]), int(subtrees[b, o, 2 * k + 1])
                if s >= 0:
                    slot[s - n_internal:e - n_internal] = k
            W = torch.zeros(K + 1, dtype=data.dtype).index_add(0, slot, w)
            S1 = torch.zeros(K + 1, D, dtype=data.dtype).index_add(0, slot, w[:, None] * p)
            safe = torch.where(W != 0, W, torch.ones_like(W))
            mean = S1 / safe[:, None]
            diff = p - mean[slot]
            S2 = torch.zeros(K + 1, D, D, dtype=data.dtype).index_add(0, slot, w[:, None, None] * diff[:, :, None] * diff[:, None, :])
            S3 = torch.zeros(K + 1, D, D, dtype=data.dtype).index_add(0, slot, w[:, None, None] * C)
            eye = torch.eye(D, dtype=data.dtype)
            used = (W != 0)[:, None, None]
            cov = torch.where(used, (S2 + S3) / safe[:, None, None], eye.expand(K + 1, D, D))
            mean = torch.where((W != 0)[:, None], mean, torch.zeros_like(mean))
            out.append(torch.cat((W[:K, None], mean[:K], cov[:K].reshape(K, D * D)), dim=1))
    return torch.stack(out).view(B, Cout, K, RF)


def convolution_fitting_backward(grad: np.ndarray, data: np.ndarray, kernels: np.ndarray, nodesobjs: np.ndarray,
                                 subtrees: np.ndarray):
    """fp64 (grad_data, grad_kernels) of sum(out * grad) with the tree frozen."""
    d = torch.from_numpy(np.asarray(data, dtype=np.float64)).requires_grad_(True)
    k = torch.from_numpy(np.asarray(kernels, dtype=np.float64)).requires_grad_(True)
    out = convolution_fitting_given_tree(d, k, nodesobjs, subtrees)
    (out * torch.from_numpy(np.asarray(grad, dtype=np.float64))).sum().backward()
    return d.grad.numpy(), k.grad.numpy(), out.detach().numpy()
