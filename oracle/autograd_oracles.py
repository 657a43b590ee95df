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


# ---------------------------------------------------------------------------------------------
# BVH-MHEM fit
# ---------------------------------------------------------------------------------------------
_EPS_SMALL = 0.0000000000001
_EPS_LARGE = 0.0000001
_KL_THRESHOLD = 0.5


def _clip(v: torch.Tensor) -> torch.Tensor:
    """max(v, small) with the reference's gradient rule: the gradient passes only where v > small (util/epsilon.h:13-14)."""
    return torch.where(v > _EPS_SMALL, v, torch.full_like(v, _EPS_SMALL))


def _fit_em(target: torch.Tensor, initial_idx, R: int) -> torch.Tensor:
    """One hierarchical-EM step (implementation_forward.h:188-323) on `target` [n, V] (R < n <= 2R) with the initial
    representatives given; returns [R, V]. The KL gate is evaluated without gradient (it is a 0/1 matrix)."""
    n, RF = target.shape
    D = {7: 2, 13: 3}[RF]
    NT = 2 * R
    dt = target.dtype
    pad = torch.zeros(NT - n, RF, dtype=dt)
    pad[:, 1 + D:] = torch.eye(D, dtype=dt).reshape(-1)
    tgt = torch.cat((target, pad), 0)
    w, mu, cov = tgt[:, 0], tgt[:, 1:1 + D], tgt[:, 1 + D:].view(NT, D, D)
    Wc = _clip(w.sum())
    a = w / Wc
    idx = torch.as_tensor([int(i) for i in initial_idx], dtype=torch.int64)
    v = w[idx]
    b = v / _clip(v.sum())
    mu_i, cov_i = mu[idx], cov[idx]
    inv_i = torch.linalg.inv(cov_i)                                            # [R, D, D]
    diff = mu[:, None, :] - mu_i[None, :, :]                                   # [NT, R, D]
    maha = torch.einsum("tsi,sij,tsj->ts", diff, inv_i, diff)
    tr = torch.einsum("sij,tji->ts", inv_i, cov)
    factor = (2 * math.pi) ** (-0.5 * D)
    val_a = torch.sqrt(torch.linalg.det(inv_i))[None, :] * factor * torch.exp(-0.5 * maha)
    val_b = torch.exp(-0.5 * tr)
    lik = torch.pow(_clip(val_a * val_b), 4.0 * a[:, None])
    with torch.no_grad():
        lg = torch.log(torch.linalg.det(cov)[:, None] / torch.linalg.det(cov_i)[None, :])
        kl = 0.5 * (maha + tr - D - lg)
        same_sign = (a[:, None] >= 0) == (b[None, :] >= 0)
        kl = torch.where(same_sign, kl, torch.zeros_like(kl))
        gate = (kl < _KL_THRESHOLD).to(dt)
        gate[torch.arange(NT), kl.argmin(dim=1)] = 1.0
    x = _clip(b[None, :] * lik) * gate
    r1 = x / x.sum(1, keepdim=True)
    r2 = r1 * a[:, None]
    fw = r2.sum(0)
    r3 = r2 / _clip(fw)[None, :]
    pos = torch.einsum("ts,ti->si", r3, mu)
    d = mu[:, None, :] - pos[None, :, :]
    q = d[:, :, :, None] * d[:, :, None, :] + cov[:, None, :, :]
    c = torch.einsum("ts,tsij->sij", r3, q)
    degenerate = (fw < _EPS_LARGE)[:, None, None]
    c = torch.where(degenerate, torch.eye(D, dtype=dt).expand(R, D, D), c)
    return torch.cat(((fw * Wc)[:, None], pos, c.reshape(R, D * D)), 1)


def mhem_fit_given_decisions(mixture: torch.Tensor, nodes: np.ndarray, counts: np.ndarray, integrals: np.ndarray,
                             initial: np.ndarray, K: int, R: int) -> torch.Tensor:
    """Forward of the BVH-MHEM fit for ONE mixture [G, V] with the tree, the per-node Gaussian counts / integrals (for
    the selection) and the initial indices taken from the forward oracle; differentiable in `mixture`."""
    G, RF = mixture.shape
    D = {7: 2, 13: 3}[RF]
    n_internal = G - 1
    nodes = nodes.astype(np.int64)
    attr = {}

    def gaussians_of(node):
        if node >= n_internal:
            return mixture[nodes[node, 3]][None, :]
        return attr[node]

    # post-order over internal nodes
    order, stack = [], [0]
    while stack:
        node = stack.pop()
        if node >= n_internal:
            continue
        order.append(node)
        stack.extend((int(nodes[node, 1]), int(nodes[node, 2])))
    for node in reversed(order):
        child = torch.cat((gaussians_of(int(nodes[node, 1])), gaussians_of(int(nodes[node, 2]))), 0)
        keep = (child[:, 0].detach().abs() >= _EPS_LARGE).nonzero()[:, 0]
        child = child[keep]
        assert min(R, child.shape[0]) == counts[node], "count mismatch with the forward oracle"
        attr[node] = _fit_em(child, initial[node], R) if child.shape[0] > R else child

    def rating(node):
        return -2.0 if counts[node] < R else abs(float(integrals[node]))

    selected, ratings = [0], [rating(0)]
    n_selected = int(counts[0])
    while n_selected < K - R:
        best, best_rating = -1, -1.0
        for i, r in enumerate(ratings):
            if r > best_rating:
                best, best_rating = i, r
        if best < 0:
            break
        node = selected[best]
        l, r = int(nodes[node, 1]), int(nodes[node, 2])
        selected[best], ratings[best] = l, rating(l)
        selected.append(r)
        ratings.append(rating(r))
        n_selected = n_selected - R + int(counts[l]) + int(counts[r])
    rows = [gaussians_of(node) for node in selected]
    out = torch.cat(rows, 0)
    pad = torch.zeros(K - out.shape[0], RF, dtype=mixture.dtype)
    pad[:, 1 + D:] = torch.eye(D, dtype=mixture.dtype).reshape(-1)
    return torch.cat((out, pad), 0)


def mhem_fit_backward(grad: np.ndarray, mixtures: np.ndarray, dump: dict, K: int, R: int):
    """fp64 gradient of sum(fit(mixture) * grad) for mixtures [n, G, V]; also returns the fp64 forward."""
    n = mixtures.shape[0]
    grads, outs = [], []
    for i in range(n):
        m = torch.from_numpy(np.asarray(mixtures[i], dtype=np.float64)).requires_grad_(True)
        out = mhem_fit_given_decisions(m, dump["nodes"][i], dump["counts"][i], dump["integrals"][i], dump["initial"][i], K, R)
        (out * torch.from_numpy(np.asarray(grad[i], dtype=np.float64))).sum().backward()
        grads.append(m.grad.numpy())
        outs.append(out.detach().numpy())
    return np.stack(grads), np.stack(outs)
