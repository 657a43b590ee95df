"""Generates the golden fixtures of this folder by running the REFERENCE's own Python on CPU.

Run where the reference checkout exists:   python tests/golden/make_golden.py
Inputs are seeded fp32 tensors; outputs come from the reference's gm.old_evaluate_inversed
(src/gmc/mixture.py:102-141, the ground truth of the reference's own src/gmc/test_cpp_eval.py) evaluated in
fp64 on the same values, with gradients from torch autograd through it.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_python  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def eval_cases(gm):
    cases = {}
    g = torch.Generator().manual_seed(1234)
    idx = 0
    # the reference's hand-made known-answer case (src/gmc/test_cpp_eval.py:25-28)
    specs = [("known", None)]
    for D in (2, 3):
        for (B, L, G, N, bx, lx) in ((1, 1, 1, 1, True, True), (2, 3, 6, 23, True, True), (2, 3, 17, 8, False, False),
                                     (3, 2, 50, 50, False, True), (2, 4, 64, 33, True, True)):
            specs.append((f"d{D}", (D, B, L, G, N, bx, lx)))
    for name, spec in specs:
        if spec is None:
            mixture = torch.tensor([1.0, 0.0, 0.0, 2.0, 0.0, 0.0, 2.0]).view(1, 1, 1, -1)
            xes = torch.zeros(1, 1, 1, 2)
        else:
            D, B, L, G, N, bx, lx = spec
            w = torch.rand(B, L, G, generator=g) * 2 - 1
            p = torch.rand(B, L, G, D, generator=g) * 20 - 10
            A = torch.rand(B, L, G, D, D, generator=g) * 2 - 1
            cov = (A @ A.transpose(-1, -2) + torch.eye(D) * 0.01) * 10
            mixture = gm.pack_mixture(w, p, cov.inverse().transpose(-2, -1)).contiguous()
            xes = torch.rand(B if bx else 1, L if lx else 1, N, D, generator=g) * 20 - 10
        m64 = mixture.double().requires_grad_(True)
        x64 = xes.double().requires_grad_(True)
        # the reference accumulates into an fp32 buffer (mixture.py:115); sum the fp64 slices directly instead
        out = gm.evaluate_componentwise_inversed(m64, x64).sum(-1)
        grad_out = torch.randn(out.shape, generator=g).float()
        (out * grad_out.double()).sum().backward()
        key = f"eval{idx:02d}_{name}"
        cases[key + "_mixture"] = mixture.numpy()
        cases[key + "_xes"] = xes.numpy()
        cases[key + "_grad_out"] = grad_out.numpy()
        cases[key + "_out"] = out.detach().numpy()
        cases[key + "_grad_mixture"] = m64.grad.numpy()
        cases[key + "_grad_xes"] = x64.grad.numpy()
        # the reference's fp32 function on the same inputs (cross-check of the fp64 route)
        cases[key + "_out_f32ref"] = gm.old_evaluate_inversed(mixture, xes).numpy()
        idx += 1
    return cases


def convolve_cases(gm):
    """Inputs and the reference's gm.convolve (src/gmc/mixture.py:243-274) per output channel.
    gm.convolve(data [B, Cin, G, V], kernels[o] [1, Cin, Gk, V]) -> [B, Cin, G*Gk, V] (pairs of one input channel)."""
    cases = {}
    g = torch.Generator().manual_seed(4321)
    for idx, (D, B, Cin, G, Cout, Gk) in enumerate(((2, 2, 3, 6, 2, 4), (3, 2, 2, 5, 3, 3))):
        def mixture(n0, n1, n2, pos, cov_scale, wscale):
            w = torch.randn(n0, n1, n2, generator=g) * wscale
            p = torch.randn(n0, n1, n2, D, generator=g) * pos
            A = torch.rand(n0, n1, n2, D, D, generator=g) * 2 - 1
            c = (A @ A.transpose(-1, -2) + torch.eye(D) * 0.05) * cov_scale
            return gm.pack_mixture(w, p, c).contiguous()
        data = mixture(B, Cin, G, 1.0, 0.05, 1.0)
        kernels = mixture(Cout, Cin, Gk, 0.1, 0.01, 0.1)
        per_channel = torch.stack([gm.convolve(data, kernels[o:o + 1]) for o in range(Cout)], dim=1)
        cases[f"conv{idx}_data"] = data.numpy()
        cases[f"conv{idx}_kernels"] = kernels.numpy()
        cases[f"conv{idx}_out"] = per_channel.reshape(B, Cout, Cin * G * Gk, -1).numpy()   # set of products per (b, o)
    return cases


def relu_fit_cases(gm, fitting):
    """Inputs and outputs of the reference's initial_approx_to_relu / fixed_point_iteration_to_relu
    (src/gmc/fitting.py:279-312), evaluated in fp64."""
    cases = {}
    g = torch.Generator().manual_seed(999)
    for idx, (D, B, L, G) in enumerate(((2, 2, 3, 12), (3, 2, 2, 9))):
        w = torch.randn(B, L, G, generator=g)
        p = torch.rand(B, L, G, D, generator=g) * 2 - 1
        A = torch.rand(B, L, G, D, D, generator=g) * 2 - 1
        c = (A @ A.transpose(-1, -2) + torch.eye(D) * 0.05) * 0.05
        mixture = gm.pack_mixture(w, p, c).contiguous()
        constant = torch.randn(B, L, generator=g) * 0.3
        m64, c64 = mixture.double(), constant.double()
        initial = fitting.initial_approx_to_relu(m64, c64)
        fp, ret_const = fitting.fixed_point_iteration_to_relu(m64, c64, initial)
        cases[f"relu{idx}_mixture"] = mixture.numpy()
        cases[f"relu{idx}_constant"] = constant.numpy()
        cases[f"relu{idx}_initial"] = initial.numpy()
        cases[f"relu{idx}_fixed_point"] = fp.numpy()
        cases[f"relu{idx}_ret_const"] = ret_const.numpy()
    return cases


def strategy_cases(gm, fitting):
    """Outputs of the reference's other ReLU-fit strategies (src/gmc/fitting.py:19-54 solver, :117-153
    fixed_point_and_max, :204-240 fixed_point_and_mhem with representative_select_for_relu / mhem_fit_a_to_b,
    :243-276 splitter), evaluated in fp64 on seeded inputs."""
    cases = {}
    g = torch.Generator().manual_seed(2024)
    for idx, (D, B, L, G, K) in enumerate(((2, 2, 2, 20, 8), (3, 2, 2, 12, 4))):
        w = torch.randn(B, L, G, generator=g)
        p = torch.rand(B, L, G, D, generator=g) * 2 - 1
        A = torch.rand(B, L, G, D, D, generator=g) * 2 - 1
        c = (A @ A.transpose(-1, -2) + torch.eye(D) * 0.05) * 0.05
        mixture = gm.pack_mixture(w, p, c).contiguous()
        constant = torch.randn(B, L, generator=g) * 0.3
        m64, c64 = mixture.double(), constant.double()
        cases[f"s{idx}_mixture"] = mixture.numpy()
        cases[f"s{idx}_constant"] = constant.numpy()
        cases[f"s{idx}_k"] = np.array(K)
        out, const, _ = fitting.fixed_point_and_max(m64, c64, K)
        cases[f"s{idx}_max"], cases[f"s{idx}_max_const"] = out.numpy(), const.numpy()
        out, const, steps = fitting.fixed_point_and_mhem(m64, c64, K)
        cases[f"s{idx}_mhem"], cases[f"s{idx}_mhem_selected"] = out.numpy(), steps[2].numpy()
        # the dense EM raises likelihoods to powers of about 20 |w|: the reference's own fp32 run differs from its
        # fp64 run by up to 6e-3, so the fp32 result is stored as well
        cases[f"s{idx}_mhem_f32"] = fitting.fixed_point_and_mhem(mixture, constant, K)[0].numpy()
        # the reference's solver adds the constant without a trailing axis (fitting.py:40): it only accepts [B, L, 1]
        out, const, _ = fitting.solver(m64, c64.unsqueeze(-1), K)
        cases[f"s{idx}_solver"] = out.numpy()
        positive = gm.pack_mixture(gm.weights(m64).abs() + 0.1, gm.positions(m64), gm.covariances(m64))
        cases[f"s{idx}_split"] = fitting.splitter(positive, [G + 3, G + 5]).numpy()
    return cases


def main():
    gm, fitting, mat_tools = ref_python.load()
    np.savez_compressed(os.path.join(HERE, "eval_inversed.npz"), **eval_cases(gm))
    print("wrote eval_inversed.npz")
    np.savez_compressed(os.path.join(HERE, "convolve.npz"), **convolve_cases(gm))
    print("wrote convolve.npz")
    # gm.evaluate inside the fixed-point iteration runs in fp64 through the reference's dense formulation
    gm.evaluate_inversed = lambda m, x: gm.evaluate_componentwise_inversed(m, x).sum(-1)
    np.savez_compressed(os.path.join(HERE, "relu_fit.npz"), **relu_fit_cases(gm, fitting))
    print("wrote relu_fit.npz")
    np.savez_compressed(os.path.join(HERE, "strategies.npz"), **strategy_cases(gm, fitting))
    print("wrote strategies.npz")


if __name__ == "__main__":
    main()
