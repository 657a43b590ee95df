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


def main():
    gm, fitting, mat_tools = ref_python.load()
    np.savez_compressed(os.path.join(HERE, "eval_inversed.npz"), **eval_cases(gm))
    print("wrote eval_inversed.npz")


if __name__ == "__main__":
    main()
