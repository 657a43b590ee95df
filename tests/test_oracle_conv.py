"""CPU: the convolution oracles against the golden products from the reference's gm.convolve, and the conv-fit oracle
against the exact convolution when every product gets its own output slot."""
import os

import numpy as np

from conftest import ROOT
from oracle import cpu_oracle


def _sorted_rows(a):
    return a[np.lexsort(a.T[::-1])]


def test_exact_convolution_oracle_matches_reference_products():
    golden = dict(np.load(os.path.join(ROOT, "tests", "golden", "convolve.npz")))
    for idx in (0, 1):
        data, kernels, ref = golden[f"conv{idx}_data"], golden[f"conv{idx}_kernels"], golden[f"conv{idx}_out"]
        out = cpu_oracle.convolution_forward(data, kernels)
        assert out.shape == ref.shape
        for b in range(out.shape[0]):
            for o in range(out.shape[1]):
                np.testing.assert_allclose(_sorted_rows(out[b, o]), _sorted_rows(ref[b, o]), rtol=1e-6, atol=1e-7)


def test_exact_convolution_oracle_index_order():
    # t = comp_in + G * (ch_in + Cin * comp_k)  (src/gmc/cpp/extensions/util/helper.h:9-24)
    data = np.zeros((1, 2, 3, 7), np.float32)
    kernels = np.zeros((1, 2, 2, 7), np.float32)
    data[0, :, :, 0] = [[1, 2, 3], [4, 5, 6]]
    kernels[0, :, :, 0] = [[10, 100], [1000, 10000]]
    out = cpu_oracle.convolution_forward(data, kernels)
    assert out[0, 0, :, 0].tolist() == [10, 20, 30, 4000, 5000, 6000, 100, 200, 300, 40000, 50000, 60000]


def test_convolution_fitting_oracle_k_equal_t_and_mass():
    golden = dict(np.load(os.path.join(ROOT, "tests", "golden", "convolve.npz")))
    for idx in (0, 1):
        data, kernels, ref = golden[f"conv{idx}_data"], golden[f"conv{idx}_kernels"], golden[f"conv{idx}_out"]
        T = ref.shape[2]
        out, cached, objs, sub = cpu_oracle.convolution_fitting_forward(data, kernels, T)
        for b in range(out.shape[0]):
            for o in range(out.shape[1]):
                np.testing.assert_allclose(_sorted_rows(out[b, o]), _sorted_rows(ref[b, o]), rtol=1e-5, atol=1e-6)
                assert sorted(objs[b, o].tolist()) == list(range(T))
        # fewer outputs: leaf ranges partition the leaves, the integral is preserved
        K = 6
        out, cached, objs, sub = cpu_oracle.convolution_fitting_forward(data, kernels, K)
        for b in range(out.shape[0]):
            for o in range(out.shape[1]):
                ranges = sorted((sub[b, o, 2 * k], sub[b, o, 2 * k + 1]) for k in range(K))
                assert ranges[0][0] == T - 1 and ranges[-1][1] == 2 * T - 1
                assert all(a[1] == c[0] for a, c in zip(ranges, ranges[1:]))
        np.testing.assert_allclose(out[..., 0].sum(-1), ref[..., 0].sum(-1), rtol=1e-4, atol=1e-5)
