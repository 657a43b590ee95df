"""CPU: pins the restated oracles (oracle/cpu/*, oracle/autograd_oracles.py) to the REFERENCE's own native code.

Two routes:
* tests/golden/reference_native.npz — outputs of the reference's native CPU path (built from the reference sources by
  oracle/build_ref.py, written by tests/golden/make_golden.py) on the inline mixtures and gradient sets of the
  reference's unit tests (src/gmc/cpp/extensions/unittests/support.h:228-1020) and on small seeded cases. Always runs.
* the reference library itself (oracle/_ref/libgmc_ref.so) at the benchmark shapes, when it has been built.

Bars: Morton keys, sort permutation, node arrays, subtree ranges bit-exact; fitted values 1e-6; the fp64 autograd
gradient oracles against the reference's hand-written fp32 backward 2e-5.
"""
import os

import numpy as np
import pytest
import torch

from conftest import ROOT, rel_inf
from oracle import autograd_oracles, cpu_oracle, ref_native
import synthetic_inputs as synthetic

GOLDEN = os.path.join(ROOT, "tests", "golden", "reference_native.npz")
FIELDS = lambda D: (("weight", slice(0, 1)), ("position", slice(1, 1 + D)), ("covariance", slice(1 + D, None)))  # noqa: E731


@pytest.fixture(scope="module")
def golden():
    return dict(np.load(GOLDEN))


@pytest.fixture(scope="module")
def reference_library():
    from oracle import build_ref
    if build_ref.reference_ext_dir() is not None:
        build_ref.build()
    if not ref_native.available():
        pytest.skip("oracle/_ref/libgmc_ref.so is not built (needs the reference checkout)")
    return ref_native


def test_golden_lbvh_and_fit_forward(golden):
    n = int(golden["n_mhem"])
    assert n >= 40
    worst = 0.0
    for i in range(n):
        key = f"mhem{i:03d}"
        m = golden[key + "_mixture"]
        K, R = (int(v) for v in golden[key + "_kr"])
        G, V = m.shape[-2:]
        flat = m.reshape(-1, G, V)
        keys, nodes = cpu_oracle.lbvh_build(flat)
        assert np.array_equal(keys, golden[key + "_keys"]), f"{key}: Morton keys / sort permutation"
        assert np.array_equal(nodes, golden[key + "_nodes"]), f"{key}: node arrays"
        fit, dump = cpu_oracle.mhem_fit_forward(flat, K, R, dump=True)
        assert np.array_equal(dump["counts"], golden[key + "_counts"]), f"{key}: Gaussians per node"
        err = rel_inf(fit, golden[key + "_fitting"])
        worst = max(worst, err)
        assert err <= 1e-6, f"{key} ({golden[key + '_source']}): fitting rel {err:.2e}"
    print(f"fit forward oracle vs reference native: worst rel {worst:.2e} over {n} cases")


def test_golden_fit_backward(golden):
    n = int(golden["n_mhem"])
    worst = 0.0
    for i in range(n):
        key = f"mhem{i:03d}"
        m = golden[key + "_mixture"]
        K, R = (int(v) for v in golden[key + "_kr"])
        G, V = m.shape[-2:]
        D = {7: 2, 13: 3}[V]
        flat = m.reshape(-1, G, V)
        _, dump = cpu_oracle.mhem_fit_forward(flat, K, R, dump=True)
        grad64, _ = autograd_oracles.mhem_fit_backward(golden[key + "_grad"].reshape(-1, K, V), flat, dump, K, R)
        ref = golden[key + "_grad_target"]
        scale = max(np.abs(ref).max(), 1e-30)
        for field, sl in FIELDS(D):
            err = float(np.abs(grad64[..., sl] - ref[..., sl]).max() / scale)
            worst = max(worst, err)
            assert err <= 2e-5, f"{key} ({golden[key + '_source']}) {field}: rel {err:.2e}"
    print(f"fit backward autograd oracle vs reference native: worst rel {worst:.2e}")


def test_golden_convolution_fitting(golden):
    for i in range(int(golden["n_cf"])):
        key = f"cf{i}"
        data, kernels, K = golden[key + "_data"], golden[key + "_kernels"], int(golden[key + "_k"])
        D = {7: 2, 13: 3}[data.shape[-1]]
        out, cached, objs, sub, keys = cpu_oracle.convolution_fitting_forward(data, kernels, K, with_keys=True)
        assert np.array_equal(keys, golden[key + "_keys"]), f"{key}: keys"
        assert np.array_equal(objs, golden[key + "_nodesobjs"]), f"{key}: nodesobjs"
        assert np.array_equal(sub, golden[key + "_subtrees"]), f"{key}: fitting_subtrees"
        assert rel_inf(out, golden[key + "_fitting"]) <= 1e-6
        assert rel_inf(cached, golden[key + "_cached"]) <= 1e-5
        gd, gk, _ = autograd_oracles.convolution_fitting_backward(golden[key + "_grad"], data, kernels, objs, sub)
        for name, a, r in (("grad_data", gd, golden[key + "_grad_data"]), ("grad_kernels", gk, golden[key + "_grad_kernels"])):
            scale = max(np.abs(r).max(), 1e-30)
            for field, sl in FIELDS(D):
                err = float(np.abs(a[..., sl] - r[..., sl]).max() / scale)
                assert err <= 2e-5, f"{key} {name} {field}: rel {err:.2e}"


def _positive(m):
    m = m.copy()
    m[..., 0] = np.abs(m[..., 0]) + 1e-3
    return m


@pytest.mark.parametrize("D,G,K,R,n", [(2, 1024, 64, 4, 6), (2, 257, 32, 2, 4), (3, 64, 16, 4, 8), (3, 333, 32, 4, 3)])
def test_library_fit_forward_at_benchmark_shapes(reference_library, D, G, K, R, n):
    """oracle/cpu == reference library on the config-2 shape (2D, 1024 -> 64, R=4) and 3D shapes."""
    if D == 2:
        m = _positive(synthetic.fit_target_2d(1, n, G, 1002).numpy())
    else:
        reps = (G + 63) // 64
        base = synthetic.config4_input(n * reps, 1004).numpy().reshape(1, n, reps * 64, 13)[:, :, :G]
        m = np.ascontiguousarray(base)
    V = m.shape[-1]
    keys_r, nodes_r = reference_library.lbvh_build(m)
    keys_o, nodes_o = cpu_oracle.lbvh_build(m.reshape(-1, G, V))
    assert np.array_equal(keys_o, keys_r) and np.array_equal(nodes_o, nodes_r)
    fit_r, dump_r = reference_library.mhem_fit_forward(m, K, R, dump=True)
    fit_o, dump_o = cpu_oracle.mhem_fit_forward(m.reshape(-1, G, V), K, R, dump=True)
    assert np.array_equal(dump_o["counts"], dump_r["counts"])
    fitted = dump_o["counts"][:, :G - 1] == R
    assert np.array_equal(dump_o["initial"][:, :G - 1][fitted & _was_fitted(dump_o, G, R)],
                          dump_r["initial"][:, :G - 1][fitted & _was_fitted(dump_o, G, R)])
    assert rel_inf(dump_o["gaussians"], dump_r["gaussians"]) <= 1e-6
    assert rel_inf(dump_o["integrals"], dump_r["integrals"]) <= 1e-6
    assert rel_inf(fit_o, fit_r) <= 1e-6


def _was_fitted(dump, G, R):
    nd = dump["nodes"].astype(np.int64)
    cnt = dump["counts"]
    left = np.take_along_axis(cnt, nd[:, :G - 1, 1], axis=1)
    right = np.take_along_axis(cnt, nd[:, :G - 1, 2], axis=1)
    return (left + right) > R


def _kernels(Cout, Cin, Gk, D, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(Cout, Cin, Gk, generator=g) * 0.3
    p = torch.randn(Cout, Cin, Gk, D, generator=g) * 0.1
    cov, _ = synthetic.covariances_and_inverses((Cout, Cin, Gk), D, 0.02, 0.1, g)
    return synthetic.pack(w, p, cov).numpy()


# config 3 and the four layer shapes of config 4 (Cout reduced: trees of different output channels are independent)
@pytest.mark.parametrize("D,B,Cin,G,Cout,Gk,K", [(2, 2, 8, 128, 3, 5, 128), (3, 2, 1, 64, 4, 5, 64), (3, 2, 8, 64, 3, 5, 32),
                                                 (3, 2, 16, 32, 3, 5, 16), (3, 2, 32, 16, 3, 5, 8)])
def test_library_convolution_fitting_at_benchmark_shapes(reference_library, D, B, Cin, G, Cout, Gk, K):
    if D == 2:
        data = synthetic.fit_target_2d(B, Cin, G, 1003).numpy()
    else:
        data = np.ascontiguousarray(synthetic.config4_input(B * Cin, 1004).numpy().reshape(B, Cin, 64, 13)[:, :, :G])
        data[..., 0] *= np.where(np.arange(G) % 5 == 0, -1.0, 1.0)      # mixed signs, as after a convolution layer
    kernels = _kernels(Cout, Cin, Gk, D, 5 + Cin)
    out_o, cached_o, objs_o, sub_o, keys_o = cpu_oracle.convolution_fitting_forward(data, kernels, K, with_keys=True)

    def forward():
        out_r, cached_r, objs_r, sub_r, tree = reference_library.convolution_fitting_forward(data, kernels, K, tree=True)
        assert np.array_equal(keys_o, tree["keys"])
        assert np.array_equal(objs_o, objs_r) and np.array_equal(sub_o, sub_r)
        assert rel_inf(out_o, out_r) <= 1e-6 and rel_inf(cached_o, cached_r) <= 1e-5

    # serial: the reference's create_attributes adds a node's mass and its count with two independent atomics
    # (src/gmc/cpp/extensions/convolution_fitting/Tree.cu:289-294); with its CPU threads running concurrently a later
    # child can climb with a stale mass and the run selects other subtrees. One thread at a time is race-free.
    with reference_library.serial():
        forward()
    grad = np.random.default_rng(K).standard_normal(out_o.shape).astype(np.float32)
    gd_o, gk_o, _ = autograd_oracles.convolution_fitting_backward(grad, data, kernels, objs_o, sub_o)

    def backward():
        gd_r, gk_r = reference_library.convolution_fitting_backward(grad, data, kernels, K)
        for a, r in ((gd_o, gd_r), (gk_o, gk_r)):
            scale = max(np.abs(r).max(), 1e-30)
            for field, sl in FIELDS(D):
                assert float(np.abs(a[..., sl] - r[..., sl]).max() / scale) <= 2e-5, field

    with reference_library.serial():
        backward()


@pytest.mark.parametrize("D,G,K,R", [(2, 128, 32, 4), (3, 64, 16, 2)])
def test_library_fit_backward(reference_library, D, G, K, R):
    if D == 2:
        m = _positive(synthetic.fit_target_2d(1, 3, G, 77).numpy())
    else:
        m = np.ascontiguousarray(synthetic.config4_input(3, 78).numpy().reshape(1, 3, 64, 13)[:, :, :G])
    V = m.shape[-1]
    grad = np.random.default_rng(G).standard_normal((1, 3, K, V)).astype(np.float32)
    ref = reference_library.mhem_fit_backward(grad, m, K, R)
    _, dump = cpu_oracle.mhem_fit_forward(m.reshape(-1, G, V), K, R, dump=True)
    g64, _ = autograd_oracles.mhem_fit_backward(grad.reshape(-1, K, V), m.reshape(-1, G, V), dump, K, R)
    scale = max(np.abs(ref).max(), 1e-30)
    for field, sl in FIELDS(D):
        assert float(np.abs(g64[..., sl] - ref[..., sl]).max() / scale) <= 2e-5, field


def test_library_evaluation(reference_library):
    """The C restatement of the legacy evaluation against the reference's own CPU evaluation (fp32 and fp64)."""
    for cfg in (synthetic.config0(), synthetic.eval_config(2, 2, 40, 300, 3, 0.03, 0.25, 5, broadcast_xes=True)):
        m, x, g = (t.numpy() for t in cfg)
        assert rel_inf(cpu_oracle.eval_forward(m, x), reference_library.eval_forward(m, x)) <= 2e-6
        m64, x64 = m.astype(np.float64), x.astype(np.float64)
        assert rel_inf(cpu_oracle.eval_forward(m64, x64), reference_library.eval_forward(m64, x64)) <= 1e-13
        gm_o, gx_o = cpu_oracle.eval_backward(g, m, x)
        gm_r, gx_r = reference_library.eval_backward(g, m, x)
        assert rel_inf(gm_o, gm_r) <= 5e-6 and rel_inf(gx_o, gx_r) <= 5e-6


def test_golden_lbvh_options():
    """Key layouts 0..4 and make_aabbs of lbvh::Config: the oracle against tests/golden/reference_lbvh_options.npz
    (reference library outputs). Keys and nodes bit-exact; boxes by cpu_oracle.compare_lbvh_boxes (1e-3 of the extent for
    leaves with separated eigenvalues, exact union for internal nodes)."""
    gold = dict(np.load(os.path.join(ROOT, "tests", "golden", "reference_lbvh_options.npz")))
    n = int(gold["n_cases"])
    assert n >= 20
    worst = 0.0
    for i in range(n):
        key = f"lbvh{i:02d}"
        mi, algorithm, make_aabbs = (int(v) for v in gold[key + "_options"])
        m = gold[f"mixture{mi}"]
        out = cpu_oracle.lbvh_build_ex(m, algorithm, bool(make_aabbs), 0.001)
        assert np.array_equal(out[0], gold[key + "_keys"]), f"{key}: keys, layout {algorithm}"
        assert np.array_equal(out[1], gold[key + "_nodes"]), f"{key}: nodes, layout {algorithm}"
        if make_aabbs:
            worst = max(worst, cpu_oracle.compare_lbvh_boxes(m, out[1], out[2], gold[key + "_aabbs"], 0.001))
            # the reference's own boxes pass the same structural checks
            cpu_oracle.compare_lbvh_boxes(m, gold[key + "_nodes"], gold[key + "_aabbs"], gold[key + "_aabbs"], 0.001)
    print(f"lbvh boxes oracle vs reference native: worst {worst:.2e} of the extent")


def test_library_lbvh_options(reference_library):
    m = synthetic_inverse_mixture(3, 2, 3, 200, 77)
    for algorithm in range(5):
        a = cpu_oracle.lbvh_build_ex(m, algorithm)
        b = reference_library.lbvh_build(m, algorithm)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    a = cpu_oracle.lbvh_build_ex(m, 1, True, 0.01)
    b = reference_library.lbvh_build(m, 1, True, 0.01)
    assert np.array_equal(a[1], b[1])
    cpu_oracle.compare_lbvh_boxes(m, a[1], a[2], b[2], 0.01)


def synthetic_inverse_mixture(D, B, L, G, seed):
    import torch
    import synthetic_inputs as synthetic
    g = torch.Generator().manual_seed(seed)
    _, inv = synthetic.covariances_and_inverses((B, L, G), D, 0.05, 0.5, g)
    w = torch.rand(B, L, G, generator=g) * 2 - 1
    p = torch.rand(B, L, G, D, generator=g) * 2 - 1
    return synthetic.pack(w, p, inv).numpy()
