"""GPU parity of the LBVH build (bit-exact keys / permutation / topology) and of the BVH-MHEM fit forward (node
level and relative L2 density error <= 1e-3 on a 64^D grid) against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from conftest import ROOT
from oracle import cpu_oracle
import synthetic_inputs as synthetic

pytestmark = pytest.mark.gpu


def _positive(m):
    m = m.clone()
    m[..., 0] = m[..., 0].abs() + 0.01
    return m


def _mixture(D, B, L, G, seed):
    if D == 2:
        return _positive(synthetic.fit_target_2d(B, L, G, seed))
    g = torch.Generator().manual_seed(seed)
    w = torch.rand(B, L, G, generator=g) * 0.8 + 0.2
    p = torch.rand(B, L, G, 3, generator=g) * 2 - 1
    cov, _ = synthetic.covariances_and_inverses((B, L, G), 3, 0.03, 0.15, g)
    return synthetic.pack(w, p, cov)


@pytest.mark.parametrize("D,G", [(2, 2), (2, 3), (2, 37), (2, 1024), (3, 64), (3, 500), (2, 5120)])
def test_lbvh_bit_exact(D, G):
    from gmc import lbvh
    m = _mixture(D, 3, 2, G, 100 + G)
    keys, nodes = lbvh.build(m.cuda())
    ref_keys, ref_nodes = cpu_oracle.lbvh_build(m.numpy())
    assert np.array_equal(keys.cpu().numpy().view(np.uint64).reshape(-1, G), ref_keys)
    assert np.array_equal(nodes.cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4), ref_nodes)
    keys2, nodes2 = lbvh.build(m.cuda())
    assert torch.equal(keys, keys2) and torch.equal(nodes, nodes2)      # deterministic


@pytest.mark.parametrize("D,G", [(2, 8193), (2, 20000), (3, 20000), (2, 32768)])
def test_lbvh_bit_exact_beyond_the_shared_memory_size(D, G):
    """More than 8192 components per mixture: the tree is built in global memory. Same keys, same nodes."""
    from gmc import lbvh
    m = _mixture(D, 2, 1, G, 300 + G)
    m[0, 0, 100:164, 1:1 + D] = m[0, 0, 99:100, 1:1 + D]          # equal Morton cells: the component id breaks the tie
    keys, nodes = lbvh.build(m.cuda())
    ref_keys, ref_nodes = cpu_oracle.lbvh_build(m.numpy())
    assert np.array_equal(keys.cpu().numpy().view(np.uint64).reshape(-1, G), ref_keys)
    assert np.array_equal(nodes.cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4), ref_nodes)
    with pytest.raises(RuntimeError):
        lbvh.build(_mixture(D, 1, 1, 32769, 1).cuda())


def _inverse_form_mixture(D, B, L, G, seed):
    g = torch.Generator().manual_seed(seed)
    _, inv = synthetic.covariances_and_inverses((B, L, G), D, 0.05, 0.5, g)
    w = torch.rand(B, L, G, generator=g) * 2 - 1
    w = torch.where(w.abs() < 0.05, torch.full_like(w, 0.05), w)
    p = torch.rand(B, L, G, D, generator=g) * 2 - 1
    return synthetic.pack(w, p, inv)


@pytest.mark.parametrize("D,G", [(2, 50), (3, 333), (2, 4000), (3, 9000)])
@pytest.mark.parametrize("algorithm", [0, 1, 2, 3, 4])
def test_lbvh_key_layouts_bit_exact(D, G, algorithm):
    """The covariance-aware key layouts of lbvh::Config::MortonCodeAlgorithm: keys and nodes bit-exact against the
    oracle (itself bit-exact against the reference library, tests/test_oracle_vs_reference.py), shared-memory and
    global-memory build."""
    from gmc import lbvh
    m = _inverse_form_mixture(D, 2, 2, G, 500 + G + algorithm)
    keys, nodes = lbvh.build(m.cuda(), morton_code_algorithm=algorithm)
    ref_keys, ref_nodes = cpu_oracle.lbvh_build_ex(m.numpy(), algorithm)
    assert np.array_equal(keys.cpu().numpy().view(np.uint64).reshape(-1, G), ref_keys)
    assert np.array_equal(nodes.cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4), ref_nodes)


@pytest.mark.parametrize("D,G,algorithm,threshold", [(2, 50, 0, 0.001), (3, 333, 1, 0.001), (3, 64, 0, 0.05), (2, 9000, 1, 0.01)])
def test_lbvh_boxes(D, G, algorithm, threshold):
    """make_aabbs: ellipsoid boxes of the leaves and their unions (lbvh/bvh.cu:164-231, 460-510), see
    cpu_oracle.compare_lbvh_boxes for the bars. Repeated launches give identical boxes."""
    from gmc import lbvh
    m = _inverse_form_mixture(D, 2, 3, G, 700 + G)
    keys, nodes, boxes = lbvh.build(m.cuda(), algorithm, True, threshold)
    ref_keys, ref_nodes, ref_boxes = cpu_oracle.lbvh_build_ex(m.numpy(), algorithm, True, threshold)
    assert np.array_equal(keys.cpu().numpy().view(np.uint64).reshape(-1, G), ref_keys)
    nodes_np = nodes.cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4)
    assert np.array_equal(nodes_np, ref_nodes)
    worst = cpu_oracle.compare_lbvh_boxes(m.numpy(), nodes_np, boxes.cpu().numpy(), ref_boxes, threshold)
    print(f"lbvh boxes D={D} G={G}: worst leaf error {worst:.2e} of the extent")
    _, _, again = lbvh.build(m.cuda(), algorithm, True, threshold)
    assert torch.equal(boxes, again)
    with pytest.raises(RuntimeError):
        lbvh.build(m.cuda(), 2, True, threshold)      # the leaf of layouts 2..4 does not name its component


def test_lbvh_boxes_against_reference_fixture():
    """The boxes of the reference library itself (tests/golden/reference_lbvh_options.npz)."""
    from gmc import lbvh
    gold = dict(np.load(os.path.join(ROOT, "tests", "golden", "reference_lbvh_options.npz")))
    checked = 0
    for i in range(int(gold["n_cases"])):
        key = f"lbvh{i:02d}"
        mi, algorithm, make_aabbs = (int(v) for v in gold[key + "_options"])
        m = gold[f"mixture{mi}"]
        G = m.shape[-2]
        out = lbvh.build(torch.from_numpy(m).cuda(), algorithm, bool(make_aabbs), 0.001)
        assert np.array_equal(out[0].cpu().numpy().view(np.uint64).reshape(-1, G), gold[key + "_keys"])
        nodes_np = out[1].cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4)
        assert np.array_equal(nodes_np, gold[key + "_nodes"])
        if make_aabbs:
            cpu_oracle.compare_lbvh_boxes(m, nodes_np, out[2].cpu().numpy(), gold[key + "_aabbs"], 0.001)
            checked += 1
    assert checked >= 8


@pytest.mark.parametrize("D,G,K,R", [(2, 20000, 64, 4), (3, 9000, 32, 2)])
def test_fit_of_large_mixtures_matches_oracle(D, G, K, R):
    """The reference plans for mixtures of 2 000 to 20 000 components
    (src/gmc/cpp/extensions/evaluate_inversed/parallel_implementation_optimised_backward.cu:121-125); above 8192 the
    fit keeps its per-node bookkeeping in global scratch. Forward against the oracle, backward against the reference
    library where it is present."""
    import gmc.cpp.extensions.bvh_mhem_fit.binding as fit
    from oracle import ref_native
    m = _mixture(D, 1, 2, G, 5 * G + K)
    RF = m.shape[-1]
    mt = m.cuda().requires_grad_(True)
    out = fit.apply(mt, K, R)
    fitting, nodes, attribs = fit.forward(m.cuda(), K, R)
    flat = m.numpy().reshape(-1, G, RF)
    ref, dump = cpu_oracle.mhem_fit_forward(flat, K, R, dump=True)
    assert np.array_equal(nodes.cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4), dump["nodes"])
    gaussians, integrals, counts, initial = _unpack_attrs(attribs, G, R, RF)
    assert np.array_equal(counts, dump["counts"][:, :G - 1])
    got = out.detach().cpu().numpy().reshape(-1, K, RF)
    np.testing.assert_allclose(got, ref, rtol=5e-3, atol=1e-5)
    err = cpu_oracle.density_rel_l2(got, ref, ref, res=64 if D == 2 else 24)
    assert err.max() <= 1e-3
    g = torch.randn(out.shape, generator=torch.Generator().manual_seed(2))
    out.backward(g.cuda())
    grad = mt.grad.cpu().numpy().reshape(-1, G, RF)
    assert np.isfinite(grad).all() and np.abs(grad).max() > 0
    if ref_native.available():
        gref = ref_native.mhem_fit_backward(g.numpy(), m.numpy(), K, R)
        scale = max(np.abs(gref).max(), 1e-30)
        assert float(np.abs(grad - gref).max() / scale) <= 1e-4


def test_lbvh_degenerate_axes_and_duplicate_positions():
    from gmc import lbvh
    m = _mixture(2, 1, 2, 33, 5)
    m[0, 0, :, 1] = 0.25          # zero extent in x
    m[0, 1, 5:9, 1:3] = m[0, 1, 4:5, 1:3]   # duplicate means: equal Morton cells, ids break the tie
    keys, nodes = lbvh.build(m.cuda())
    ref_keys, ref_nodes = cpu_oracle.lbvh_build(m.numpy())
    assert np.array_equal(keys.cpu().numpy().view(np.uint64).reshape(-1, 33), ref_keys)
    assert np.array_equal(nodes.cpu().numpy().view(np.uint16).reshape(-1, 65, 4), ref_nodes)


@pytest.mark.parametrize("D", [2, 3])
def test_lbvh_sort_with_crowded_cells(D):
    """The shared-memory build orders the keys by their top code bits first and fixes runs of equal top bits afterwards;
    runs longer than 64 fall back to full radix passes. Three mixtures: tight clusters (runs of 2..60 equal prefixes),
    200 identical means (fall-back path), all means identical."""
    from gmc import lbvh
    G = 700
    m = _mixture(D, 3, 1, G, 77)
    g = torch.Generator().manual_seed(5)
    centres = torch.rand(20, D, generator=g) * 2 - 1
    m[0, 0, :, 1:1 + D] = centres[torch.randint(0, 20, (G,), generator=g)] + torch.randn(G, D, generator=g) * 1e-4
    m[0, 0, :2, 1:1 + D] = torch.tensor([[-1.0] * D, [1.0] * D])          # keeps the box wide, the clusters narrow
    m[1, 0, 100:300, 1:1 + D] = m[1, 0, 99:100, 1:1 + D]
    m[2, 0, :, 1:1 + D] = m[2, 0, :1, 1:1 + D]
    keys, nodes = lbvh.build(m.cuda())
    ref_keys, ref_nodes = cpu_oracle.lbvh_build(m.numpy())
    assert np.array_equal(keys.cpu().numpy().view(np.uint64).reshape(-1, G), ref_keys)
    assert np.array_equal(nodes.cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4), ref_nodes)


def _unpack_attrs(attribs, G, R, RF):
    a = attribs.cpu().numpy().reshape(attribs.shape[0], G - 1, R * RF + 4)
    gaussians = a[..., :R * RF].reshape(a.shape[0], G - 1, R, RF)
    integrals = a[..., R * RF]
    counts = a[..., R * RF + 1].view(np.int32)
    initial = a[..., R * RF + 2].copy().view(np.uint8).reshape(a.shape[0], G - 1, 4)[..., :R]
    return gaussians, integrals, counts, initial


@pytest.mark.parametrize("D,G,K,R", [(2, 64, 16, 4), (2, 1024, 64, 4), (2, 100, 32, 2), (3, 64, 32, 4), (3, 333, 16, 2),
                                     (2, 8, 8, 4), (2, 2, 4, 4)])
def test_fit_forward_matches_oracle(D, G, K, R):
    import gmc.cpp.extensions.bvh_mhem_fit.binding as fit
    m = _mixture(D, 4, 3, G, 7 * G + K)
    RF = m.shape[-1]
    fitting, nodes, attribs = fit.forward(m.cuda(), K, R)
    flat = m.numpy().reshape(-1, G, RF)
    ref, dump = cpu_oracle.mhem_fit_forward(flat, K, R, dump=True)
    assert np.array_equal(nodes.cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4), dump["nodes"])
    gaussians, integrals, counts, initial = _unpack_attrs(attribs, G, R, RF)
    assert np.array_equal(counts, dump["counts"][:, :G - 1])
    np.testing.assert_allclose(integrals, dump["integrals"][:, :G - 1], rtol=1e-6, atol=1e-7)
    fitted = dump["initial"][:, :G - 1, 0] != 255
    assert np.array_equal(initial[fitted], dump["initial"][:, :G - 1][fitted])
    np.testing.assert_allclose(gaussians, dump["gaussians"][:, :G - 1], rtol=2e-3, atol=1e-5)
    out = fitting.cpu().numpy().reshape(-1, K, RF)
    assert np.isfinite(out).all()
    err = cpu_oracle.density_rel_l2(out, ref, flat)
    assert err.max() <= 1e-3, f"relative L2 density error {err.max():.3e}"
    # slots agree one to one as well (same selection order), and unused slots are (0, 0, I)
    np.testing.assert_allclose(out, ref, rtol=5e-3, atol=1e-5)


@pytest.mark.parametrize("D,R", [(2, 4), (3, 4), (2, 2)])
def test_fit_with_equal_centre_distances_follows_the_heap_order(D, R):
    """Centres on a regular grid (many exactly equal pair distances) and a repeated centre (distance 0): the order in
    which the reference's heap pops equal keys decides the clustering, so the kernel must leave its ranked fast path.
    (Ties between FITTED centres of higher levels are decided by rounding noise and are not a parity case.)"""
    import gmc.cpp.extensions.bvh_mhem_fit.binding as fit
    G, K = 64, 16
    m = _mixture(D, 2, 2, G, 900 + D + R)
    side = 8 if D == 2 else 4
    axes = [torch.arange(side, dtype=torch.float32) * 0.25 for _ in range(D)]
    grid = torch.stack(torch.meshgrid(*axes, indexing="ij"), -1).reshape(-1, D)
    m[0, 0, :, 1:1 + D] = grid[:G]
    m[0, 1, :, 1:1 + D] = grid[:G] * 0.5
    m[1, 0, 8:10, 1:1 + D] = m[1, 0, 8:9, 1:1 + D]          # two Gaussians on one centre
    RF = m.shape[-1]
    fitting, nodes, attribs = fit.forward(m.cuda(), K, R)
    flat = m.numpy().reshape(-1, G, RF)
    ref, dump = cpu_oracle.mhem_fit_forward(flat, K, R, dump=True)
    assert np.array_equal(nodes.cpu().numpy().view(np.uint16).reshape(-1, 2 * G - 1, 4), dump["nodes"])
    gaussians, integrals, counts, initial = _unpack_attrs(attribs, G, R, RF)
    assert np.array_equal(counts, dump["counts"][:, :G - 1])
    fitted = dump["initial"][:, :G - 1, 0] != 255
    assert np.array_equal(initial[fitted], dump["initial"][:, :G - 1][fitted])
    np.testing.assert_allclose(fitting.cpu().numpy().reshape(-1, K, RF), ref, rtol=5e-3, atol=1e-5)


def test_fit_large_k_returns_the_input_set():
    import gmc.cpp.extensions.bvh_mhem_fit.binding as fit
    G, R = 48, 4
    m = _mixture(2, 2, 2, G, 77)
    fitting, _, _ = fit.forward(m.cuda(), G + R, R)
    out = fitting.cpu().numpy().reshape(-1, G + R, 7)
    flat = m.numpy().reshape(-1, G, 7)
    for i in range(flat.shape[0]):
        a = out[i][out[i][:, 0] != 0]
        assert a.shape[0] == G
        assert np.array_equal(a[np.lexsort(a.T[::-1])], flat[i][np.lexsort(flat[i].T[::-1])])
        np.testing.assert_array_equal(out[i][G:], np.tile(np.array([0, 0, 0, 1, 0, 0, 1], np.float32), (R, 1)))


def test_fit_rejects_bad_arguments():
    import gmc.cpp.extensions.bvh_mhem_fit.binding as fit
    m = _mixture(2, 1, 1, 16, 1).cuda()
    with pytest.raises(RuntimeError):
        fit.forward(m, 10, 4)          # K not a multiple of R
    with pytest.raises(RuntimeError):
        fit.forward(m, 8, 3)           # unsupported R
    with pytest.raises(RuntimeError):
        fit.forward(m[:, :, :1], 4, 4)  # a single component


@pytest.mark.parametrize("D,G,K,R", [(2, 64, 16, 4), (2, 40, 12, 2), (3, 48, 16, 4), (3, 30, 8, 2), (2, 16, 20, 4), (2, 100, 8, 4)])
def test_fit_backward_matches_autograd_oracle(D, G, K, R):
    """Analytic CUDA backward against fp64 autograd through the restated forward with all discrete decisions frozen
    (that oracle agrees with the reference's hand-written fp32 backward to 4e-6: tests/test_oracle_vs_reference.py).
    Bar: relative 1e-4 of the gradient tensor's largest entry, per field; the measured error is printed."""
    import gmc.cpp.extensions.bvh_mhem_fit.binding as fit
    from conftest import rel_inf
    from oracle import autograd_oracles
    m = _mixture(D, 2, 2, G, 11 * G + K)
    RF = m.shape[-1]
    mt = m.cuda().requires_grad_(True)
    out = fit.apply(mt, K, R)
    g = torch.randn(out.shape, generator=torch.Generator().manual_seed(9))
    out.backward(g.cuda())
    grad_gpu = mt.grad.cpu().numpy().reshape(-1, G, RF)
    flat = m.numpy().reshape(-1, G, RF)
    ref_fit, dump = cpu_oracle.mhem_fit_forward(flat, K, R, dump=True)
    grad_ref, out64 = autograd_oracles.mhem_fit_backward(g.numpy().reshape(-1, K, RF), flat, dump, K, R)
    assert np.isfinite(grad_gpu).all()
    scale = max(np.abs(grad_ref).max(), 1e-30)
    for field, sl in (("weight", slice(0, 1)), ("position", slice(1, 1 + D)), ("covariance", slice(1 + D, None))):
        err = float(np.abs(grad_gpu[..., sl] - grad_ref[..., sl]).max() / scale)
        per_field = rel_inf(grad_gpu[..., sl], grad_ref[..., sl])
        print(f"fit backward D={D} G={G} K={K} R={R} {field}: rel(tensor) {err:.2e}, rel(field) {per_field:.2e}")
        assert err < 1e-4, f"{field}: rel {err:.2e}"
    # the saved tensors are not modified: a second backward gives the same gradient
    mt.grad = None
    out2 = fit.apply(mt, K, R)
    out2.backward(g.cuda())
    assert rel_inf(mt.grad.cpu().numpy().reshape(-1, G, RF), grad_gpu) < 1e-6
