"""CPU: properties that pin the LBVH and BVH-MHEM oracles (oracle/cpu/lbvh.cpp, mhem_fit.cpp). The reference holds no
golden outputs for these stages, so the restatement is checked through invariants of the algorithm itself."""
import numpy as np

from oracle import cpu_oracle
import synthetic_inputs as synthetic


def _positive_mixture(B, L, G, seed, D=2):
    if D == 2:
        m = synthetic.fit_target_2d(B, L, G, seed).numpy()
    else:
        m = synthetic.config4_input(B * L, seed).numpy().reshape(B * L, 1, 64, 13)[:, :, :G]
    m = m.copy()
    m[..., 0] = np.abs(m[..., 0]) + 0.01
    return m.reshape(-1, m.shape[-2], m.shape[-1])


def test_expand_bits_known_answers():
    # Morton key of a 2x2 layout: component ids in the low 16 bits, x before y before z in the interleave
    m = np.zeros((1, 4, 7), dtype=np.float32)
    m[0, :, 1:3] = [[0, 0], [1, 0], [0, 1], [1, 1]]
    m[0, :, 3] = m[0, :, 6] = 1
    keys, nodes = cpu_oracle.lbvh_build(m)
    full = (1 << 30) - 1
    x_bits = sum(1 << (3 * i + 2) for i in range(10))
    y_bits = sum(1 << (3 * i + 1) for i in range(10))
    assert [int(k) >> 16 for k in keys[0]] == [0, y_bits, x_bits, x_bits | y_bits]
    assert [int(k) & 0xFFFF for k in keys[0]] == [0, 2, 1, 3]
    assert (x_bits | y_bits) < full            # z bits stay clear in 2D


def test_tree_topology_invariants():
    for D, G in ((2, 37), (2, 256), (3, 64)):
        m = _positive_mixture(3, 2, G, 11, D)
        keys, nodes = cpu_oracle.lbvh_build(m)
        n = m.shape[0]
        assert (np.diff(keys.astype(np.int64), axis=1) > 0).all()          # strictly ascending, unique
        for i in range(n):
            nd = nodes[i].astype(np.int64)
            assert nd[0, 0] == 0xFFFF
            assert sorted(nd[G - 1:, 3].tolist()) == list(range(G))         # leaves are a permutation of the ids
            assert (nd[G - 1:, 3] == (keys[i] & 0xFFFF).astype(np.int64)).all()
            children = np.concatenate((nd[:G - 1, 1], nd[:G - 1, 2]))
            assert sorted(children.tolist()) == list(range(1, 2 * G - 1))   # every node but the root has one parent
            for node in range(G - 1):
                assert nd[nd[node, 1], 0] == node and nd[nd[node, 2], 0] == node


def test_fit_preserves_integral_and_reproduces_input_when_k_is_large():
    for D, R in ((2, 4), (2, 2), (3, 4)):
        m = _positive_mixture(2, 2, 64, 3, D)
        G = m.shape[1]
        fit = cpu_oracle.mhem_fit_forward(m, 16, R)
        assert np.isfinite(fit).all()
        np.testing.assert_allclose(fit[..., 0].sum(1), m[..., 0].sum(1), rtol=1e-4)
        big = cpu_oracle.mhem_fit_forward(m, G + R, R)
        for i in range(m.shape[0]):
            a = big[i][big[i][:, 0] != 0]
            assert a.shape[0] == G
            sa = a[np.lexsort(a.T[::-1])]
            sb = m[i][np.lexsort(m[i].T[::-1])]
            assert np.array_equal(sa, sb)


def test_fit_density_improves_with_k():
    m = _positive_mixture(2, 2, 128, 5)
    errs = [cpu_oracle.density_rel_l2(cpu_oracle.mhem_fit_forward(m, K, 4), m, m).mean() for K in (8, 32, 128)]
    assert errs[0] > errs[1] > errs[2]
    assert errs[2] < 0.35


def test_fit_node_rules():
    m = _positive_mixture(1, 2, 64, 9)
    fit, dump = cpu_oracle.mhem_fit_forward(m, 16, 4, dump=True)
    G = 64
    for i in range(m.shape[0]):
        nd, cnt, integ = dump["nodes"][i].astype(np.int64), dump["counts"][i], dump["integrals"][i]
        assert (cnt[G - 1:] == 1).all()
        for node in range(G - 1):
            l, r = nd[node, 1], nd[node, 2]
            assert cnt[node] == min(4, cnt[l] + cnt[r])
            assert integ[node] == np.float32(integ[l] + integ[r])
        # a fitted node keeps the integral of its children (all weights positive)
        g = dump["gaussians"][i]
        full = np.where(cnt[:G - 1] == 4)[0]
        np.testing.assert_allclose(g[full][..., 0].sum(-1), integ[full], rtol=2e-4)
        init = dump["initial"][i]
        fitted = [n for n in full if cnt[nd[n, 1]] + cnt[nd[n, 2]] > 4]
        assert all(len(set(init[n].tolist())) == 4 and init[n].max() < 8 for n in fitted)
