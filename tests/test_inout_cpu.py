"""CPU: on-disk formats (versioned torch dictionary, PLY) and the host-side packing helpers of gmc.mixture."""
import math

import pytest
import torch


def _mixture3d(n=5):
    import gmc.mixture as gm
    torch.manual_seed(3)
    return gm.generate_random_mixtures(2, 1, n, 3, pos_radius=1, cov_radius=0.1)


def test_save_and_load_round_trip(tmp_path, monkeypatch):
    import gmc.config as config
    import gmc.inout as inout
    monkeypatch.setattr(config, "data_base_path", tmp_path)
    m = _mixture3d()
    inout.save(m, "a.torch", meta_info={"k": 1})
    loaded, meta = inout.load("a.torch")
    assert torch.equal(loaded, m) and meta == {"k": 1}
    # version 5 files hold amplitudes
    import gmc.mixture as gm
    torch.save({"type": "gm.Mixture", "version": 5, "data": gm.convert_priors_to_amplitudes(m), "meta_info": None},
               tmp_path / "b.torch")
    loaded5, _ = inout.load("b.torch")
    assert torch.allclose(loaded5, m, rtol=1e-5, atol=1e-7)


def test_ply_round_trip(tmp_path):
    import gmc.inout as inout
    import gmc.mixture as gm
    m = _mixture3d(7)[:1]
    path = str(tmp_path / "sub" / "m.ply")
    inout.write_gm_to_ply(gm.weights(m), gm.positions(m), gm.covariances(m), 0, path)
    text = open(path).read()
    assert text.startswith("ply\nformat ascii 1.0\nelement component 7\nproperty float x\n")
    back = inout.read_gm_from_ply(path, ismodel=False, device="cpu")
    assert back.shape == (1, 1, 7, 13)
    assert torch.allclose(back, m, rtol=1e-5, atol=1e-6)


def test_amplitude_prior_round_trip_and_spatial_scale():
    # properties of the reference's src/gmc/test_mixture.py:154-200
    import gmc.mixture as gm
    m = _mixture3d(6)
    assert torch.allclose(gm.convert_amplitudes_to_priors(gm.convert_priors_to_amplitudes(m)), m, rtol=1e-5, atol=1e-7)
    s = torch.tensor([[[2.0]], [[0.5]]]).expand(2, 1, 1)
    scaled = gm.spatial_scale(m, s)
    assert torch.equal(gm.weights(scaled), gm.weights(m))
    assert torch.allclose(gm.positions(scaled), gm.positions(m) * s.unsqueeze(-1))
    assert torch.allclose(gm.covariances(scaled), gm.covariances(m) * (s * s).unsqueeze(-1).unsqueeze(-1))
    # dense evaluation of the scaled mixture at scaled points = original density / s^D
    x = torch.rand(2, 1, 9, 3) * 2 - 1
    inv = lambda mm: gm.pack_mixture(gm.weights(mm), gm.positions(mm), torch.linalg.inv(gm.covariances(mm)))
    a = gm.old_evaluate_inversed(inv(m), x)
    b = gm.old_evaluate_inversed(inv(scaled), x * s.unsqueeze(-1))
    assert torch.allclose(b * (s ** 3), a, rtol=1e-4, atol=1e-6)


def test_polynomial_mul_repeat_known_answer():
    import gmc.mixture as gm
    A = torch.arange(2 * 1 * 3 * 1).view(2, 1, 3, 1)
    B = torch.arange(10, 10 + 2 * 1 * 2 * 1).view(2, 1, 2, 1)
    a, b = gm._polynomial_mul_repeat(A, B)
    assert a[0, 0, :, 0].tolist() == [0, 1, 2, 0, 1, 2]
    assert b[0, 0, :, 0].tolist() == [10, 10, 10, 11, 11, 11]


def test_mat_tools_index_helpers():
    import gmc.mat_tools as mat_tools
    a = torch.tensor([[[1, 1337], [2, 1337], [3, 1337]], [[4, 1337], [5, 1337], [6, 1337]], [[7, 1337], [8, 1337], [9, 1337]]])
    i = torch.tensor([[0, 1], [0, 2], [1, 2]])
    b = mat_tools.batched_index_select(a, 1, i)
    assert b[:, :, 0].tolist() == [[1, 2], [4, 6], [8, 9]]
    idx = torch.arange(3 * 5 * 7).view(3, 5, 7)
    coords = torch.tensor([[2, 4, 6], [1, 0, 3]])
    assert mat_tools.flatten_index(coords, idx.shape).tolist() == [idx[2, 4, 6].item(), idx[1, 0, 3].item()]
    assert math.isclose(mat_tools.trace(torch.eye(3).unsqueeze(0)).item(), 3.0)


def test_files_written_by_the_reference_load_here(monkeypatch):
    """tests/golden/inout/ holds a version-6 file written by the reference's inout.save, dictionaries in the older
    layouts (3, 4, 5: amplitudes) and a PLY written by the reference's write_gm_to_ply, with what the reference's own
    load / read_gm_from_ply return for them (src/gmc/inout.py:12-141)."""
    import os
    import pathlib
    import numpy as np
    import gmc.config as config
    import gmc.inout as inout
    folder = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "inout")
    expected = dict(np.load(os.path.join(folder, "expected.npz")))
    monkeypatch.setattr(config, "data_base_path", pathlib.Path(folder))
    for v in (3, 4, 5, 6):
        loaded, meta = inout.load(f"mixture_v{v}.torch")
        assert loaded.shape == (2, 1, 5, 13)
        assert np.allclose(loaded.numpy(), expected[f"v{v}"], rtol=1e-6, atol=1e-8), v
    assert inout.load("mixture_v6.torch")[1] == {"source": "reference inout.save", "n": 5}
    assert np.array_equal(inout.load("mixture_v6.torch")[0].numpy(), expected["mixture"])
    ply = os.path.join(folder, "mixture.ply")
    assert np.allclose(inout.read_gm_from_ply(ply, ismodel=False, device="cpu").numpy(), expected["ply_plain"], rtol=1e-6)
    assert np.allclose(inout.read_gm_from_ply(ply, ismodel=True, device="cpu").numpy(), expected["ply_model"], rtol=1e-5)


def test_ply_written_here_equals_the_reference_file(tmp_path):
    import os
    import numpy as np
    import gmc.inout as inout
    import gmc.mixture as gm
    folder = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "inout")
    m = torch.from_numpy(dict(np.load(os.path.join(folder, "expected.npz")))["mixture"])
    path = str(tmp_path / "mine.ply")
    inout.write_gm_to_ply(gm.weights(m), gm.positions(m), gm.covariances(m), 1, path)
    assert open(path).read() == open(os.path.join(folder, "mixture.ply")).read()
