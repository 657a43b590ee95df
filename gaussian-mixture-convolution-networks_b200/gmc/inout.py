"""Mixtures on disk: the versioned torch dictionary of the reference and its ASCII PLY layout for 3D mixtures.

Counterpart of the reference's src/gmc/inout.py:12-141 (same dictionary keys and versions, same PLY properties), so
files written by either implementation load in the other.
"""
import os
import typing

import numpy as np
import torch
from torch import Tensor

import gmc.mixture as gm
import gmc.config as config

_PLY_PROPERTIES = ("x", "y", "z", "covxx", "covxy", "covxz", "covyy", "covyz", "covzz", "weight")


def save(mixture: Tensor, file_name: str, meta_info=None) -> None:
    """Writes {"type": "gm.Mixture", "version": 6, "data", "meta_info"} below config.data_base_path."""
    assert gm.is_valid_mixture(mixture)
    torch.save({"type": "gm.Mixture", "version": 6, "data": mixture.detach().cpu(), "meta_info": meta_info},
               config.data_base_path / file_name)


def load(file_name: str) -> typing.Tuple[Tensor, typing.Any]:
    """Reads versions 3..6; versions below 6 stored amplitudes and are converted to integral weights."""
    d = torch.load(config.data_base_path / file_name)
    assert d["type"] == "gm.Mixture"
    version = d["version"]
    if version == 3:
        w, p, c = d["weights"], d["positions"], d["covariances"]
        n, dims = w.shape[1], p.shape[2]
        mixture = gm.pack_mixture(w.view(-1, 1, n), p.view(-1, 1, n, dims), c.view(-1, 1, n, dims, dims))
        mixture = gm.convert_amplitudes_to_priors(mixture)
    elif version == 4:
        mixture = gm.convert_amplitudes_to_priors(gm.pack_mixture(d["weights"], d["positions"], d["covariances"]))
    elif version == 5:
        mixture = gm.convert_amplitudes_to_priors(d["data"])
    else:
        assert version == 6
        mixture = d["data"]
    assert gm.is_valid_mixture(mixture)
    return mixture, d["meta_info"]


def write_gm_to_ply(m_weights: Tensor, m_positions: Tensor, m_covariances: Tensor, index: int, filename: str):
    """One 3D mixture (batch element `index`, single layer) as an ASCII PLY with one "component" element per Gaussian."""
    assert m_weights.dim() == 3 and m_positions.dim() == 4 and m_covariances.dim() == 5
    assert m_weights.shape[1] == m_positions.shape[1] == m_covariances.shape[1] == 1
    assert m_positions.shape[3] == 3 and m_covariances.shape[3:] == (3, 3)
    n = m_weights.shape[2]
    cov = m_covariances[index, 0].detach().cpu().reshape(n, 3, 3)
    rows = torch.cat((m_positions[index, 0].detach().cpu().reshape(n, 3),
                      torch.stack((cov[:, 0, 0], cov[:, 0, 1], cov[:, 0, 2], cov[:, 1, 1], cov[:, 1, 2], cov[:, 2, 2]), 1),
                      m_weights[index, 0].detach().cpu().reshape(n, 1)), dim=1)
    folder = os.path.dirname(filename)
    if folder and not os.path.exists(folder):
        os.makedirs(folder)
    with open(filename, "w") as f:
        f.write("ply\nformat ascii 1.0\n")
        f.write(f"element component {n}\n")
        for name in _PLY_PROPERTIES:
            f.write(f"property float {name}\n")
        f.write("end_header\n")
    with open(filename, "ab") as f:
        np.savetxt(f, rows.numpy(), delimiter="  ")


def write_gm_to_ply2(m: Tensor, path_without_ending: str):
    assert gm.n_dimensions(m) == 3
    for b in range(gm.n_batch(m)):
        for l in range(gm.n_layers(m)):
            t = m[b:b + 1, l:l + 1]
            write_gm_to_ply(gm.weights(t), gm.positions(t), gm.covariances(t), 0, f"{path_without_ending}_b{b}_l{l}.ply")


def read_gm_from_ply(filename: str, ismodel: bool = False, device='cuda') -> Tensor:
    """Reads a PLY written by write_gm_to_ply -> [1, 1, n, 13]. With ismodel the stored weights are priors that are
    normalised to sum one and converted to amplitudes; otherwise they are returned as stored."""
    n = None
    with open(filename) as f:
        header_lines = 0
        for line in f:
            header_lines += 1
            if line.startswith("element component "):
                n = int(line[len("element component "):])
            if line.startswith("end_header"):
                break
    assert n is not None
    rows = torch.from_numpy(np.loadtxt(filename, skiprows=header_lines, ndmin=2).astype(np.float32))
    assert rows.shape == (n, 10)
    pos = rows[:, 0:3].reshape(1, 1, n, 3)
    cxx, cxy, cxz, cyy, cyz, czz = (rows[:, i] for i in range(3, 9))
    cov = torch.stack((cxx, cxy, cxz, cxy, cyy, cyz, cxz, cyz, czz), dim=1).reshape(1, 1, n, 3, 3)
    w = rows[:, 9].reshape(1, 1, n)
    if ismodel:
        w = w / w.sum()
        w = w / (cov.det().sqrt() * 15.74960995)
    return gm.pack_mixture(w, pos, cov).to(device)
