"""TEST INFRASTRUCTURE. ctypes access to oracle/_build/liboracle.so (built by oracle/build.py from oracle/cpu/)."""
import ctypes
import os

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.LIB_PATH
        if not os.path.exists(path):
            path = _build.build()
        _lib = ctypes.CDLL(path)
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def use_all_cores() -> int:
    """Makes the OpenMP loops of the oracle use every core this process may run on, whatever OMP_NUM_THREADS says."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().oracle_set_num_threads(ctypes.c_int(n))
    return num_threads()


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _eval_dims(mixture, xes):
    B, L, G, RF = mixture.shape
    D = {7: 2, 13: 3}[RF]
    Bx, Lx, N, Dx = xes.shape
    assert Dx == D and Bx in (1, B) and Lx in (1, L)
    return B, L, G, D, Bx, Lx, N


def eval_forward(mixture: np.ndarray, xes: np.ndarray) -> np.ndarray:
    """Restated evaluate_inversed forward; dtype of `mixture` (float32 or float64) selects the arithmetic."""
    dt = mixture.dtype
    assert dt in (np.float32, np.float64) and xes.dtype == dt
    mixture = np.ascontiguousarray(mixture)
    xes = np.ascontiguousarray(xes)
    dims = _eval_dims(mixture, xes)
    out = np.empty((dims[0], dims[1], dims[6]), dtype=dt)
    fn = lib().oracle_eval_forward_f32 if dt == np.float32 else lib().oracle_eval_forward_f64
    fn(_p(mixture), _p(xes), _p(out), *[ctypes.c_int(d) for d in dims])
    return out


def eval_backward(grad_out: np.ndarray, mixture: np.ndarray, xes: np.ndarray):
    """Restated evaluate_inversed backward -> (grad_mixture, grad_xes)."""
    dt = mixture.dtype
    assert dt in (np.float32, np.float64) and xes.dtype == dt and grad_out.dtype == dt
    mixture = np.ascontiguousarray(mixture)
    xes = np.ascontiguousarray(xes)
    grad_out = np.ascontiguousarray(grad_out)
    dims = _eval_dims(mixture, xes)
    gm = np.empty_like(mixture)
    gx = np.empty_like(xes)
    fn = lib().oracle_eval_backward_f32 if dt == np.float32 else lib().oracle_eval_backward_f64
    fn(_p(grad_out), _p(mixture), _p(xes), _p(gm), _p(gx), *[ctypes.c_int(d) for d in dims])
    return gm, gx


def _flat_mixtures(mixture: np.ndarray):
    mixture = np.ascontiguousarray(mixture, dtype=np.float32)
    RF = mixture.shape[-1]
    D = {7: 2, 13: 3}[RF]
    G = mixture.shape[-2]
    return mixture.reshape(-1, G, RF), G, D


def lbvh_build(mixture: np.ndarray):
    """Restated LBVH build over the means: mixture [..., G, 7|13] -> (sorted keys uint64 [n, G], nodes uint16 [n, 2G-1, 4])."""
    flat, G, D = _flat_mixtures(mixture)
    n = flat.shape[0]
    keys = np.empty((n, G), dtype=np.uint64)
    nodes = np.empty((n, 2 * G - 1, 4), dtype=np.uint16)
    lib().oracle_lbvh_build(_p(flat), ctypes.c_int(n), ctypes.c_int(G), ctypes.c_int(D), _p(keys), _p(nodes))
    return keys, nodes


def lbvh_build_ex(mixture: np.ndarray, algorithm: int = 0, make_aabbs: bool = False, aabb_threshold: float = 0.001):
    """LBVH build with the options of lbvh::Config -> (keys, nodes[, aabbs fp32 [n, 2G-1, 8]]). With make_aabbs the
    matrix slot of the mixture must hold inverse covariances."""
    flat, G, D = _flat_mixtures(mixture)
    n = flat.shape[0]
    keys = np.empty((n, G), dtype=np.uint64)
    nodes = np.empty((n, 2 * G - 1, 4), dtype=np.uint16)
    aabbs = np.empty((n, 2 * G - 1, 8), dtype=np.float32) if make_aabbs else None
    rc = lib().oracle_lbvh_build_ex(_p(flat), ctypes.c_int(n), ctypes.c_int(G), ctypes.c_int(D), ctypes.c_int(algorithm),
                                    ctypes.c_int(int(make_aabbs)), ctypes.c_float(aabb_threshold), _p(keys), _p(nodes), _p(aabbs))
    assert rc == 0
    return (keys, nodes, aabbs) if make_aabbs else (keys, nodes)


def compare_lbvh_boxes(mixture: np.ndarray, nodes: np.ndarray, boxes: np.ndarray, expected: np.ndarray, threshold: float,
                       tolerance: float = 1e-3, min_gap: float = 0.05):
    """Checks LBVH boxes `boxes` [n, 2G-1, 8] of inverse-covariance mixtures against `expected`.

    The reference's leaf half-extents delta[r]^2 = factor^2 * sum_k lambda_k v_r[k]^2 depend on the eigenVECTORS of the
    covariance, so two close eigenvalues make them a function of the rounding (any basis of the shared eigenspace is
    valid). Hence: (1) leaves whose eigenvalues are separated by more than min_gap (relative) agree within `tolerance`
    of the largest coordinate; (2) every leaf keeps 0 < delta^2 <= factor^2 lambda_max (the closed form's third
    vector is a cross product of two unit vectors, shorter than 1 when those are not orthogonal) and is centred on its mean; (3) every internal box is EXACTLY the union of its children's boxes. Returns the worst error of (1)."""
    flat, G, D = _flat_mixtures(mixture)
    n = flat.shape[0]
    nodes = nodes.reshape(n, 2 * G - 1, 4).astype(np.int64)
    boxes = boxes.reshape(n, 2 * G - 1, 8)
    expected = expected.reshape(n, 2 * G - 1, 8)
    scale = np.abs(expected).max()
    leaves = nodes[:, G - 1:, 3]                                          # component of every leaf
    comp = np.take_along_axis(flat, leaves[..., None], axis=1)            # [n, G, RF]
    cov = np.linalg.inv(comp[..., 1 + D:].reshape(n, G, D, D).astype(np.float64))
    lam = np.linalg.eigvalsh(0.5 * (cov + np.swapaxes(cov, -1, -2)))
    gap = (np.diff(lam, axis=-1) / lam[..., -1:]).min(-1)
    factor2 = np.maximum(-2.0 * np.log(threshold / np.abs(comp[..., 0].astype(np.float64))), 5.991464547107982)
    lb, le = boxes[:, G - 1:], expected[:, G - 1:]
    err = np.abs(lb - le).max(-1)
    well = gap > min_gap
    assert well.mean() > 0.5, "test mixtures must mostly have separated eigenvalues"
    worst = float(err[well].max() / scale)
    assert worst <= tolerance, f"leaf boxes off by {worst:.2e} of the extent"
    half = 0.5 * (lb[..., :D] - lb[..., 4:4 + D]).astype(np.float64)
    centre = 0.5 * (lb[..., :D] + lb[..., 4:4 + D]).astype(np.float64)
    assert np.abs(centre - comp[..., 1:1 + D]).max() <= 1e-5 * scale
    hi = factor2[..., None] * lam[..., -1:] * (1 + 1e-3)
    assert ((half > 0) & (half ** 2 <= hi)).all(), "leaf half-extents outside (0, lambda_max * factor^2]"
    assert (boxes[..., 3] == 0).all() and (boxes[..., 7] == 0).all() and (boxes[..., D:3] == 0).all()
    left = np.take_along_axis(boxes, nodes[:, :G - 1, 1:2], axis=1)
    right = np.take_along_axis(boxes, nodes[:, :G - 1, 2:3], axis=1)
    union = np.concatenate((np.maximum(left[..., :4], right[..., :4]), np.minimum(left[..., 4:], right[..., 4:])), -1)
    assert np.array_equal(boxes[:, :G - 1], union), "internal boxes are not the union of their children"
    return worst


def mhem_fit_forward(mixture: np.ndarray, K: int, R: int, nodes: np.ndarray = None, dump: bool = False):
    """Restated BVH-MHEM fit: mixture [..., G, V] (covariance form) -> fitting [n, K, V]
    (+ per-node Gaussians / counts / integrals / initial indices when dump=True)."""
    flat, G, D = _flat_mixtures(mixture)
    n = flat.shape[0]
    RF = flat.shape[-1]
    if nodes is None:
        _, nodes = lbvh_build(flat)
    nodes = np.ascontiguousarray(nodes.reshape(n, 2 * G - 1, 4), dtype=np.uint16)
    out = np.empty((n, K, RF), dtype=np.float32)
    ng = np.empty((n, 2 * G - 1, R, RF), dtype=np.float32) if dump else None
    nc = np.empty((n, 2 * G - 1), dtype=np.int32) if dump else None
    ni = np.empty((n, 2 * G - 1), dtype=np.float32) if dump else None
    nn = np.empty((n, 2 * G - 1, R), dtype=np.uint8) if dump else None
    rc = lib().oracle_mhem_fit_forward(_p(flat), ctypes.c_int(n), ctypes.c_int(G), ctypes.c_int(D), _p(nodes),
                                       ctypes.c_int(K), ctypes.c_int(R), _p(out), _p(ng), _p(nc), _p(ni), _p(nn))
    assert rc == 0
    if dump:
        return out, dict(gaussians=ng, counts=nc, integrals=ni, initial=nn, nodes=nodes)
    return out


def density_grid(mixtures: np.ndarray, lo: np.ndarray, hi: np.ndarray, res: int = 64) -> np.ndarray:
    """fp64 density of covariance-form mixtures [n, G, V] on a res^D grid spanning [lo, hi] per mixture -> [n, res^D]."""
    mixtures = np.asarray(mixtures, dtype=np.float64)
    n, G, RF = mixtures.shape
    D = {7: 2, 13: 3}[RF]
    cov = mixtures[..., 1 + D:].reshape(n, G, D, D)
    inv = np.linalg.inv(cov)
    inv = 0.5 * (inv + np.swapaxes(inv, -1, -2))
    packed = np.concatenate((mixtures[..., :1 + D], inv.reshape(n, G, D * D)), -1).reshape(n, 1, G, RF)
    axes = [np.linspace(0.0, 1.0, res) for _ in range(D)]
    unit = np.stack(np.meshgrid(*axes, indexing="ij"), -1).reshape(-1, D)
    xes = lo[:, None, :] + unit[None] * (hi - lo)[:, None, :]
    return eval_forward(np.ascontiguousarray(packed), np.ascontiguousarray(xes.reshape(n, 1, -1, D)))[:, 0]


def density_rel_l2(fit_a: np.ndarray, fit_b: np.ndarray, target: np.ndarray, res: int = 64) -> np.ndarray:
    """Relative L2 distance of the densities of two fitted mixtures per mixture, ||a - b|| / ||b||, on a res^D grid
    spanning [min mu - 3 sigma_max, max mu + 3 sigma_max] of the target mixture."""
    target = np.asarray(target, dtype=np.float64)
    n, G, RF = target.shape
    D = {7: 2, 13: 3}[RF]
    mu = target[..., 1:1 + D]
    cov = target[..., 1 + D:].reshape(n, G, D, D)
    sigma_max = np.sqrt(np.linalg.eigvalsh(cov).max(axis=(1, 2)))
    lo = mu.min(1) - 3 * sigma_max[:, None]
    hi = mu.max(1) + 3 * sigma_max[:, None]
    da = density_grid(fit_a, lo, hi, res)
    db = density_grid(fit_b, lo, hi, res)
    return np.linalg.norm(da - db, axis=1) / np.maximum(np.linalg.norm(db, axis=1), 1e-300)


def convolution_forward(data: np.ndarray, kernels: np.ndarray) -> np.ndarray:
    """Exact convolution of src/gmc/cpp/extensions/convolution/implementation_forward.h:60-100:
    out[b, o, t] = (w_d w_k, mu_d + mu_k, C_d + C_k), t = comp_in + G * (ch_in + Cin * comp_k)."""
    B, Cin, G, RF = data.shape
    Cout, Cin2, Gk, _ = kernels.shape
    assert Cin == Cin2
    d = data[:, None, None, :, :, :]            # [B, 1, 1(k), Cin, G, RF]
    k = kernels[None, :, :, :, :].transpose(0, 1, 3, 2, 4)[:, :, :, :, None, :]   # [1, Cout, Gk, Cin, 1, RF]
    out = d + k
    out[..., 0] = d[..., 0] * k[..., 0]
    return np.ascontiguousarray(out.reshape(B, Cout, Gk * Cin * G, RF))


def convolution_backward(grad: np.ndarray, data: np.ndarray, kernels: np.ndarray):
    """Gradient of convolution_forward (implementation_backward.h:64-118) -> (grad_data, grad_kernels)."""
    B, Cin, G, RF = data.shape
    Cout, _, Gk, _ = kernels.shape
    g = grad.reshape(B, Cout, Gk, Cin, G, RF).astype(np.float64)
    gd = g.sum(axis=(1, 2))                                   # [B, Cin, G, RF]
    gk = g.sum(axis=(0, 4)).transpose(0, 2, 1, 3)             # [Cout, Cin, Gk, RF]
    gd[..., 0] = (g[..., 0] * kernels.transpose(0, 2, 1, 3)[None, :, :, :, None, 0]).sum(axis=(1, 2))
    gk[..., 0] = (g[..., 0] * data[:, None, None, :, :, 0]).sum(axis=(0, 4)).transpose(0, 2, 1)
    return gd, gk


def convolution_fitting_forward(data: np.ndarray, kernels: np.ndarray, K: int, with_keys: bool = False):
    """Restated convolution_fitting forward -> (fitting [B, Cout, K, V], cached_pos_covs, nodesobjs, subtrees[, keys])."""
    data = np.ascontiguousarray(data, dtype=np.float32)
    kernels = np.ascontiguousarray(kernels, dtype=np.float32)
    B, Cin, G, RF = data.shape
    Cout, Cin2, Gk, _ = kernels.shape
    assert Cin == Cin2
    D = {7: 2, 13: 3}[RF]
    T = Cin * G * Gk
    out = np.empty((B, Cout, K, RF), dtype=np.float32)
    cached = np.empty((B, Cout, K, D * D), dtype=np.float32)
    nodesobjs = np.empty((B, Cout, T), dtype=np.int32)
    subtrees = np.empty((B, Cout, 2 * K), dtype=np.int32)
    keys = np.empty((B, Cout, T), dtype=np.uint64) if with_keys else None
    rc = lib().oracle_convolution_fitting_forward(_p(data), _p(kernels), *[ctypes.c_int(v) for v in (B, Cin, G, Cout, Gk, D, K)],
                                                  _p(out), _p(cached), _p(nodesobjs), _p(subtrees), _p(keys))
    assert rc == 0
    if with_keys:
        return out, cached, nodesobjs, subtrees, keys
    return out, cached, nodesobjs, subtrees
