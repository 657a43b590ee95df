"""TEST INFRASTRUCTURE. ctypes access to oracle/_ref/libgmc_ref.so: the REFERENCE's own native CPU code, compiled by
oracle/build_ref.py from the reference checkout (entry points: oracle/ref_entry.cu).  Array conventions match
oracle/cpu_oracle.py so the two can be compared call for call."""
import ctypes
import os

import numpy as np

from . import build_ref as _build

_libs = {}


def available() -> bool:
    return _build.available()


def _load(path):
    if path not in _libs:
        import torch  # noqa: F401  (the libraries link against libtorch; importing torch loads it)
        if not os.path.exists(path):
            raise FileNotFoundError(path + " is not built (run oracle/build_ref.py beside a reference checkout)")
        handle = ctypes.CDLL(path)          # RTLD_LOCAL: the two libraries do not see each other's symbols
        handle.gmc_ref_last_error.restype = ctypes.c_char_p
        _libs[path] = handle
    return _libs[path]


def lib():
    """LBVH, BVH-MHEM fit and evaluation (the reference's bvh_mhem_fit / evaluate_inversed extension sources)."""
    return _load(_build.LIB_FIT)


def lib_convfit():
    """Convolution fitting (the reference's convolution_fitting extension sources)."""
    return _load(_build.LIB_CONVFIT)


class serial:
    """Context manager: the reference's CPU threads run one after the other inside (race-free, reproducible). The
    reference's convolution_fitting mass pass is racy when its threads run concurrently
    (src/gmc/cpp/extensions/convolution_fitting/Tree.cu:289-294). Not for mhem_fit_backward (it waits on a CPU barrier)."""

    def __enter__(self):
        for handle in (lib(), lib_convfit()):
            handle.gmc_ref_set_serial(ctypes.c_int(1))
        return self

    def __exit__(self, *exc):
        for handle in (lib(), lib_convfit()):
            handle.gmc_ref_set_serial(ctypes.c_int(0))
        return False


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _check(rc, handle=None):
    if rc != 0:
        raise RuntimeError("reference raised: " + (handle or lib()).gmc_ref_last_error().decode(errors="replace"))


def _ints(*v):
    return [ctypes.c_int(int(x)) for x in v]


def _mix4(mixture):
    mixture = np.ascontiguousarray(mixture, dtype=np.float32)
    V = mixture.shape[-1]
    D = {7: 2, 13: 3}[V]
    if mixture.ndim == 3:
        mixture = mixture[:, None]
    B, L, G, _ = mixture.shape
    return mixture, B, L, G, D, V


def lbvh_build(mixture, algorithm: int = 0, make_aabbs: bool = False, aabb_threshold: float = 0.001):
    """lbvh::Bvh::construct -> (sorted keys uint64 [n, G], nodes uint16 [n, 2G-1, 4][, aabbs fp32 [n, 2G-1, 8]]).
    With make_aabbs the mixture must be in inverse-covariance form."""
    m, B, L, G, D, V = _mix4(mixture)
    n = B * L
    keys = np.empty((n, G), dtype=np.int64)
    nodes = np.empty((n, 2 * G - 1, 4), dtype=np.int16)
    aabbs = np.empty((n, 2 * G - 1, 8), dtype=np.float32) if make_aabbs else None
    _check(lib().gmc_ref_lbvh_build(_p(m), *_ints(B, L, G, D, algorithm, int(make_aabbs)), ctypes.c_float(aabb_threshold),
                                    _p(keys), _p(nodes), _p(aabbs)))
    out = (keys.view(np.uint64), nodes.view(np.uint16))
    return out + (aabbs,) if make_aabbs else out


def mhem_fit_forward(mixture, K: int, R: int, dump: bool = False, kl_threshold: float = 0.5):
    """bvh_mhem_fit::forward_impl_t -> fitting [n, K, V] (+ per-node dump like cpu_oracle.mhem_fit_forward)."""
    m, B, L, G, D, V = _mix4(mixture)
    n = B * L
    out = np.empty((n, K, V), dtype=np.float32)
    nodes = np.empty((n, 2 * G - 1, 4), dtype=np.int16)
    ng = np.empty((n, 2 * G - 1, R, V), dtype=np.float32) if dump else None
    nc = np.empty((n, 2 * G - 1), dtype=np.int32) if dump else None
    ni = np.empty((n, 2 * G - 1), dtype=np.float32) if dump else None
    nn = np.empty((n, 2 * G - 1, R), dtype=np.uint8) if dump else None
    nl = np.empty((n, 2 * G - 1), dtype=np.int32) if dump else None
    _check(lib().gmc_ref_mhem_fit_forward(_p(m), *_ints(B, L, G, D, K, R), ctypes.c_float(kl_threshold), _p(out), _p(nodes),
                                          _p(ng), _p(nc), _p(ni), _p(nn), _p(nl)))
    if dump:
        return out, dict(gaussians=ng, counts=nc, integrals=ni, initial=nn, child_leaves=nl, nodes=nodes.view(np.uint16))
    return out


def mhem_fit_backward(grad, mixture, K: int, R: int, kl_threshold: float = 0.5):
    """Reference forward followed by bvh_mhem_fit::backward_impl_t -> grad_target [n, G, V]."""
    m, B, L, G, D, V = _mix4(mixture)
    g = np.ascontiguousarray(grad, dtype=np.float32).reshape(B, L, K, V)
    gt = np.empty((B * L, G, V), dtype=np.float32)
    _check(lib().gmc_ref_mhem_fit_backward(_p(g), _p(m), *_ints(B, L, G, D, K, R), ctypes.c_float(kl_threshold), _p(gt)))
    return gt


def _conv_dims(data, kernels):
    data = np.ascontiguousarray(data, dtype=np.float32)
    kernels = np.ascontiguousarray(kernels, dtype=np.float32)
    B, Cin, G, V = data.shape
    Cout, Cin2, Gk, _ = kernels.shape
    assert Cin == Cin2
    return data, kernels, B, Cin, G, Cout, Gk, {7: 2, 13: 3}[V], V


def convolution_fitting_forward(data, kernels, K: int, tree: bool = False):
    """convolution_fitting::forward_impl_t -> (fitting, cached_pos_covs, nodesobjs, fitting_subtrees[, tree dict])."""
    data, kernels, B, Cin, G, Cout, Gk, D, V = _conv_dims(data, kernels)
    T = Cin * G * Gk
    out = np.empty((B, Cout, K, V), dtype=np.float32)
    cached = np.empty((B, Cout, K, D * D), dtype=np.float32)
    objs = np.empty((B, Cout, T), dtype=np.int32)
    sub = np.empty((B, Cout, 2 * K), dtype=np.int32)
    nodes = np.empty((B, Cout, 2 * T - 1, 3), dtype=np.int32) if tree else None
    mass = np.empty((B, Cout, T - 1), dtype=np.float32) if tree else None
    count = np.empty((B, Cout, T - 1), dtype=np.int32) if tree else None
    keys = np.empty((B, Cout, T), dtype=np.int64) if tree else None
    _check(lib_convfit().gmc_ref_convolution_fitting_forward(_p(data), _p(kernels), *_ints(B, Cin, G, Cout, Gk, D, K), _p(out),
                                                             _p(cached), _p(objs), _p(sub), _p(nodes), _p(mass), _p(count),
                                                             _p(keys)), lib_convfit())
    if tree:
        return out, cached, objs, sub, dict(nodes=nodes, mass=mass, count=count, keys=keys.view(np.uint64))
    return out, cached, objs, sub


def convolution_fitting_backward(grad, data, kernels, K: int):
    """Reference forward followed by convolution_fitting::backward_impl_t -> (grad_data, grad_kernels)."""
    data, kernels, B, Cin, G, Cout, Gk, D, V = _conv_dims(data, kernels)
    g = np.ascontiguousarray(grad, dtype=np.float32).reshape(B, Cout, K, V)
    gd = np.empty_like(data)
    gk = np.empty_like(kernels)
    _check(lib_convfit().gmc_ref_convolution_fitting_backward(_p(g), _p(data), _p(kernels), *_ints(B, Cin, G, Cout, Gk, D, K),
                                                              _p(gd), _p(gk)), lib_convfit())
    return gd, gk


def _eval_dims(mixture, xes):
    B, L, G, V = mixture.shape
    D = {7: 2, 13: 3}[V]
    Bx, Lx, N, Dx = xes.shape
    assert Dx == D and Bx in (1, B) and Lx in (1, L)
    return B, L, G, D, Bx, Lx, N


def eval_forward(mixture, xes):
    """parallel_forward_impl (the reference's CPU evaluation); float32 or float64 by the dtype of `mixture`."""
    dt = mixture.dtype
    mixture = np.ascontiguousarray(mixture)
    xes = np.ascontiguousarray(xes, dtype=dt)
    dims = _eval_dims(mixture, xes)
    out = np.empty((dims[0], dims[1], dims[6]), dtype=dt)
    fn = lib().gmc_ref_eval_forward if dt == np.float32 else lib().gmc_ref_eval_forward_f64
    _check(fn(_p(mixture), _p(xes), _p(out), *_ints(*dims)))
    return out


def eval_backward(grad_out, mixture, xes, need_mixture: bool = True, need_xes: bool = True):
    """parallel_backward_impl (fp32) -> (grad_mixture, grad_xes)."""
    mixture = np.ascontiguousarray(mixture, dtype=np.float32)
    xes = np.ascontiguousarray(xes, dtype=np.float32)
    grad_out = np.ascontiguousarray(grad_out, dtype=np.float32)
    dims = _eval_dims(mixture, xes)
    gm = np.empty_like(mixture) if need_mixture else None
    gx = np.empty_like(xes) if need_xes else None
    _check(lib().gmc_ref_eval_backward(_p(grad_out), _p(mixture), _p(xes), _p(gm), _p(gx), *_ints(*dims)))
    return gm, gx
