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
