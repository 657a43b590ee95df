"""ctypes binding of libgmc_b200.so, the C-ABI library that holds every CUDA kernel of this package.

There is no CPU or eager-PyTorch code path behind these functions: if the shared object is missing the
import fails, and a tensor that does not live on a CUDA device is rejected.
"""
import ctypes
import os

import torch

# GMC_B200_LIB selects another build of the same library (for example one compiled with different tuning macros).
_LIB_PATH = os.environ.get("GMC_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lib",
                                                            "libgmc_b200.so")

if not os.path.exists(_LIB_PATH):
    raise ImportError(
        f"{_LIB_PATH} not found. Build it first (python build.py in the package root); "
        "this package has no fallback implementation.")

lib = ctypes.CDLL(_LIB_PATH)

_c_float_p = ctypes.c_void_p
_c_int = ctypes.c_int
_c_void_p = ctypes.c_void_p

lib.gmc_status_string.restype = ctypes.c_char_p
lib.gmc_status_string.argtypes = [_c_int]
lib.gmc_last_cuda_error.restype = ctypes.c_char_p
lib.gmc_last_cuda_error.argtypes = []
lib.gmc_version.restype = ctypes.c_char_p
lib.gmc_version.argtypes = []
lib.gmc_device_check_word.restype = _c_int
lib.gmc_device_check_word.argtypes = [ctypes.POINTER(_c_int)]


def _declare(name, argtypes):
    fn = getattr(lib, name)
    fn.restype = _c_int
    fn.argtypes = argtypes
    return fn


_declare("gmc_eval_inversed_forward", [_c_float_p] * 3 + [_c_int] * 7 + [_c_void_p])
_declare("gmc_eval_inversed_backward", [_c_float_p] * 5 + [_c_int] * 7 + [_c_void_p])
_declare("gmc_debug_eval_forward_lost_copy", [_c_float_p] * 3 + [_c_int] * 7 + [_c_void_p])
_declare("gmc_sync_and_check", [_c_void_p])
_declare("gmc_debug_index_check", [_c_float_p, _c_float_p, ctypes.c_longlong, ctypes.c_longlong, _c_void_p])
_declare("gmc_eval_inversed_host", [_c_float_p] * 6 + [_c_int] * 8)
_declare("gmc_host_pipeline_release", [])
_declare("gmc_relu_fixed_point", [_c_float_p] * 5 + [ctypes.c_longlong, _c_int, _c_int, _c_void_p])
_declare("gmc_relu_fixed_point_layer", [_c_float_p] * 5 + [ctypes.c_longlong, _c_int, _c_int, ctypes.c_float, _c_float_p,
                                        _c_int, _c_void_p])
_declare("gmc_matrix_inverse", [_c_float_p] * 2 + [ctypes.c_longlong, _c_int, _c_void_p])
_declare("gmc_matrix_inverse_backward", [_c_float_p] * 3 + [ctypes.c_longlong, _c_int, _c_void_p])
_declare("gmc_lbvh_build", [_c_float_p, ctypes.c_longlong, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p])
_declare("gmc_lbvh_build_ex", [_c_float_p, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_int, ctypes.c_float, _c_void_p,
                               _c_void_p, _c_void_p, _c_void_p])
lib.gmc_mhem_fit_attribute_floats.restype = ctypes.c_size_t
lib.gmc_mhem_fit_attribute_floats.argtypes = [_c_int, _c_int, _c_int]
_declare("gmc_mhem_fit_forward", [_c_float_p, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p,
                                  _c_void_p, _c_void_p, _c_void_p])
lib.gmc_mhem_fit_forward_noalloc_capacity.restype = ctypes.c_longlong
lib.gmc_mhem_fit_forward_noalloc_capacity.argtypes = []
_declare("gmc_mhem_fit_forward_noalloc", [_c_float_p, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                          _c_void_p, _c_void_p, _c_void_p])
_declare("gmc_convolution_forward", [_c_float_p] * 3 + [_c_int] * 6 + [_c_void_p])
_declare("gmc_convolution_backward", [_c_float_p] * 5 + [_c_int] * 6 + [_c_void_p])
_declare("gmc_convolution_fitting_forward", [_c_float_p] * 2 + [_c_int] * 7 + [_c_void_p] * 5)
_declare("gmc_convolution_fitting_backward", [_c_float_p] * 3 + [_c_int] * 7 + [_c_void_p] * 7)
_declare("gmc_convolution_fitting_forward_large", [_c_float_p] * 2 + [_c_int] * 7 + [_c_void_p] * 5 + [ctypes.c_size_t, _c_void_p])
lib.gmc_convolution_fitting_large_scratch_bytes.restype = ctypes.c_size_t
lib.gmc_convolution_fitting_large_scratch_bytes.argtypes = [_c_int] * 5
_declare("gmc_mhem_fit_backward", [_c_float_p, _c_float_p, ctypes.c_longlong, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                                   _c_void_p, _c_void_p, _c_void_p, _c_void_p])
_declare("gmc_symeig", [_c_float_p] * 3 + [ctypes.c_longlong, _c_int, _c_void_p])
_declare("gmc_integrate", [_c_float_p] * 2 + [ctypes.c_longlong, _c_int, _c_int, _c_void_p])
_declare("gmc_trace_scale", [_c_float_p] * 3 + [ctypes.c_longlong, _c_int, _c_int, _c_void_p])
_declare("gmc_spatial_scale", [_c_float_p] * 3 + [ctypes.c_longlong, _c_int, _c_int, _c_void_p])
_declare("gmc_input_normalise", [_c_float_p, _c_void_p, _c_float_p, _c_float_p, ctypes.c_longlong, _c_int, _c_int, _c_int,
                                 _c_void_p, _c_void_p, _c_void_p])


class GmcError(RuntimeError):
    pass


_entry_calls = 0


def entry_calls() -> int:
    """Number of library calls checked so far in this process (every operator call passes through check())."""
    return _entry_calls


def check(status: int, what: str) -> None:
    global _entry_calls
    _entry_calls += 1
    if status != 0:
        msg = lib.gmc_status_string(status).decode()
        cuda_msg = lib.gmc_last_cuda_error().decode()
        if cuda_msg:
            msg = f"{msg} ({cuda_msg})"
        raise GmcError(f"{what}: {msg}")


def ptr(t) -> ctypes.c_void_p:
    """Device address of a tensor (None -> NULL)."""
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream_of(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def require_cuda_f32(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise GmcError(f"{name} must be a CUDA tensor: this library has no CPU implementation")
    if t.dtype != torch.float32:
        raise GmcError(f"{name} must be float32 (got {t.dtype})")
    if not t.is_contiguous():
        raise GmcError(f"{name} must be contiguous")


def sync_and_check(device=None) -> None:
    """Waits for the current stream of `device` and raises GmcError if a kernel reported a give-up since the last check."""
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    check(lib.gmc_sync_and_check(stream), "device-side check")


def device_check_word() -> int:
    w = _c_int(0)
    check(lib.gmc_device_check_word(ctypes.byref(w)), "gmc_device_check_word")
    return w.value
