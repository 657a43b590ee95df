"""Mixture evaluation in inverse-covariance form as a differentiable operator.

Same import path, class name and `apply` signature as the reference's
src/gmc/cpp/extensions/evaluate_inversed/evaluate_inversed.py:18-40; the work is done by
gmc_eval_inversed_forward / gmc_eval_inversed_backward of libgmc_b200.so.
"""
import torch
import torch.autograd

from gmc import _native


def _check_shapes(mixture: torch.Tensor, xes: torch.Tensor):
    """Shape rules of gpe::check_input_and_get_ns (src/gmc/cpp/extensions/util/mixture.h:107-127)."""
    if mixture.dim() != 4:
        raise RuntimeError("mixture must have 4 dimensions")
    n_batch, n_layers, n_components, vec = mixture.shape
    if vec == 7:
        n_dims = 2
    elif vec == 13:
        n_dims = 3
    else:
        raise RuntimeError(f"mixture must have a last dimension of 7 (2d) or 13 (3d), got {vec}")
    if xes.dim() != 4:
        raise RuntimeError("xes must have 4 dimensions")
    if xes.dtype != mixture.dtype:
        raise RuntimeError("mixture and xes must have the same dtype")
    if xes.device != mixture.device:
        raise RuntimeError("mixture and xes must have the same device")
    if xes.shape[0] not in (1, n_batch):
        raise RuntimeError("xes must have a batch dimension equal to one or the mixture")
    if xes.shape[1] not in (1, n_layers):
        raise RuntimeError("xes must have a layer dimension equal to one or the mixture")
    if xes.shape[3] != n_dims:
        raise RuntimeError("xes must have the last dimension equal to the number of dimensions of the mixture")
    return n_batch, n_layers, n_components, n_dims, xes.shape[0], xes.shape[1], xes.shape[2]


def _require_host_f32(t: torch.Tensor, name: str) -> None:
    if t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous():
        raise _native.GmcError(f"{name} must be a contiguous float32 CPU tensor")


def host_forward_backward(mixture: torch.Tensor, xes: torch.Tensor, grad_output: torch.Tensor = None,
                          requires_grad_mixture: bool = True, requires_grad_xes: bool = True, n_slices: int = 0,
                          out: torch.Tensor = None, grad_mixture: torch.Tensor = None, grad_xes: torch.Tensor = None,
                          device=None, want_forward: bool = True):
    """Evaluation (and, with grad_output, its gradients) of CPU tensors on the GPU through
    gmc_eval_inversed_host: batch slices are copied in, computed and copied out in a pipeline of copy and kernel streams.
    Page-locked tensors (`pin_memory()`) let the copies overlap the kernels; result tensors may be passed in
    to reuse page-locked storage. Returns (out, grad_mixture, grad_xes); entries not asked for are None."""
    ns = _check_shapes(mixture, xes)
    _require_host_f32(mixture, "mixture")
    _require_host_f32(xes, "xes")
    n_batch, n_layers, n_components, _, _, _, n_xes = ns
    do_backward = grad_output is not None
    if do_backward:
        _require_host_f32(grad_output, "grad_output")
        if tuple(grad_output.shape) != (n_batch, n_layers, n_xes):
            raise RuntimeError("grad_output has the wrong shape")

    def result(t, shape, name, wanted):
        if not wanted:
            return None
        if t is None:
            return torch.empty(shape, dtype=torch.float32)
        _require_host_f32(t, name)
        if tuple(t.shape) != tuple(shape):
            raise RuntimeError(f"{name} has the wrong shape")
        return t

    out = result(out, (n_batch, n_layers, n_xes), "out", want_forward)
    grad_mixture = result(grad_mixture, mixture.shape, "grad_mixture", do_backward and requires_grad_mixture)
    grad_xes = result(grad_xes, xes.shape, "grad_xes", do_backward and requires_grad_xes)
    if n_xes == 0 or n_components == 0 or n_batch == 0 or n_layers == 0:
        for t in (out, grad_mixture, grad_xes):
            if t is not None:
                t.zero_()
        return out, grad_mixture, grad_xes
    if not torch.cuda.is_available():
        raise _native.GmcError("no CUDA device: this library has no CPU implementation")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        _native.check(_native.lib.gmc_eval_inversed_host(
            _native.ptr(mixture), _native.ptr(xes), _native.ptr(grad_output), _native.ptr(out),
            _native.ptr(grad_mixture), _native.ptr(grad_xes), *ns, int(n_slices)), "evaluate_inversed (host buffers)")
    return out, grad_mixture, grad_xes


def parallel_forward(mixture: torch.Tensor, xes: torch.Tensor):
    if not mixture.is_cuda and not xes.is_cuda:
        # CPU tensors (the reference runs its host implementation for them, evaluate_inversed.cpp:19): GPU through staging
        return (host_forward_backward(mixture.contiguous(), xes.contiguous())[0],)
    ns = _check_shapes(mixture, xes)
    _native.require_cuda_f32(mixture, "mixture")
    _native.require_cuda_f32(xes, "xes")
    n_batch, n_layers, _, _, _, _, n_xes = ns
    out = torch.empty((n_batch, n_layers, n_xes), dtype=torch.float32, device=mixture.device)
    if out.numel() == 0 or ns[2] == 0:
        return (out.zero_(),)
    with torch.cuda.device_of(mixture):
        _native.check(_native.lib.gmc_eval_inversed_forward(
            _native.ptr(mixture), _native.ptr(xes), _native.ptr(out), *ns, _native.stream_of(mixture)),
            "evaluate_inversed forward")
    return (out,)


def parallel_backward(grad_output, mixture, xes, forward_out, requires_grad_mixture: bool, requires_grad_xes: bool):
    if not mixture.is_cuda and not xes.is_cuda and not grad_output.is_cuda:
        _, gm_, gx_ = host_forward_backward(mixture.contiguous(), xes.contiguous(), grad_output.contiguous(),
                                            requires_grad_mixture, requires_grad_xes, want_forward=False)
        # gradients that are not required come back as zeros, as below
        return (gm_ if gm_ is not None else torch.zeros_like(mixture)), (gx_ if gx_ is not None else torch.zeros_like(xes))
    ns = _check_shapes(mixture, xes)
    _native.require_cuda_f32(mixture, "mixture")
    _native.require_cuda_f32(xes, "xes")
    _native.require_cuda_f32(grad_output, "grad_output")
    n_batch, n_layers, n_components, _, _, _, n_xes = ns
    if tuple(grad_output.shape) != (n_batch, n_layers, n_xes):
        raise RuntimeError("grad_output has the wrong shape")
    # gradients that are not required come back as zeros, as in the reference
    # (parallel_implementation_optimised_backward.cu:129-130)
    alloc = torch.empty if requires_grad_mixture else torch.zeros
    grad_mixture = alloc(mixture.shape, dtype=torch.float32, device=mixture.device)
    alloc = torch.empty if requires_grad_xes else torch.zeros
    grad_xes = alloc(xes.shape, dtype=torch.float32, device=mixture.device)
    if n_xes == 0 or n_components == 0:
        return grad_mixture.zero_(), grad_xes.zero_()
    with torch.cuda.device_of(mixture):
        _native.check(_native.lib.gmc_eval_inversed_backward(
            _native.ptr(grad_output), _native.ptr(mixture), _native.ptr(xes),
            _native.ptr(grad_mixture if requires_grad_mixture else None),
            _native.ptr(grad_xes if requires_grad_xes else None),
            *ns, _native.stream_of(mixture)), "evaluate_inversed backward")
    return grad_mixture, grad_xes


class EvaluateInversed(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mixture: torch.Tensor, xes: torch.Tensor):
        if not mixture.is_contiguous():
            mixture = mixture.contiguous()
        if not xes.is_contiguous():
            xes = xes.contiguous()
        output = parallel_forward(mixture, xes)
        ctx.save_for_backward(mixture, xes)
        return output[0]

    @staticmethod
    def backward(ctx, grad_output):
        if not grad_output.is_contiguous():
            grad_output = grad_output.contiguous()
        mixture, xes = ctx.saved_tensors
        grad_mixture, grad_xes = parallel_backward(grad_output, mixture, xes, None,
                                                   ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return grad_mixture, grad_xes


apply = EvaluateInversed.apply
