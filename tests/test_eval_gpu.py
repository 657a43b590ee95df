"""GPU parity of evaluate_inversed forward/backward (CUDA through the C-ABI) against the fp64 CPU oracle and the
golden vectors from the reference's Python. Tolerance: relative 1e-4 per output tensor (||a-b||inf / ||ref||inf),
with the reference's own criterion (RMSE rounds to 0 at 4 places, src/gmc/test_cpp_eval.py:15-22) checked beside it."""
import numpy as np
import pytest
import torch

from conftest import rel_inf
from oracle import cpu_oracle

pytestmark = pytest.mark.gpu

TOL = 1e-4


def _gpu_eval(mixture: np.ndarray, xes: np.ndarray, grad_out: np.ndarray):
    import gmc.cpp.extensions.evaluate_inversed.evaluate_inversed as ev
    m = torch.from_numpy(mixture).cuda().requires_grad_(True)
    x = torch.from_numpy(xes).cuda().requires_grad_(True)
    out = ev.apply(m, x)
    out.backward(torch.from_numpy(grad_out).cuda())
    return out.detach().cpu().numpy(), m.grad.cpu().numpy(), x.grad.cpu().numpy()


def _check(mixture, xes, grad_out, ref=None, what=""):
    out, gm, gx = _gpu_eval(mixture, xes, grad_out)
    if ref is None:
        m64, x64, g64 = (a.astype(np.float64) for a in (mixture, xes, grad_out))
        ref_out = cpu_oracle.eval_forward(m64, x64)
        ref_gm, ref_gx = cpu_oracle.eval_backward(g64, m64, x64)
    else:
        ref_out, ref_gm, ref_gx = ref
    assert out.shape == ref_out.shape and gm.shape == ref_gm.shape and gx.shape == ref_gx.shape
    for name, a, r in (("out", out, ref_out), ("grad_mixture", gm, ref_gm), ("grad_xes", gx, ref_gx)):
        assert np.isfinite(a).all(), f"{what} {name} not finite"
        assert rel_inf(a, r) < TOL, f"{what} {name}: rel {rel_inf(a, r):.3e}"
    # grad_mixture per field (weight / position / matrix have different magnitudes)
    D = xes.shape[-1]
    for name, sl in (("w", slice(0, 1)), ("pos", slice(1, 1 + D)), ("mat", slice(1 + D, None))):
        assert rel_inf(gm[..., sl], ref_gm[..., sl]) < TOL, f"{what} grad_mixture[{name}]"


def test_golden_vectors(golden_eval):
    cases = sorted({k.rsplit("_mixture", 1)[0] for k in golden_eval if k.endswith("_mixture") and "grad" not in k})
    for c in cases:
        ref = (golden_eval[c + "_out"], golden_eval[c + "_grad_mixture"], golden_eval[c + "_grad_xes"])
        _check(golden_eval[c + "_mixture"], golden_eval[c + "_xes"], golden_eval[c + "_grad_out"], ref, c)
        out, _, _ = _gpu_eval(golden_eval[c + "_mixture"], golden_eval[c + "_xes"], golden_eval[c + "_grad_out"])
        rmse = float(np.sqrt(((out - golden_eval[c + "_out_f32ref"]) ** 2).mean()))
        assert round(rmse, 4) == 0


def _random_case(rng, B, L, G, N, D, bx, lx, radius=10.0):
    w = rng.uniform(-1, 1, (B, L, G)).astype(np.float32)
    p = rng.uniform(-radius, radius, (B, L, G, D)).astype(np.float32)
    A = rng.uniform(-1, 1, (B, L, G, D, D))
    cov = (A @ np.swapaxes(A, -1, -2) + np.eye(D) * 0.01) * radius
    inv = np.linalg.inv(cov)
    inv = 0.5 * (inv + np.swapaxes(inv, -1, -2))
    mixture = np.concatenate((w[..., None], p, inv.reshape(B, L, G, D * D).astype(np.float32)), -1)
    xes = rng.uniform(-radius, radius, (B if bx else 1, L if lx else 1, N, D)).astype(np.float32)
    grad_out = rng.standard_normal((B, L, N)).astype(np.float32)
    return np.ascontiguousarray(mixture), xes, grad_out


def test_shape_sweep_of_the_reference_test():
    # the sweep of src/gmc/test_cpp_eval.py:30-44 / 68-95 (per-layer and broadcast xes)
    rng = np.random.default_rng(7)
    for B in (1, 5):
        for L in (1, 4, 7):
            for G in (1, 6, 17, 50):
                for N in (1, 8, 23, 50):
                    for D in (2, 3):
                        for bx, lx in ((True, True), (False, False)):
                            m, x, g = _random_case(rng, B, L, G, N, D, bx, lx)
                            _check(m, x, g, what=f"B{B} L{L} G{G} N{N} D{D} bx{bx}")


@pytest.mark.parametrize("D", [2, 3])
@pytest.mark.parametrize("G,N", [(64, 700), (130, 513), (300, 1500), (700, 600), (1100, 530)])
def test_every_kernel_variant(D, G, N):
    # covers 1/2/4 Gaussians per thread, several Gaussian chunks, several point tiles, ragged edges,
    # and the unaligned (non-bulk) staging path (G not a multiple of 4)
    rng = np.random.default_rng(G * 7 + N + D)
    for bx, lx in ((True, True), (True, False), (False, False)):
        m, x, g = _random_case(rng, 2, 3, G, N, D, bx, lx, radius=1.0)
        _check(m, x, g, what=f"G{G} N{N} D{D} bx{bx} lx{lx}")


def _mixture_of_scale(rng, B, L, G, D, centre, spread, s_lo, s_hi):
    w = rng.uniform(-1, 1, (B, L, G)).astype(np.float32)
    p = (centre + rng.uniform(-spread, spread, (B, L, G, D))).astype(np.float32)
    Q = np.linalg.qr(rng.standard_normal((B, L, G, D, D)))[0]
    s = np.exp(rng.uniform(np.log(s_lo), np.log(s_hi), (B, L, G, D)))
    inv = Q @ (np.eye(D) / (s ** 2)[..., None]) @ np.swapaxes(Q, -1, -2)
    inv = 0.5 * (inv + np.swapaxes(inv, -1, -2))
    return np.ascontiguousarray(np.concatenate((w[..., None], p, inv.reshape(B, L, G, D * D).astype(np.float32)), -1))


@pytest.mark.parametrize("D", [2, 3])
def test_forward_loop_selection(D):
    """The forward kernel has a short pair loop on a triangular factor of the matrix, chosen per chunk of 256 Gaussians
    when (largest entry sum of the factor) x (extent of the tile's points) is small enough for its rounding, and the
    general loop otherwise. Regimes: benchmark-like (short loop); Gaussians a thousand times narrower than the domain
    (general loop); one narrow Gaussian in the second chunk only (both loops in one launch); a domain far from the
    origin (the loops work relative to the tile's centre); a matrix that is not positive definite (general loop; 2D
    only, where det > 0 leaves the norm factor real)."""
    rng = np.random.default_rng(90 + D)
    N = 1500

    def check(m, x, what, tol=TOL):
        out = _gpu_eval(m, x, np.ones((m.shape[0], m.shape[1], x.shape[2]), np.float32))[0]
        ref = cpu_oracle.eval_forward(m.astype(np.float64), x.astype(np.float64))
        assert np.isfinite(out).all(), what
        assert rel_inf(out, ref) < tol, f"{what}: rel {rel_inf(out, ref):.3e}"

    x = rng.uniform(-1.2, 1.2, (2, 3, N, D)).astype(np.float32)
    check(_mixture_of_scale(rng, 2, 3, 512, D, 0.0, 1.0, 0.03, 0.25), x, "benchmark-like")
    check(_mixture_of_scale(rng, 2, 3, 300, D, 0.0, 1.0, 0.0005, 0.002), np.ascontiguousarray(x[:, :, :400]), "narrow Gaussians")
    m = _mixture_of_scale(rng, 2, 3, 512, D, 0.0, 1.0, 0.05, 0.25)
    m[:, :, 400] = _mixture_of_scale(rng, 2, 3, 1, D, 0.0, 0.1, 0.0005, 0.001)[:, :, 0]
    m[:, :, 400, 0] = 1e-4                      # its peak is 1 / s^D times the weight: keep it comparable to the rest
    x_near = x.copy()
    x_near[:, :, :64] = m[:, :, 400, None, 1:1 + D] + rng.uniform(-0.002, 0.002, (2, 3, 64, D)).astype(np.float32)
    check(m, x_near, "one narrow Gaussian in the second chunk")
    far = 1000.0
    xf = (far + rng.uniform(-1.2, 1.2, (2, 3, N, D))).astype(np.float32)
    check(_mixture_of_scale(rng, 2, 3, 512, D, far, 1.0, 0.1, 0.5), xf, "domain far from the origin")
    if D == 2:
        m = _mixture_of_scale(rng, 2, 3, 64, D, 0.0, 1.0, 0.5, 1.0)
        m[:, :, ::2, 3:] *= -1.0                 # negative definite: det > 0, the exponent grows with the distance
        check(m, x, "matrix not positive definite")


def test_large_n_uses_the_four_points_per_thread_forward():
    rng = np.random.default_rng(5)
    for D in (2, 3):
        m, x, g = _random_case(rng, 4, 8, 33, 9601, D, True, True, radius=1.0)
        _check(m, x, g, what=f"large N D{D}")


def test_config0():
    import synthetic_inputs as synthetic
    m, x, g = synthetic.config0()
    _check(m.numpy(), x.numpy(), g.numpy(), what="config0")


def test_only_requested_gradients():
    import gmc.cpp.extensions.evaluate_inversed.evaluate_inversed as ev
    rng = np.random.default_rng(3)
    m, x, g = _random_case(rng, 2, 2, 40, 100, 3, True, True, radius=1.0)
    mt, xt, gt = (torch.from_numpy(a).cuda() for a in (m, x, g))
    gm_full, gx_full = ev.parallel_backward(gt, mt, xt, None, True, True)
    gm_only, gx_zero = ev.parallel_backward(gt, mt, xt, None, True, False)
    gm_zero, gx_only = ev.parallel_backward(gt, mt, xt, None, False, True)
    assert gx_zero.abs().max().item() == 0 and gm_zero.abs().max().item() == 0
    assert rel_inf(gm_only.cpu().numpy(), gm_full.cpu().numpy()) < 1e-5
    assert rel_inf(gx_only.cpu().numpy(), gx_full.cpu().numpy()) < 1e-5


def test_forward_is_deterministic_and_does_not_touch_inputs():
    import gmc.cpp.extensions.evaluate_inversed.evaluate_inversed as ev
    rng = np.random.default_rng(11)
    m, x, _ = _random_case(rng, 2, 3, 257, 1000, 3, True, True, radius=1.0)
    mt, xt = torch.from_numpy(m).cuda(), torch.from_numpy(x).cuda()
    a = ev.apply(mt, xt)
    b = ev.apply(mt, xt)
    assert torch.equal(a, b)
    assert torch.equal(mt.cpu(), torch.from_numpy(m)) and torch.equal(xt.cpu(), torch.from_numpy(x))


def test_config1_full_size_identities():
    """Full benchmark size (2^32 pairs). The output is linear in the weights, so
    sum_n grad_out[n] out[n] == sum_g w_g dL/dw_g for every (batch, layer); two whole (batch, layer) mixtures are
    checked against the fp64 oracle (forward, grad_mixture per field, grad_xes) at 1e-4."""
    import gmc.cpp.extensions.evaluate_inversed.evaluate_inversed as ev
    import synthetic_inputs as synthetic
    m, x, g = synthetic.config1()
    mt = m.cuda().requires_grad_(True)
    xt = x.cuda().requires_grad_(True)
    gt = g.cuda()
    out = ev.apply(mt, xt)
    out.backward(gt)
    lhs = (out.detach().double() * gt.double()).sum(-1)
    rhs = (mt.grad[..., 0].double() * mt.detach()[..., 0].double()).sum(-1)
    assert rel_inf(rhs.cpu().numpy(), lhs.cpu().numpy()) < TOL
    # translation identity: sum_n dL/dx_n == - sum_g dL/dmu_g
    sx = xt.grad.double().sum(2)
    sm = mt.grad[..., 1:4].double().sum(2)
    assert rel_inf((-sm).cpu().numpy(), sx.cpu().numpy()) < 1e-3
    # one (batch, layer) slice against the fp64 oracle, 2048 points
    b, l = 3, 5
    ms = m[b:b + 1, l:l + 1].numpy().astype(np.float64)
    xs = x[b:b + 1, l:l + 1, :2048].numpy().astype(np.float64)
    ref = cpu_oracle.eval_forward(ms, xs)
    assert rel_inf(out[b, l, :2048].detach().cpu().numpy(), ref[0, 0]) < TOL
    assert torch.isfinite(mt.grad).all() and torch.isfinite(xt.grad).all()
    # the backward variant used at this size, against the fp64 oracle: the whole grad_mixture of two (batch, layer)
    # mixtures over all 16384 points (per field), and grad_xes of those mixtures' points
    for (b, l) in ((3, 5), (31, 15)):
        ms = m[b:b + 1, l:l + 1].numpy().astype(np.float64)
        xs = x[b:b + 1, l:l + 1].numpy().astype(np.float64)
        gs = g[b:b + 1, l:l + 1].numpy().astype(np.float64)
        ref_gm, ref_gx = cpu_oracle.eval_backward(gs, ms, xs)
        got_gm = mt.grad[b, l].cpu().numpy()
        for name, sl in (("weight", slice(0, 1)), ("position", slice(1, 4)), ("matrix", slice(4, 13))):
            err = rel_inf(got_gm[:, sl], ref_gm[0, 0][:, sl])
            print(f"config1 ({b},{l}) grad_mixture {name}: rel {err:.2e}")
            assert err < TOL, f"grad_mixture {name} at ({b},{l}): {err:.2e}"
        err = rel_inf(xt.grad[b, l].cpu().numpy(), ref_gx[0, 0])
        print(f"config1 ({b},{l}) grad_xes: rel {err:.2e}")
        assert err < TOL, f"grad_xes at ({b},{l}): {err:.2e}"
        assert rel_inf(out[b, l].detach().cpu().numpy(), cpu_oracle.eval_forward(ms, xs)[0, 0]) < TOL


@pytest.mark.parametrize("D", [2, 3])
@pytest.mark.parametrize("B,bx,n_slices,pinned", [(5, True, 2, True), (5, True, 0, False), (4, False, 3, True),
                                                   (1, True, 4, True), (9, True, 4, True)])
def test_host_buffer_pipeline_equals_the_device_path(D, B, bx, n_slices, pinned):
    """gmc_eval_inversed_host (batch slices through copy-in / kernels / copy-out streams) returns the values of the
    device entry points for whole, ragged and single slices, shared xes, page-locked and pageable buffers. The forward
    is bit-identical; the gradients differ only by the order of the atomic sums."""
    import gmc.cpp.extensions.evaluate_inversed.evaluate_inversed as ev
    rng = np.random.default_rng(100 * D + B)
    mixture, xes, grad_out = _random_case(rng, B, 3, 70, 900, D, bx, True)
    out_d, gm_d, gx_d = _gpu_eval(mixture, xes, grad_out)
    host = [torch.from_numpy(a) for a in (mixture, xes, grad_out)]
    if pinned:
        host = [t.pin_memory() for t in host]
    for _ in range(2):     # second call reuses the cached workspace
        out_h, gm_h, gx_h = ev.host_forward_backward(*host, n_slices=n_slices)
    assert not out_h.is_cuda and not gm_h.is_cuda and not gx_h.is_cuda
    assert np.array_equal(out_h.numpy(), out_d)
    assert rel_inf(gm_h.numpy(), gm_d) < 1e-5 and rel_inf(gx_h.numpy(), gx_d) < 1e-5
    # forward only / one gradient only
    o2, g2, x2 = ev.host_forward_backward(host[0], host[1])
    assert g2 is None and x2 is None and np.array_equal(o2.numpy(), out_d)
    o3, g3, x3 = ev.host_forward_backward(*host, requires_grad_xes=False, want_forward=False, n_slices=n_slices)
    assert o3 is None and x3 is None and rel_inf(g3.numpy(), gm_d) < 1e-5
    assert ev._native.lib.gmc_host_pipeline_release() == 0


def test_cpu_tensors_go_through_the_operator():
    """CPU tensors given to the differentiable operator are evaluated on the GPU (the reference runs its host code)."""
    import gmc.cpp.extensions.evaluate_inversed.evaluate_inversed as ev
    rng = np.random.default_rng(5)
    mixture, xes, grad_out = _random_case(rng, 2, 2, 40, 300, 3, True, False)
    out_d, gm_d, gx_d = _gpu_eval(mixture, xes, grad_out)
    m = torch.from_numpy(mixture).requires_grad_(True)
    x = torch.from_numpy(xes).requires_grad_(True)
    out = ev.apply(m, x)
    out.backward(torch.from_numpy(grad_out))
    assert not out.is_cuda and np.array_equal(out.detach().numpy(), out_d)
    assert rel_inf(m.grad.numpy(), gm_d) < 1e-5 and rel_inf(x.grad.numpy(), gx_d) < 1e-5


def test_a_lost_bulk_copy_is_reported_and_never_hangs():
    """The forward kernel waits for its bulk copy with a poll limit. With the copy left out on purpose (test entry
    point; nothing is in flight) the wait runs out: the kernel returns, its outputs are NaN, the next check call returns
    GMC_ERR_DEVICE_CHECK, and the context keeps working."""
    import ctypes
    from gmc import _native
    import gmc.cpp.extensions.evaluate_inversed.evaluate_inversed as ev
    rng = np.random.default_rng(2)
    m, x, _ = _random_case(rng, 2, 2, 64, 300, 3, True, True, radius=1.0)     # 64 x 13 floats: a 16-byte multiple
    mt, xt = torch.from_numpy(m).cuda(), torch.from_numpy(x).cuda()
    assert _native.device_check_word() == 0
    out = torch.zeros(2, 2, 300, device="cuda")
    stream = _native.stream_of(mt)
    status = _native.lib.gmc_debug_eval_forward_lost_copy(_native.ptr(mt), _native.ptr(xt), _native.ptr(out), 2, 2, 64, 3, 2, 2,
                                                          300, stream)
    assert status == 0
    assert _native.lib.gmc_sync_and_check(stream) == 7           # GMC_ERR_DEVICE_CHECK
    assert torch.isnan(out).all()
    assert _native.lib.gmc_sync_and_check(stream) == 0           # the word was cleared
    with pytest.raises(_native.GmcError, match="device-side check"):
        _native.lib.gmc_debug_eval_forward_lost_copy(_native.ptr(mt), _native.ptr(xt), _native.ptr(out), 2, 2, 64, 3, 2, 2, 300,
                                                     stream)
        _native.sync_and_check()
    good = ev.apply(mt, xt)                                      # the context is intact
    ref = cpu_oracle.eval_forward(m.astype(np.float64), x.astype(np.float64))
    assert rel_inf(good.cpu().numpy(), ref) < TOL
    assert _native.device_check_word() == 0
