"""Generates the golden fixtures of this folder by running the REFERENCE's own Python on CPU.

Run where the reference checkout exists:   python tests/golden/make_golden.py
reference_native.npz additionally holds outputs of the reference's NATIVE code (CPU path) built by oracle/build_ref.py.
Inputs are seeded fp32 tensors; outputs come from the reference's gm.old_evaluate_inversed
(src/gmc/mixture.py:102-141, the ground truth of the reference's own src/gmc/test_cpp_eval.py) evaluated in
fp64 on the same values, with gradients from torch autograd through it.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_python  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def eval_cases(gm):
    cases = {}
    g = torch.Generator().manual_seed(1234)
    idx = 0
    # the reference's hand-made known-answer case (src/gmc/test_cpp_eval.py:25-28)
    specs = [("known", None)]
    for D in (2, 3):
        for (B, L, G, N, bx, lx) in ((1, 1, 1, 1, True, True), (2, 3, 6, 23, True, True), (2, 3, 17, 8, False, False),
                                     (3, 2, 50, 50, False, True), (2, 4, 64, 33, True, True)):
            specs.append((f"d{D}", (D, B, L, G, N, bx, lx)))
    for name, spec in specs:
        if spec is None:
            mixture = torch.tensor([1.0, 0.0, 0.0, 2.0, 0.0, 0.0, 2.0]).view(1, 1, 1, -1)
            xes = torch.zeros(1, 1, 1, 2)
        else:
            D, B, L, G, N, bx, lx = spec
            w = torch.rand(B, L, G, generator=g) * 2 - 1
            p = torch.rand(B, L, G, D, generator=g) * 20 - 10
            A = torch.rand(B, L, G, D, D, generator=g) * 2 - 1
            cov = (A @ A.transpose(-1, -2) + torch.eye(D) * 0.01) * 10
            mixture = gm.pack_mixture(w, p, cov.inverse().transpose(-2, -1)).contiguous()
            xes = torch.rand(B if bx else 1, L if lx else 1, N, D, generator=g) * 20 - 10
        m64 = mixture.double().requires_grad_(True)
        x64 = xes.double().requires_grad_(True)
        # the reference accumulates into an fp32 buffer (mixture.py:115); sum the fp64 slices directly instead
        out = gm.evaluate_componentwise_inversed(m64, x64).sum(-1)
        grad_out = torch.randn(out.shape, generator=g).float()
        (out * grad_out.double()).sum().backward()
        key = f"eval{idx:02d}_{name}"
        cases[key + "_mixture"] = mixture.numpy()
        cases[key + "_xes"] = xes.numpy()
        cases[key + "_grad_out"] = grad_out.numpy()
        cases[key + "_out"] = out.detach().numpy()
        cases[key + "_grad_mixture"] = m64.grad.numpy()
        cases[key + "_grad_xes"] = x64.grad.numpy()
        # the reference's fp32 function on the same inputs (cross-check of the fp64 route)
        cases[key + "_out_f32ref"] = gm.old_evaluate_inversed(mixture, xes).numpy()
        idx += 1
    return cases


def convolve_cases(gm):
    """Inputs and the reference's gm.convolve (src/gmc/mixture.py:243-274) per output channel.
    gm.convolve(data [B, Cin, G, V], kernels[o] [1, Cin, Gk, V]) -> [B, Cin, G*Gk, V] (pairs of one input channel)."""
    cases = {}
    g = torch.Generator().manual_seed(4321)
    for idx, (D, B, Cin, G, Cout, Gk) in enumerate(((2, 2, 3, 6, 2, 4), (3, 2, 2, 5, 3, 3))):
        def mixture(n0, n1, n2, pos, cov_scale, wscale):
            w = torch.randn(n0, n1, n2, generator=g) * wscale
            p = torch.randn(n0, n1, n2, D, generator=g) * pos
            A = torch.rand(n0, n1, n2, D, D, generator=g) * 2 - 1
            c = (A @ A.transpose(-1, -2) + torch.eye(D) * 0.05) * cov_scale
            return gm.pack_mixture(w, p, c).contiguous()
        data = mixture(B, Cin, G, 1.0, 0.05, 1.0)
        kernels = mixture(Cout, Cin, Gk, 0.1, 0.01, 0.1)
        per_channel = torch.stack([gm.convolve(data, kernels[o:o + 1]) for o in range(Cout)], dim=1)
        cases[f"conv{idx}_data"] = data.numpy()
        cases[f"conv{idx}_kernels"] = kernels.numpy()
        cases[f"conv{idx}_out"] = per_channel.reshape(B, Cout, Cin * G * Gk, -1).numpy()   # set of products per (b, o)
    return cases


def relu_fit_cases(gm, fitting):
    """Inputs and outputs of the reference's initial_approx_to_relu / fixed_point_iteration_to_relu
    (src/gmc/fitting.py:279-312), evaluated in fp64."""
    cases = {}
    g = torch.Generator().manual_seed(999)
    for idx, (D, B, L, G) in enumerate(((2, 2, 3, 12), (3, 2, 2, 9))):
        w = torch.randn(B, L, G, generator=g)
        p = torch.rand(B, L, G, D, generator=g) * 2 - 1
        A = torch.rand(B, L, G, D, D, generator=g) * 2 - 1
        c = (A @ A.transpose(-1, -2) + torch.eye(D) * 0.05) * 0.05
        mixture = gm.pack_mixture(w, p, c).contiguous()
        constant = torch.randn(B, L, generator=g) * 0.3
        m64, c64 = mixture.double(), constant.double()
        initial = fitting.initial_approx_to_relu(m64, c64)
        fp, ret_const = fitting.fixed_point_iteration_to_relu(m64, c64, initial)
        cases[f"relu{idx}_mixture"] = mixture.numpy()
        cases[f"relu{idx}_constant"] = constant.numpy()
        cases[f"relu{idx}_initial"] = initial.numpy()
        cases[f"relu{idx}_fixed_point"] = fp.numpy()
        cases[f"relu{idx}_ret_const"] = ret_const.numpy()
    return cases


def strategy_cases(gm, fitting):
    """Outputs of the reference's other ReLU-fit strategies (src/gmc/fitting.py:19-54 solver, :117-153
    fixed_point_and_max, :204-240 fixed_point_and_mhem with representative_select_for_relu / mhem_fit_a_to_b,
    :243-276 splitter), evaluated in fp64 on seeded inputs."""
    cases = {}
    g = torch.Generator().manual_seed(2024)
    for idx, (D, B, L, G, K) in enumerate(((2, 2, 2, 20, 8), (3, 2, 2, 12, 4))):
        w = torch.randn(B, L, G, generator=g)
        p = torch.rand(B, L, G, D, generator=g) * 2 - 1
        A = torch.rand(B, L, G, D, D, generator=g) * 2 - 1
        c = (A @ A.transpose(-1, -2) + torch.eye(D) * 0.05) * 0.05
        mixture = gm.pack_mixture(w, p, c).contiguous()
        constant = torch.randn(B, L, generator=g) * 0.3
        m64, c64 = mixture.double(), constant.double()
        cases[f"s{idx}_mixture"] = mixture.numpy()
        cases[f"s{idx}_constant"] = constant.numpy()
        cases[f"s{idx}_k"] = np.array(K)
        out, const, _ = fitting.fixed_point_and_max(m64, c64, K)
        cases[f"s{idx}_max"], cases[f"s{idx}_max_const"] = out.numpy(), const.numpy()
        out, const, steps = fitting.fixed_point_and_mhem(m64, c64, K)
        cases[f"s{idx}_mhem"], cases[f"s{idx}_mhem_selected"] = out.numpy(), steps[2].numpy()
        # the dense EM raises likelihoods to powers of about 20 |w|: the reference's own fp32 run differs from its
        # fp64 run by up to 6e-3, so the fp32 result is stored as well
        cases[f"s{idx}_mhem_f32"] = fitting.fixed_point_and_mhem(mixture, constant, K)[0].numpy()
        # the reference's solver adds the constant without a trailing axis (fitting.py:40): it only accepts [B, L, 1]
        out, const, _ = fitting.solver(m64, c64.unsqueeze(-1), K)
        cases[f"s{idx}_solver"] = out.numpy()
        positive = gm.pack_mixture(gm.weights(m64).abs() + 0.1, gm.positions(m64), gm.covariances(m64))
        cases[f"s{idx}_split"] = fitting.splitter(positive, [G + 3, G + 5]).numpy()
    return cases


def support_collections(reference_root):
    """The inline 2D mixtures and incoming-gradient sets of the reference's native unit tests
    (src/gmc/cpp/extensions/unittests/support.h:228-1020), read from the header as text:
    {function name: [arrays of shape [n, 7]]}."""
    import re
    path = os.path.join(reference_root, "src", "gmc", "cpp", "extensions", "unittests", "support.h")
    text = open(path).read()
    heads = [(m.start(), m.group(1)) for m in re.finditer(r"std::vector<torch::Tensor>\s+(\w+)\s*\(\)", text)]
    out = {}
    for i, (pos, name) in enumerate(heads):
        body = text[pos:heads[i + 1][0] if i + 1 < len(heads) else len(text)]
        tensors = []
        for m in re.finditer(r"torch::tensor\(\{(.*?)\}\)\s*\.view\(\{([\d, ]+)\}\)", body, re.S):
            shape = [int(v) for v in m.group(2).split(",")]
            values = [float(v.rstrip("f")) for v in re.findall(r"-?\d*\.?\d+(?:e-?\d+)?f?", m.group(1))]
            tensors.append(np.asarray(values, dtype=np.float32).reshape(shape[-2], shape[-1]))
        if tensors:
            out[name] = tensors
    return out


def reference_native_cases(reference_root):
    """Outputs of the REFERENCE's own native CPU code (oracle/_ref/libgmc_ref.so, built from the reference sources by
    oracle/build_ref.py) on (a) the inline mixtures / gradient sets of its unit tests and (b) small seeded cases:
    LBVH keys and nodes, BVH-MHEM fit forward + backward, convolution_fitting forward + backward."""
    from oracle import ref_native
    cases = {}
    coll = support_collections(reference_root)
    grads_by_k = {2: coll["_collectionOf2d2GsGrads"], 4: coll["_collectionOf2d4GsGrads"],
                  8: coll["_collectionOf2d8GsGrads"], 32: coll["_collectionOf2d32GsGradsWellBehaving"]}
    plan = []   # (collection, K, R)
    for name, tensors in sorted(coll.items()):
        if "Mixtures" not in name:
            continue
        G = tensors[0].shape[0]
        plan.append((name, {4: 2, 8: 4, 16: 8, 128: 32}[G], {4: 2, 8: 4, 16: 4, 128: 4}[G]))
        if G == 8:
            plan.append((name, 4, 2))
    idx = 0
    for name, K, R in plan:
        for mi, mixture in enumerate(coll[name]):
            G = mixture.shape[0]
            m = mixture.reshape(1, 1, G, 7)
            grad = grads_by_k[K][mi % len(grads_by_k[K])].reshape(1, 1, K, 7)
            fit, dump = ref_native.mhem_fit_forward(m, K, R, dump=True)
            if not (np.isfinite(fit).all()):
                continue
            key = f"mhem{idx:03d}"
            cases[key + "_source"] = np.array(f"{name}[{mi}] K={K} R={R}")
            cases[key + "_mixture"] = m
            cases[key + "_kr"] = np.array([K, R])
            cases[key + "_grad"] = grad
            cases[key + "_fitting"] = fit
            cases[key + "_nodes"] = dump["nodes"]
            cases[key + "_counts"] = dump["counts"]
            cases[key + "_grad_target"] = ref_native.mhem_fit_backward(grad, m, K, R)
            keys, nodes = ref_native.lbvh_build(m)
            cases[key + "_keys"] = keys
            idx += 1
    # seeded cases: 3D fit, convolution fitting in 2D and 3D
    g = torch.Generator().manual_seed(31337)

    def mixture(n0, n1, n2, D, pos, cov_scale, wlo, whi):
        w = torch.rand(n0, n1, n2, generator=g) * (whi - wlo) + wlo
        p = torch.randn(n0, n1, n2, D, generator=g) * pos
        A = torch.rand(n0, n1, n2, D, D, generator=g) * 2 - 1
        c = (A @ A.transpose(-1, -2) + torch.eye(D) * 0.05) * cov_scale
        return torch.cat((w.unsqueeze(-1), p, c.reshape(n0, n1, n2, D * D)), -1).contiguous().numpy()

    for D, G, K, R in ((3, 40, 8, 4), (3, 24, 8, 2), (2, 96, 16, 4)):
        m = mixture(1, 2, G, D, 1.0, 0.02, 0.1, 1.0)
        grad = torch.randn(1, 2, K, m.shape[-1], generator=g).numpy()
        fit, dump = ref_native.mhem_fit_forward(m, K, R, dump=True)
        key = f"mhem{idx:03d}"
        cases[key + "_source"] = np.array(f"seeded D={D} G={G} K={K} R={R}")
        cases[key + "_mixture"], cases[key + "_kr"], cases[key + "_grad"] = m, np.array([K, R]), grad
        cases[key + "_fitting"], cases[key + "_nodes"], cases[key + "_counts"] = fit, dump["nodes"], dump["counts"]
        cases[key + "_grad_target"] = ref_native.mhem_fit_backward(grad, m, K, R)
        cases[key + "_keys"] = ref_native.lbvh_build(m)[0]
        idx += 1
    cases["n_mhem"] = np.array(idx)
    for ci, (D, B, Cin, G, Cout, Gk, K) in enumerate(((2, 2, 3, 16, 2, 5, 8), (3, 1, 4, 12, 3, 5, 6), (2, 1, 2, 9, 2, 3, 54))):
        data = mixture(B, Cin, G, D, 1.0, 0.02, -1.0, 1.0)
        kernels = mixture(Cout, Cin, Gk, D, 0.1, 0.005, -0.3, 0.3)
        grad = torch.randn(B, Cout, K, data.shape[-1], generator=g).numpy()
        with ref_native.serial():     # race-free run of the reference's mass pass (see oracle/ref_entry.cu)
            out, cached, objs, sub, tree = ref_native.convolution_fitting_forward(data, kernels, K, tree=True)
            gd, gk = ref_native.convolution_fitting_backward(grad, data, kernels, K)
        key = f"cf{ci}"
        cases[key + "_data"], cases[key + "_kernels"], cases[key + "_k"], cases[key + "_grad"] = data, kernels, np.array(K), grad
        cases[key + "_fitting"], cases[key + "_cached"], cases[key + "_nodesobjs"], cases[key + "_subtrees"] = out, cached, objs, sub
        cases[key + "_keys"], cases[key + "_nodes"], cases[key + "_mass"] = tree["keys"], tree["nodes"], tree["mass"]
        cases[key + "_grad_data"], cases[key + "_grad_kernels"] = gd, gk
    cases["n_cf"] = np.array(3)
    return cases


def gmcn3d_network_case():
    """The REFERENCE's own network (src/gmc/model.py Net with src/gmc/modules.py layers) run on CPU with every
    extension routed to the reference's native CPU code: the layer stack of benchmark configuration 4 (conv 1->8 fit
    64, 8->16 fit 32, 16->32 fit 16, 32->64 fit 8; 5-component kernels; default ReLU fit and normalisation settings;
    evaluation mode; parameters from the constructors under torch.manual_seed(4)) on a batch of 2 seeded inputs.
    Stored: the mixture after every layer's normalisation, the integrated features, and per-parameter checksums
    (the constructors of this package draw the same values under the same seed; the test asserts that first)."""
    sys.path.insert(0, ROOT)
    import synthetic_inputs as synthetic
    gm, modules, model = ref_python.load_network()
    cfg = model.Config(n_dims=3)
    cfg.n_classes = 64            # the reference's forward ends in view(n_batch, n_classes); the tail is not stored
    cfg.layers = [model.Layer(8, 1, 64, 64), model.Layer(16, 1, 32, 32), model.Layer(32, 1, 16, 16), model.Layer(64, 1, 8, 8)]
    torch.manual_seed(4)
    net = model.Net(config=cfg).eval()
    x = synthetic.config4_input(2, 1004)
    acts, feats, convs = [], [], []
    for i in range(4):
        net.norms[i].register_forward_hook(lambda mod, inp, out: acts.append(out[0].detach().clone()))
        net.gmcs[i].register_forward_hook(lambda mod, inp, out: convs.append(out[0].detach().clone()))
    net.normX.register_forward_hook(lambda mod, inp, out: feats.append(inp[0].detach().clone()))
    norm0 = []
    net.norm0.register_forward_hook(lambda mod, inp, out: norm0.append((out[0].detach().clone(), out[1].detach().clone())))
    with torch.no_grad():
        net(x)
    # the input normalisation estimates a standard deviation from RANDOM sample points (src/gmc/modules.py:374-425), so its
    # output depends on the random stream; it is stored and fed to the layers under test instead of being recomputed
    cases = {"input": x.numpy(), "features": feats[0].numpy(), "norm0": norm0[0][0].numpy(), "norm0_constant": norm0[0][1].numpy()}
    for i in range(4):
        cases[f"layer{i}"] = acts[i].numpy()
        cases[f"conv{i}"] = convs[i].numpy()
    names = sorted(net.state_dict().keys())
    cases["param_names"] = np.array(names)
    cases["param_checksums"] = np.array([[float(v.double().sum()), float(v.double().abs().sum())]
                                         for v in (net.state_dict()[n] for n in names)])
    return cases


def relu_tree_hem_case():
    """The reference's fixed_point_and_tree_hem (src/gmc/fitting.py:162-201, tree_hem :342-358) with the reference's
    native BVH-MHEM fit and native evaluation, at the shape of benchmark configuration 2 (2D, 1024 -> 64, R = 4) on
    two mixtures, and in 3D (64 -> 16, R = 4 and R = 2)."""
    import gmc.fitting as fitting
    import synthetic_inputs as synthetic
    cases = {}
    target, constant = synthetic.config2(n_batch=1, n_layers=2, seed=1002)
    out, ret_const, steps = fitting.fixed_point_and_tree_hem(target, constant, 64, fitting.Config(n_reduction=4))
    cases["c2_target"], cases["c2_constant"] = target.numpy(), constant.numpy()
    cases["c2_fixed_point"], cases["c2_fitting"], cases["c2_ret_const"] = steps[1].numpy(), out.numpy(), ret_const.numpy()
    t3 = synthetic.config4_input(2, 2004).view(1, 2, 64, 13).contiguous()
    t3[..., 0] = t3[..., 0] * torch.where(torch.arange(64) % 3 == 0, -1.0, 1.0)
    c3 = torch.tensor([[0.05, -0.02]])
    for R in (4, 2):
        out, ret_const, steps = fitting.fixed_point_and_tree_hem(t3, c3, 16, fitting.Config(n_reduction=R))
        cases[f"d3r{R}_fitting"], cases[f"d3r{R}_ret_const"] = out.numpy(), ret_const.numpy()
    cases["d3_target"], cases["d3_constant"] = t3.numpy(), c3.numpy()
    return cases


def inout_files(gm):
    """Files written by the REFERENCE's own src/gmc/inout.py (save -> version 6, write_gm_to_ply) plus dictionaries in
    the older layouts its load() accepts (versions 3, 4, 5), with what the reference's load / read_gm_from_ply return
    for each of them.  Written to tests/golden/inout/."""
    import pathlib
    import gmc.config as ref_config
    import gmc.inout as ref_inout
    folder = os.path.join(HERE, "inout")
    os.makedirs(folder, exist_ok=True)
    ref_config.data_base_path = pathlib.Path(folder)
    g = torch.Generator().manual_seed(77)
    w = torch.rand(2, 1, 5, generator=g) + 0.1
    p = torch.rand(2, 1, 5, 3, generator=g) * 2 - 1
    A = torch.rand(2, 1, 5, 3, 3, generator=g) * 2 - 1
    c = A @ A.transpose(-1, -2) * 0.1 + torch.eye(3) * 0.02
    m = gm.pack_mixture(w, p, c)
    ref_inout.save(m, "mixture_v6.torch", meta_info={"source": "reference inout.save", "n": 5})
    amplitudes = gm.convert_priors_to_amplitudes(m)
    torch.save({"type": "gm.Mixture", "version": 5, "data": amplitudes, "meta_info": None}, os.path.join(folder, "mixture_v5.torch"))
    torch.save({"type": "gm.Mixture", "version": 4, "weights": gm.weights(amplitudes), "positions": gm.positions(amplitudes),
                "covariances": gm.covariances(amplitudes), "meta_info": "v4"}, os.path.join(folder, "mixture_v4.torch"))
    torch.save({"type": "gm.Mixture", "version": 3, "weights": gm.weights(amplitudes).view(2, 5),
                "positions": gm.positions(amplitudes).view(2, 5, 3), "covariances": gm.covariances(amplitudes).view(2, 5, 3, 3),
                "meta_info": None}, os.path.join(folder, "mixture_v3.torch"))
    expected = {}
    for v in (3, 4, 5, 6):
        loaded, _ = ref_inout.load(f"mixture_v{v}.torch")
        expected[f"v{v}"] = loaded.numpy()
    ply = os.path.join(folder, "mixture.ply")
    ref_inout.write_gm_to_ply(gm.weights(m), gm.positions(m), gm.covariances(m), 1, ply)
    expected["ply_plain"] = ref_inout.read_gm_from_ply(ply, ismodel=False, device="cpu").numpy()
    expected["ply_model"] = ref_inout.read_gm_from_ply(ply, ismodel=True, device="cpu").numpy()
    expected["mixture"] = m.numpy()
    np.savez_compressed(os.path.join(folder, "expected.npz"), **expected)


def lbvh_option_cases():
    """LBVH builds of the reference's native CPU code with the options of lbvh::Config: the five key layouts, and
    make_aabbs with layouts 0 and 1 (mixtures in inverse-covariance form, as lbvh/bvh.cu:204 expects)."""
    from oracle import ref_native
    cases = {}
    idx = 0
    for mi, (D, G) in enumerate(((2, 50), (3, 50), (2, 333), (3, 600))):
        g = torch.Generator().manual_seed(9000 + 10 * D + G)
        w = torch.rand(2, 2, G, generator=g) * 2 - 1
        w = torch.where(w.abs() < 0.05, torch.full_like(w, 0.05), w)
        p = torch.rand(2, 2, G, D, generator=g) * 2 - 1
        A = torch.rand(2, 2, G, D, D, generator=g) * 2 - 1
        cov = (A @ A.transpose(-1, -2) + torch.eye(D) * 0.2) * 0.05
        inv = torch.linalg.inv(cov.double())
        inv = (0.5 * (inv + inv.transpose(-1, -2))).float()
        m = torch.cat((w.unsqueeze(-1), p, inv.reshape(2, 2, G, D * D)), -1).contiguous().numpy()
        for algorithm in range(5):
            for make_aabbs in ((False, True) if algorithm < 2 else (False,)):
                out = ref_native.lbvh_build(m, algorithm, make_aabbs, 0.001)
                key = f"lbvh{idx:02d}"
                cases[f"mixture{mi}"] = m
                cases[key + "_options"] = np.array([mi, algorithm, int(make_aabbs)])
                cases[key + "_keys"], cases[key + "_nodes"] = out[0], out[1]
                if make_aabbs:
                    cases[key + "_aabbs"] = out[2]
                idx += 1
    cases["n_cases"] = np.array(idx)
    return cases


def main():
    if "--lbvh-options" in sys.argv:
        from oracle import build_ref
        build_ref.build()
        np.savez_compressed(os.path.join(HERE, "reference_lbvh_options.npz"), **lbvh_option_cases())
        print("wrote reference_lbvh_options.npz")
        return
    if "--network" in sys.argv:
        from oracle import build_ref
        build_ref.build()
        np.savez_compressed(os.path.join(HERE, "gmcn3d_forward.npz"), **gmcn3d_network_case())
        print("wrote gmcn3d_forward.npz")
        np.savez_compressed(os.path.join(HERE, "relu_tree_hem.npz"), **relu_tree_hem_case())
        print("wrote relu_tree_hem.npz")
        return
    import subprocess
    subprocess.run([sys.executable, os.path.abspath(__file__), "--network"], check=True)   # a process of its own
    reference_root = os.environ.get("GMC_REFERENCE_ROOT", "/root/reference")
    from oracle import build_ref
    build_ref.build()
    np.savez_compressed(os.path.join(HERE, "reference_native.npz"), **reference_native_cases(reference_root))
    print("wrote reference_native.npz")
    np.savez_compressed(os.path.join(HERE, "reference_lbvh_options.npz"), **lbvh_option_cases())
    print("wrote reference_lbvh_options.npz")
    gm, fitting, mat_tools = ref_python.load()
    np.savez_compressed(os.path.join(HERE, "eval_inversed.npz"), **eval_cases(gm))
    print("wrote eval_inversed.npz")
    np.savez_compressed(os.path.join(HERE, "convolve.npz"), **convolve_cases(gm))
    print("wrote convolve.npz")
    # gm.evaluate inside the fixed-point iteration runs in fp64 through the reference's dense formulation
    gm.evaluate_inversed = lambda m, x: gm.evaluate_componentwise_inversed(m, x).sum(-1)
    np.savez_compressed(os.path.join(HERE, "relu_fit.npz"), **relu_fit_cases(gm, fitting))
    print("wrote relu_fit.npz")
    np.savez_compressed(os.path.join(HERE, "strategies.npz"), **strategy_cases(gm, fitting))
    print("wrote strategies.npz")
    inout_files(gm)
    print("wrote inout/")


if __name__ == "__main__":
    main()
