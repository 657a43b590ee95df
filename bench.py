"""Benchmark of the mixture-evaluation hot path: evaluate_inversed forward + backward, 3D, fp32.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one forward + backward pass over one batch of the 3D evaluation configuration
(B=32 per GPU, L=16, G=512 components, N=16384 query points: 2^32 Gaussian-point pairs per GPU and step).
With N > 1 (launched under torch.distributed.run, one rank per GPU) every rank owns its own batch shard
(weak scaling); the only inter-GPU traffic is an NCCL all-gather of the forward outputs, enqueued on a side
stream so that it overlaps the backward kernel. Rank 0 prints one JSON line.

--impl reference times the reference's CPU algorithm (the oracle restatement of its OpenMP path, fp32) on the
host cores for the same metric, on a bounded batch slice of the same workload.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "gaussian-mixture-convolution-networks_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

METRIC = "gaussian_point_evals_per_s_fwd_bwd_3d"
UNIT = "pair-evals/s"
L, G, N, D = 16, 512, 16384, 3
B_PER_GPU = 32
FLOP_FWD, FLOP_BWD = 27, 52          # algorithmic FP32 flop per (Gaussian, point) pair, 3D
N_SM_LANES = 128                      # FP32 lanes per SM


def _args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-batch", type=int, default=16, help="batch slice timed on the host cores")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=None,
                    help="batch per GPU (default: the configuration's 32; smaller values are for profiler captures)")
    ap.add_argument("--relu-fit", choices=["fixed_point_only", "fixed_point_and_tree_hem"], default="fixed_point_only",
                    help="config 4: ReLU fitting strategy of the layers (the second one runs LBVH + BVH-MHEM in 3D)")
    ap.add_argument("--no-cuda-graph", action="store_true", help="config 4: launch the forward kernel by kernel")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiler captures)")
    ap.add_argument("--config", type=int, default=1, choices=[1, 2, 3, 4],
                    help="1 (default, the headline): 3D evaluation fwd+bwd; 2: 2D ReLU fit with BVH-MHEM reduction; "
                         "3: 2D convolution fitting layer; 4: 3D GMCN forward")
    return ap.parse_args()


def _measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "sm_max_mhz": 1965.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def _run(self):
        nv = self.nvml
        names = {}
        for n in dir(nv):
            if n.startswith("nvmlClocksEventReason") or n.startswith("nvmlClocksThrottleReason"):
                v = getattr(nv, n)
                if isinstance(v, int) and v != 0:
                    names.setdefault(v, n.replace("nvmlClocksEventReason", "").replace("nvmlClocksThrottleReason", ""))
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit and bin(bit).count("1") == 1:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.02)

    def start(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unsampled"]}
        s = sorted(self.samples)
        reasons = sorted(r for r in self.reasons if r not in ("None", "GpuIdle", "ApplicationsClocksSetting"))
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(s)}


def _repeat_for(fn, min_seconds=10.0, max_reps=1000):
    """Runs fn() until min_seconds of wall time have passed -> (repetitions, seconds)."""
    fn()                                  # page in / thread pool warm-up, not timed
    reps, t0 = 0, time.perf_counter()
    while True:
        fn()
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or reps >= max_reps:
            return reps, dt


def _cpu_baseline(cpu_batch):
    """Reference CPU algorithm (oracle restatement, fp32, OpenMP over query points) on a batch slice."""
    import synthetic_inputs as synthetic
    from oracle import cpu_oracle
    cpu_oracle.use_all_cores()
    m, x, g = synthetic.config1(n_batch=cpu_batch)
    m, x, g = m.numpy(), x.numpy(), g.numpy()
    cpu_oracle.eval_forward(m[:1, :1], x[:1, :1])   # page in / thread pool warm-up
    t0 = time.perf_counter()
    cpu_oracle.eval_forward(m, x)
    cpu_oracle.eval_backward(g, m, x)
    dt = time.perf_counter() - t0
    pairs = cpu_batch * L * G * N
    return {"value": pairs / dt, "unit": UNIT, "cores": cpu_oracle.num_threads(), "kind": "port",
            "sample": f"batch slice B={cpu_batch} of the same workload ({pairs} pairs, one fwd+bwd, {dt:.2f} s); "
                      "fp32, OpenMP over query points"}, dt


def run_reference(args, rank):
    if rank != 0:
        return
    times = []
    base = None
    for i in range(args.warmup + args.steps):
        base, dt = _cpu_baseline(args.cpu_batch)
        if i >= args.warmup:
            times.append(dt)
        if sum(times) > 120:     # keep the whole run within a few minutes
            break
    steps = len(times)
    pairs = args.cpu_batch * L * G * N
    value = pairs * steps / sum(times)
    base["value"] = value
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"config1 slice: 3D evaluate_inversed fwd+bwd, B={args.cpu_batch} L={L} G={G} N={N}"},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    _emit(line)


def _measure_fp32_peak(torch, dev):
    """FP32 FMA peak of this GPU in TFLOP/s: the library's probe kernel (FFMA chains only), best of 5 launches."""
    import ctypes
    from gmc import _native
    sink = torch.zeros(1, device=dev)
    flop = ctypes.c_double(0.0)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    best = 0.0
    for i in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _native.check(_native.lib.gmc_fp32_fma_probe(_native.ptr(sink), 4000, ctypes.byref(flop), stream), "fp32 probe")
        e1.record()
        torch.cuda.synchronize(dev)
        if i > 0:
            best = max(best, flop.value / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import gmc.mixture as gm
    from gmc import sharding
    import synthetic_inputs as synthetic
    import gmc.cpp.extensions.evaluate_inversed.evaluate_inversed as ev

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    # every rank owns its own batch shard (different seed per rank)
    B_PER_GPU = args.batch if args.batch is not None else globals()["B_PER_GPU"]
    m_h, x_h, g_h = synthetic.config1(n_batch=B_PER_GPU, seed=1001 + rank)
    m_h, x_h, g_h = m_h.pin_memory(), x_h.pin_memory(), g_h.pin_memory()
    m, x, g = m_h.to(dev), x_h.to(dev), g_h.to(dev)
    pairs_rank = B_PER_GPU * L * G * N
    gather = sharding.OutputGatherer(world, dev) if world > 1 else None

    def step(record=None):
        out = ev.parallel_forward(m, x)[0]
        if record is not None:
            record[1].record()
        if gather is not None:
            gather.start(out)          # side stream, overlaps the backward kernel
        gm_, gx_ = ev.parallel_backward(g, m, x, None, True, True)
        if gather is not None:
            gather.finish()
        if record is not None:
            record[2].record()
        return out, gm_, gx_

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else local_rank)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    for i in range(args.steps):
        evs[i][0].record()
        step(evs[i])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    total_ms = evs[0][0].elapsed_time(evs[-1][2])
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps

    # ---- end to end through the public API with host buffers ----
    out_h = torch.empty((B_PER_GPU, L, N), dtype=torch.float32).pin_memory()
    gm_h = torch.empty_like(m_h).pin_memory()
    gx_h = torch.empty_like(x_h).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        # the public host-buffer call: batch slices pipelined through copy-in / kernels / copy-out streams
        ev.host_forward_backward(m_h, x_h, g_h, out=out_h, grad_mixture=gm_h, grad_xes=gx_h)

    e2e_ms = float("nan")
    if not args.no_e2e:
        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps

    t = torch.tensor([total_ms, fwd_ms, bwd_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, fwd_ms, bwd_ms, e2e_ms = t.tolist()
    if rank != 0:
        return

    peaks, peaks_kind = _measured_peaks()
    n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
    sm_max_mhz = float(peaks.get("sm_max_mhz", 1965.0))
    fp32_nominal_tflops = n_sm * N_SM_LANES * 2 * sm_max_mhz * 1e6 / 1e12
    fp32_peak_tflops = _measure_fp32_peak(torch, dev)     # MEASURED_PEAKS.json has no FP32 entry: measured here
    ms_per_step = total_ms / args.steps
    value = world * pairs_rank / (ms_per_step * 1e-3)
    ach_bwd = FLOP_BWD * pairs_rank / (bwd_ms * 1e-3) / 1e12
    ach_fwd = FLOP_FWD * pairs_rank / (fwd_ms * 1e-3) / 1e12
    ach_all = (FLOP_FWD + FLOP_BWD) * pairs_rank / ((fwd_ms + bwd_ms) * 1e-3) / 1e12
    h2d = (m_h.numel() + x_h.numel() + g_h.numel()) * 4
    d2h = (out_h.numel() + gm_h.numel() + gx_h.numel()) * 4
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"config1: 3D evaluate_inversed fwd+bwd, B={B_PER_GPU}/GPU L={L} G={G} N={N} "
                               f"({pairs_rank} pairs per GPU and step)",
                   "l2": f"inputs ({(m_h.numel() + x_h.numel() + g_h.numel()) * 4 / 1e6:.0f} MB per step) "
                         "are larger than L2 (126 MB) at the default batch; no explicit flush",
                   "sharding": f"batch over {world} rank(s), all-gather of forward outputs overlapped with backward"},
        "roofline": {"bound": "fp32", "kernel": "eval_backward_kernel<3,2>", "achieved": ach_bwd,
                     "peak": fp32_peak_tflops, "unit": "TFLOP/s", "frac": ach_bwd / fp32_peak_tflops,
                     # dram__bytes_read+write of one launch: 32.79 MB captured by ncu at B=4 (profiles/), scaled by B/4
                     # because every byte of traffic belongs to one (batch, layer) mixture
                     "traffic": 32.79e6 * B_PER_GPU / 4, "traffic_unit": "bytes (ncu capture at B=4, scaled by B/4)",
                     "peak_source": "measured in this run: scalar FFMA chains (gmc_fp32_fma_probe, best of 5, CUDA events); "
                                    "MEASURED_PEAKS.json has no FP32 entry",
                     "peak_nominal": fp32_nominal_tflops, "frac_of_nominal": ach_bwd / fp32_nominal_tflops,
                     "peak_nominal_source": f"{n_sm} SMs x 128 lanes x 2 flop x {sm_max_mhz:.0f} MHz "
                                            f"(sm_max_mhz from {peaks_kind} MEASURED_PEAKS.json)",
                     "algorithmic_flop_per_pair": FLOP_BWD, "ms_per_launch": bwd_ms},
        "roofline_forward": {"bound": "fp32", "kernel": "eval_forward_kernel<3,8>", "achieved": ach_fwd,
                             "peak": fp32_peak_tflops, "unit": "TFLOP/s", "frac": ach_fwd / fp32_peak_tflops,
                             "algorithmic_flop_per_pair": FLOP_FWD, "ms_per_launch": fwd_ms},
        "roofline_fwd_bwd": {"bound": "fp32", "achieved": ach_all, "peak": fp32_peak_tflops, "unit": "TFLOP/s",
                             "frac": ach_all / fp32_peak_tflops, "frac_of_nominal": ach_all / fp32_nominal_tflops,
                             "algorithmic_flop_per_pair": FLOP_FWD + FLOP_BWD},
        "e2e": None if args.no_e2e else
               {"value": world * pairs_rank / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps},
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
    }
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"], _ = _cpu_baseline(args.cpu_batch)
    _emit(line)


# ---------------------------------------------------------------------------------------------------------------
# secondary configurations (2: ReLU fit + BVH-MHEM, 3: convolution fitting, 4: GMCN-3D forward)
# ---------------------------------------------------------------------------------------------------------------
def _gmcn3d(torch, model, fitting_method=None):
    """Network of configuration 4: conv 1->8 fit 64, 8->16 fit 32, 16->32 fit 16, 32->64 fit 8 (5-component kernels),
    integrate, linear layer to 10 logits; random initialisation, evaluation mode."""
    cfg = model.Config(n_dims=3)
    cfg.layers = [model.Layer(8, 1, 64, 64), model.Layer(16, 1, 32, 32), model.Layer(32, 1, 16, 16), model.Layer(64, 1, 8, 8)]
    if fitting_method is not None:
        cfg.relu_config.fitting_method = fitting_method
    torch.manual_seed(4)
    net = model.Net(config=cfg).eval()
    head = torch.nn.Linear(64, 10)
    return net, head


def _secondary_setup(args, rank, dev):
    """-> (metric, unit, units per step and rank, step(), host_inputs, workload text, algorithmic bytes, cpu_baseline())"""
    import torch
    import synthetic_inputs as synthetic
    import gmc.fitting as fitting
    if args.config == 2:
        n_batch = args.batch if args.batch is not None else 32
        m_h, c_h = synthetic.config2(n_batch=n_batch, seed=1002 + rank)
        m, c = m_h.to(dev), c_h.to(dev)
        cfg = fitting.Config(n_reduction=4)
        units = n_batch * 32 * 1024

        def step(inputs=None):
            mm, cc = (m, c) if inputs is None else inputs
            with torch.no_grad():
                return fitting.fixed_point_and_tree_hem(mm, cc, 64, cfg)[0]

        def cpu():
            from oracle import cpu_oracle
            cpu_oracle.use_all_cores()
            sample, _ = synthetic.config2(n_batch=32)
            flat = sample.numpy().reshape(-1, 1024, 7).copy()
            flat[..., 0] = abs(flat[..., 0]) + 0.01
            reps, dt = _repeat_for(lambda: cpu_oracle.mhem_fit_forward(flat, 64, 4))
            return {"value": reps * flat.shape[0] * 1024 / dt, "unit": "gaussians/s", "cores": cpu_oracle.num_threads(),
                    "kind": "port",
                    "sample": f"LBVH + BVH-MHEM fit of {flat.shape[0]} mixtures x 1024 Gaussians, {reps} passes "
                              f"({dt:.2f} s); the fixed-point evaluations are not included in the CPU figure"}
        # LBVH 56 B/Gaussian + MHEM per mixture 28672 + 2*128*(2G-1) + 1792 B (node attributes written and read once)
        alg_bytes = units * 56 + n_batch * 32 * (28672 + 2 * 128 * 2047 + 1792)
        return ("gaussians_per_s_relu_fit_bvh_mhem_2d", "gaussians/s", units, step, (m_h, c_h),
                f"config2: fixed_point_and_tree_hem, B={n_batch}/GPU L=32 G=1024 -> K=64, R=4", alg_bytes, cpu)
    if args.config == 3:
        import gmc.cpp.extensions.convolution_fitting.binding as cf
        n_batch = args.batch if args.batch is not None else 64
        d_h, k_h, K = synthetic.config3(n_batch=n_batch, seed=1003 + rank)
        d, k = d_h.to(dev), k_h.to(dev)
        units = n_batch * 16 * 5120

        def step(inputs=None):
            dd, kk = (d, k) if inputs is None else inputs
            return cf.forward(dd, kk, K)[0]

        def cpu():
            from oracle import cpu_oracle
            cpu_oracle.use_all_cores()
            sd, sk, _ = synthetic.config3(n_batch=64)
            sdn, skn = sd.numpy(), sk.numpy()
            reps, dt = _repeat_for(lambda: cpu_oracle.convolution_fitting_forward(sdn, skn, K))
            return {"value": reps * 64 * 16 * 5120 / dt, "unit": "product-gaussians/s", "cores": cpu_oracle.num_threads(),
                    "kind": "port",
                    "sample": f"the whole layer (1024 trees x 5120 products), {reps} passes ({dt:.2f} s)"}
        alg_bytes = (d_h.numel() + k_h.numel()) * 4 + n_batch * 16 * (5120 * 4 + 2 * K * 4 + K * 7 * 4 + K * 4 * 4)
        return ("product_gaussians_per_s_convolution_fitting_2d", "product-gaussians/s", units, step, (d_h, k_h),
                f"config3: convolution_fitting forward, B={n_batch}/GPU Cin=8 G=128 Cout=16 Gk=5 -> K=128 (T=5120)",
                alg_bytes, cpu)
    import gmc.model as model
    n_batch = args.batch if args.batch is not None else 256
    x_h = synthetic.config4_input(n_batch=n_batch, seed=1004 + rank)
    x = x_h.to(dev)
    net, head = _gmcn3d(torch, model, getattr(fitting, args.relu_fit))
    net, head = net.to(dev), head.to(dev)

    def eager(xx):
        with torch.no_grad():
            return head(net.features(xx))

    graphed = None
    if not args.no_cuda_graph:
        from gmc.cuda_graph import GraphedForward
        try:
            graphed = GraphedForward(eager, x)      # the whole forward pass as one graph launch
        except RuntimeError as err:                 # a strategy that synchronises with the host cannot be captured
            print(f"CUDA graph capture failed ({str(err).splitlines()[0]}); launching kernel by kernel", file=sys.stderr)
            torch.cuda.synchronize()
            graphed = None

    def step(inputs=None):
        xx = x if inputs is None else inputs[0]
        return graphed(xx) if graphed is not None else eager(xx)

    step.uncaptured = lambda: eager(x)      # the same launches outside the graph, for the launch count

    def cpu():
        from oracle import cpu_oracle
        cpu_oracle.use_all_cores()
        # dominant stage on the CPU: the four convolution-fitting layers on a batch slice (random data of the layer shapes)
        g = torch.Generator().manual_seed(1)
        layers = []
        for (cin, gcomp, cout, kfit) in ((1, 64, 8, 64), (8, 64, 16, 32), (16, 32, 32, 16), (32, 16, 64, 8)):
            cov, _ = synthetic.covariances_and_inverses((32, cin, gcomp), 3, 0.03, 0.15, g)
            data = synthetic.pack(torch.rand(32, cin, gcomp, generator=g), torch.rand(32, cin, gcomp, 3, generator=g) * 2 - 1, cov)
            kcov, _ = synthetic.covariances_and_inverses((cout, cin, 5), 3, 0.1, 0.4, g)
            kern = synthetic.pack(torch.randn(cout, cin, 5, generator=g) + 0.1, torch.randn(cout, cin, 5, 3, generator=g), kcov)
            layers.append((data.numpy(), kern.numpy(), kfit))

        def four_layers():
            for data, kern, kfit in layers:
                cpu_oracle.convolution_fitting_forward(data, kern, kfit)

        reps, dt = _repeat_for(four_layers)
        return {"value": reps * 32 / dt, "unit": "samples/s", "cores": cpu_oracle.num_threads(), "kind": "port",
                "sample": f"the four convolution-fitting layers only (the dominant stage) on 32 samples, {reps} passes "
                          f"({dt:.2f} s); ReLU fixed-point evaluations and normalisations are not included"}
    keys = n_batch * (8 * 320 + (16 + 32 + 64) * 2560)
    return ("samples_per_s_gmcn3d_forward", "samples/s", n_batch, step, (x_h,),
            f"config4: GMCN-3D forward, B={n_batch}/GPU, 64 input Gaussians, conv-fit layers 1->8->16->32->64 "
            f"(K=64/32/16/8, ReLU fit {args.relu_fit}), integrate, linear to 10 logits; "
            + ("one CUDA graph per forward" if graphed is not None else "kernel-by-kernel launches"),
            keys * 4 + n_batch * 64 * 13 * 4, cpu)


def run_secondary(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from gmc import sharding
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    metric, unit, units, step, host_inputs, workload, alg_bytes, cpu = _secondary_setup(args, rank, dev)
    host_inputs = tuple(t.pin_memory() for t in host_inputs)
    gather = sharding.OutputGatherer(world, dev) if world > 1 else None
    # kernels of this library per step (the library counts its launches; a graph replay repeats the captured ones)
    from gmc import _native
    launches_before = _native.lib.gmc_kernel_launch_count()
    getattr(step, "uncaptured", step)()
    launches_per_step = _native.lib.gmc_kernel_launch_count() - launches_before

    def full_step():
        out = step()
        if gather is not None:
            gather.start(out)
            gather.finish()
        return out

    for _ in range(max(args.warmup, 3)):
        full_step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    e0.record()
    for _ in range(args.steps):
        full_step()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps

    e2e_steps = max(3, min(args.steps, 20))
    out_h = None

    def e2e_step():
        nonlocal out_h
        dev_in = tuple(t.to(dev, non_blocking=True) for t in host_inputs)
        out = step(dev_in)
        if out_h is None:
            out_h = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        out_h.copy_(out, non_blocking=True)

    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    if rank != 0:
        return
    peaks, peaks_kind = _measured_peaks()
    hbm = float(peaks["hbm_gbs"])
    achieved = alg_bytes / (ms * 1e-3) / 1e9
    line = {"metric": metric, "value": world * units / (ms * 1e-3), "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload, "l2": "working set of a step is smaller than L2 for some stages; not flushed",
                       "sharding": f"batch over {world} rank(s)" + (", all-gather of outputs" if world > 1 else "")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                         "traffic": None, "algorithmic_bytes_per_step": alg_bytes,
                         "note": f"whole step against {peaks_kind} copy bandwidth; the stages are latency bound at these "
                                 "sizes, see profiles/"},
            "e2e": {"value": world * units / (e2e_ms * 1e-3), "unit": unit,
                    "h2d_bytes_per_step": sum(t.numel() * 4 for t in host_inputs),
                    "d2h_bytes_per_step": out_h.numel() * 4, "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": launches_per_step * args.steps, "clocks": clocks}
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu()
    _emit(line)


_RESULT_FD = None


def _emit(line):
    """Writes the one JSON line to the process's real stdout (see main)."""
    text = json.dumps(line) + "\n"
    if _RESULT_FD is None:
        sys.stdout.write(text)
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, text.encode())


def main():
    # Libraries (NCCL's version banner, for one) write to file descriptor 1. The JSON line must be the only thing on
    # stdout, so everything else that goes to descriptor 1 is sent to stderr and the line is written to the saved one.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    args = _args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.config == 1:
            run_ours(args, rank, world, local_rank)
        else:
            run_secondary(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
