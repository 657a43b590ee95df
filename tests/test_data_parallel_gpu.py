"""GPU, two ranks over NCCL (skipped with fewer than two devices): a data-parallel training step of Net.

Each rank runs forward + backward on its half of the batch and `sharding.all_reduce_gradients` sums the parameter
gradients; the result must equal the gradients of one GPU on the whole batch, and the two-optimiser step of the
reference's runners (src/modelnet_classification/main.py:111-124: loss optimiser, then weight-decay optimiser) must
leave both ranks with the parameters the single-GPU step produces. Ranks are child processes, one GPU each; NVLS is
switched off for the collective library and no kernel of this package reads peer memory.
"""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

from conftest import PKG, ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _build_net(device):
    import gmc.model as model
    import gmc.modules as modules
    cfg = model.Config(n_dims=2)
    cfg.layers = [model.Layer(4, 1, 12, 8), model.Layer(5, 1, 8, 6)]
    torch.manual_seed(3)
    net = model.Net(config=cfg)
    # evaluation-mode normalisations (no batch statistics, which would differ between a shard and the whole batch) and
    # a deterministic per-sample input normalisation (the default one draws random sample points)
    net.norm0 = torch.nn.Sequential(modules.CovScaleNorm(1, batch_norm=False))
    return net.to(device).eval()


def _inputs():
    import synthetic_inputs as synthetic
    x = synthetic.fit_target_2d(4, 1, 10, 77)
    x[..., 0] = x[..., 0].abs() + 0.2
    target = torch.tensor([1, 0, 3, 2])
    return x, target


def _loss(net, x, target):
    feats = net.features(x)                                   # [n, 5]
    return torch.nn.functional.nll_loss(torch.log_softmax(feats, dim=1), target, reduction="sum")


def _step(net, x, target, reduce_fn=None):
    kernel_optimiser = torch.optim.Adam(net.parameters(), lr=1e-3)
    decay_optimiser = torch.optim.SGD(net.parameters(), lr=1e-2)
    kernel_optimiser.zero_grad()
    _loss(net, x, target).backward()
    if reduce_fn is not None:
        reduce_fn(net)
    grads = {n: p.grad.detach().clone() for n, p in net.named_parameters() if p.grad is not None}
    kernel_optimiser.step()
    decay_optimiser.zero_grad()
    net.weight_decay_loss().backward()
    decay_optimiser.step()
    return grads


def _worker(rank, world, port, out_dir):
    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import datetime
    import torch.distributed as dist
    from gmc import sharding
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=60))
    try:
        net = _build_net(dev)
        x, target = _inputs()
        xs = sharding.shard_batch(x, world, rank).to(dev)
        ts = sharding.shard_batch(target, world, rank).to(dev)
        grads = _step(net, xs, ts, lambda m: sharding.all_reduce_gradients(m, average=False))
        torch.save({"grads": {k: v.cpu() for k, v in grads.items()},
                    "params": {k: v.detach().cpu() for k, v in net.named_parameters()}},
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_training_step_equals_the_single_gpu_step(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        if p.is_alive():
            p.kill()
            pytest.fail("worker did not finish")
        assert p.exitcode == 0
    net = _build_net(torch.device("cuda", 0))
    x, target = _inputs()
    grads = _step(net, x.cuda(), target.cuda())
    params = {k: v.detach().cpu() for k, v in net.named_parameters()}
    for r in range(2):
        got = torch.load(os.path.join(str(tmp_path), f"rank{r}.pt"))
        # parameters the loss does not reach get no gradient on one GPU and an all-zero one from the all-reduce
        assert set(grads) <= set(got["grads"])
        for name in set(got["grads"]) - set(grads):
            assert got["grads"][name].abs().max().item() == 0, name
        for name, g in grads.items():
            scale = max(g.abs().max().item(), 1e-12)
            err = (got["grads"][name] - g.cpu()).abs().max().item() / scale
            assert err < 1e-4, f"rank {r} gradient of {name}: rel {err:.2e}"
        for name, p in params.items():
            assert torch.allclose(got["params"][name], p, rtol=1e-5, atol=1e-6), f"rank {r} parameter {name}"
