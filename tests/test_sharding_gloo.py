"""CPU, world size 2 over gloo: batch sharding and the output all-gather of gmc.sharding, including a rank that
fails before the collective (host-side failure detection)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG, ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, mode, result_dir):
    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    import datetime
    from gmc import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        full = torch.arange(6 * 3 * 5, dtype=torch.float32).view(6, 3, 5)
        shard = sharding.shard_batch(full, world, rank)
        if mode == "gather":
            out = sharding.all_gather_batch(shard * 2.0)
            assert torch.equal(out, full * 2.0)
            g = sharding.OutputGatherer(world, torch.device("cpu"))
            g.start(shard + 1.0)
            assert torch.equal(g.finish(), full + 1.0)
            torch.save(torch.tensor(1), os.path.join(result_dir, f"ok{rank}"))
        elif mode == "grads":
            torch.manual_seed(0)
            lin = torch.nn.Linear(3, 2)
            x = torch.full((4, 3), float(rank + 1))
            lin(x).sum().backward()
            local = [p.grad.clone() for p in lin.parameters()]
            sharding.all_reduce_gradients(lin, average=True)
            # ranks fed x = 1 and x = 2: the weight gradient averages to 1.5 * 4, the bias gradient stays 4
            assert torch.allclose(lin.weight.grad, torch.full((2, 3), 6.0))
            assert torch.allclose(lin.bias.grad, local[1])
            torch.save(torch.tensor(1), os.path.join(result_dir, f"ok{rank}"))
        elif mode == "grads_missing":
            # rank 1 never touches the bias: its .grad stays None, yet both ranks must issue the same collective
            torch.manual_seed(0)
            lin = torch.nn.Linear(3, 2)
            x = torch.full((4, 3), float(rank + 1))
            if rank == 0:
                lin(x).sum().backward()
            else:
                (x @ lin.weight.t()).sum().backward()
                assert lin.bias.grad is None
            sharding.all_reduce_gradients(lin, average=False)
            assert torch.allclose(lin.weight.grad, torch.full((2, 3), 12.0))
            assert torch.allclose(lin.bias.grad, torch.full((2,), 4.0))
            torch.save(torch.tensor(1), os.path.join(result_dir, f"ok{rank}"))
        elif mode == "ragged":
            bad = shard if rank == 0 else shard[:1]
            try:
                sharding.all_gather_batch(bad)
            except RuntimeError as e:
                assert "equal shard shapes" in str(e)
                torch.save(torch.tensor(1), os.path.join(result_dir, f"ok{rank}"))
        elif mode == "rank_fails":
            if rank == 1:
                raise SystemExit(3)   # leaves before the collective, nothing in flight
            try:
                sharding.all_gather_batch(shard)
            except Exception:
                torch.save(torch.tensor(1), os.path.join(result_dir, f"ok{rank}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(mode, tmp_path, expect_ok):
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
        if p.is_alive():
            p.kill()
            pytest.fail("worker did not finish")
    for r in expect_ok:
        assert os.path.exists(os.path.join(str(tmp_path), f"ok{r}")), f"rank {r} did not reach its check ({mode})"


def test_shard_range_covers_batch():
    from gmc import sharding
    for n in (1, 5, 32, 33):
        for w in (1, 2, 3, 8):
            spans = [sharding.shard_range(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(e - s for s, e in spans) - min(e - s for s, e in spans) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def test_all_gather_two_ranks(tmp_path):
    _run("gather", tmp_path, (0, 1))


def test_gradient_all_reduce_two_ranks(tmp_path):
    _run("grads", tmp_path, (0, 1))


def test_gradient_all_reduce_when_one_rank_lacks_a_gradient(tmp_path):
    _run("grads_missing", tmp_path, (0, 1))


def test_unequal_shards_raise_on_every_rank(tmp_path):
    _run("ragged", tmp_path, (0, 1))


def test_surviving_rank_gets_an_error_when_its_peer_leaves(tmp_path):
    _run("rank_fails", tmp_path, (0,))
