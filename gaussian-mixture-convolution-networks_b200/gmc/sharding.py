"""Batch sharding across the GPUs of one machine (one process per GPU, torch.distributed).

Every operator of this package treats each (batch, layer) mixture independently, so the batch axis is split into
contiguous shards, one per rank, and the kernels run unchanged on each shard. The only inter-GPU step is an
all-gather of per-shard outputs (NCCL over NVLink when the tensors live on GPUs). Gathered data always lands in the
calling rank's own memory; no kernel of this package reads another GPU's memory.
"""
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n_batch: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [start, end) of the batch axis owned by `rank`; the first n_batch % world_size ranks get one more."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    base, extra = divmod(n_batch, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch(tensor: torch.Tensor, world_size: int, rank: int) -> torch.Tensor:
    """This rank's slice of a tensor whose first axis is the batch (a broadcast axis of extent one is kept whole)."""
    if tensor.shape[0] == 1:
        return tensor
    s, e = shard_range(tensor.shape[0], world_size, rank)
    return tensor[s:e]


def all_gather_batch(shard: torch.Tensor, group=None) -> torch.Tensor:
    """Concatenation of every rank's shard along the batch axis. Shards must have equal shapes (pad the batch to a
    multiple of the world size beforehand); unequal shards raise on every rank."""
    world = dist.get_world_size(group)
    shard = shard.contiguous()
    shapes = [None] * world
    dist.all_gather_object(shapes, tuple(shard.shape), group=group)
    if any(s != shapes[0] for s in shapes):
        raise RuntimeError(f"all_gather_batch needs equal shard shapes, got {shapes}")
    out = torch.empty((world * shard.shape[0], *shard.shape[1:]), dtype=shard.dtype, device=shard.device)
    dist.all_gather_into_tensor(out, shard, group=group)
    return out


class OutputGatherer:
    """Overlapped all-gather of one output tensor per step.

    start(shard) enqueues the collective behind the kernels already issued on the current stream and returns at
    once, so kernels launched afterwards (the backward pass) run while the gather is in flight; finish() makes the
    current stream wait for the gathered data. The gathered buffer is allocated once and reused."""

    def __init__(self, world_size: int, device: torch.device, group=None):
        self.world = world_size
        self.device = device
        self.group = group
        self.buffer: Optional[torch.Tensor] = None
        self._work = None

    def start(self, shard: torch.Tensor) -> None:
        shard = shard.contiguous()
        shape = (self.world * shard.shape[0], *shard.shape[1:])
        if self.buffer is None or tuple(self.buffer.shape) != shape or self.buffer.dtype != shard.dtype:
            self.buffer = torch.empty(shape, dtype=shard.dtype, device=self.device)
        self._work = dist.all_gather_into_tensor(self.buffer, shard, group=self.group, async_op=True)

    def finish(self) -> torch.Tensor:
        if self._work is not None:
            self._work.wait()
            self._work = None
        return self.buffer


def all_reduce_gradients(module: torch.nn.Module, group=None, average: bool = True) -> None:
    """Data-parallel training step glue: sums (or averages) the parameter gradients of `module` over all ranks, in
    one flattened collective. Kernel mixtures are small, so one bucket is enough."""
    # every rank must issue a collective of the same length: the list is built from requires_grad (identical on all
    # ranks), not from which gradients happen to exist on this rank; a missing gradient counts as zeros
    params = [p for p in module.parameters() if p.requires_grad]
    if not params:
        return
    flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in params])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    if average:
        flat /= dist.get_world_size(group)
    offset = 0
    for p in params:
        n = p.numel()
        piece = flat[offset:offset + n].view_as(p)
        if p.grad is None:
            p.grad = piece.clone()
        else:
            p.grad.copy_(piece)
        offset += n
