"""Batch sharding across GPUs.

Every neuron instance is independent, so forward and input-gradient backward
need no communication: rank r simply owns a contiguous slice of the batch.  The
only exchange is for trainable time constants, whose gradients are sums over
the whole batch: after ``backward`` each rank holds the partial sum over its
slice, and one sum-allreduce of those few floats completes them.  All such
gradients of a model travel in ONE flat buffer and one collective, issued on
the current stream (NCCL over NVLink on GPUs; gloo on CPU tensors for tests).
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

TIME_CONSTANT_NAMES = ("tau_mem", "tau_syn", "alpha_mem", "alpha_syn")


def shard_bounds(batch: int, rank: int, world: int) -> Tuple[int, int]:
    """Half-open batch range of ``rank``; the first ``batch % world`` ranks get one item more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch(x: torch.Tensor, rank: Optional[int] = None, world: Optional[int] = None) -> torch.Tensor:
    """This rank's contiguous slice of a (batch, time, ...) tensor."""
    if rank is None:
        rank = dist.get_rank()
    if world is None:
        world = dist.get_world_size()
    lo, hi = shard_bounds(x.shape[0], rank, world)
    return x[lo:hi]


def time_constant_parameters(module: torch.nn.Module) -> List[torch.nn.Parameter]:
    """The trainable time-constant parameters (tau/alpha of membrane and synapse) of all layers in ``module``."""
    out = []
    for name, p in module.named_parameters():
        if name.rsplit(".", 1)[-1] in TIME_CONSTANT_NAMES and p.requires_grad:
            out.append(p)
    return out


def allreduce_gradients(params: Iterable[torch.nn.Parameter], group=None, average: bool = False) -> int:
    """Sum (or average) the ``.grad`` of ``params`` over all ranks with one collective.

    Returns the number of floats exchanged.  Parameters without a gradient on this
    rank contribute zeros so that every rank issues the same collective.
    """
    params = list(params)
    if not params or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return 0
    dev = params[0].device
    flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).to(torch.float32)
                      for p in params]).to(dev)
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    if average:
        flat /= dist.get_world_size(group)
    off = 0
    for p in params:
        n = p.numel()
        g = flat[off:off + n].reshape(p.shape).to(p.dtype)
        if p.grad is None:
            p.grad = g.clone()
        else:
            p.grad.copy_(g)
        off += n
    return int(flat.numel())


def allreduce_time_constant_grads(module: torch.nn.Module, group=None, average: bool = False) -> int:
    """``allreduce_gradients`` over the time-constant parameters of ``module``."""
    return allreduce_gradients(time_constant_parameters(module), group=group, average=average)
