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


def allreduce_time_constant_grads(module: torch.nn.Module, group=None, average: bool = False, one_shot=None) -> int:
    """``allreduce_gradients`` over the time-constant parameters of ``module`` (``one_shot``: a
    :class:`OneShotAllReduce` to use instead of the NCCL collective)."""
    params = time_constant_parameters(module)
    if one_shot is not None:
        return one_shot.allreduce_gradients(params, average=average)
    return allreduce_gradients(params, group=group, average=average)


class OneShotAllReduce:
    """Sum-allreduce of a small float vector between the GPUs of one node in ONE kernel launch per rank
    (``exb_allreduce_oneshot``): every rank publishes its vector in a buffer that all ranks have mapped over NVLink,
    signals its peers, waits -- bounded -- for theirs and adds all vectors in rank order with plain peer loads.

    For the few KB of time-constant gradients the NCCL collective of :func:`allreduce_gradients` is already cheap
    next to the kernels; this path saves the flatten / collective / scatter launches around it and gives every rank
    bit-identical sums.  It needs PyTorch's symmetric memory (CUDA peer mappings between the ranks of ``group``, all
    on one node).  Construction is collective (every rank of the group must take part) and synchronises; calls are
    collective too and are ordered on each rank's current stream.  If a peer does not arrive within the wait limit
    the result is NaN and ``sinabs_exodus_b200.device_status()`` raises.
    """

    def __init__(self, numel: int, device, group=None):
        import torch.distributed._symmetric_memory as symm
        from . import _lib
        if not dist.is_initialized():
            raise RuntimeError("OneShotAllReduce needs an initialised process group")
        group = dist.group.WORLD if group is None else group
        self.group = group
        self.numel = int(numel)
        self.device = torch.device(device)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 16:
            raise ValueError("at most 16 ranks")
        self._lib = _lib
        # data: two parities of `numel` floats; signals: two parities of `world` words, zero before the first call
        self.data = symm.empty(2 * self.numel, dtype=torch.float32, device=self.device)
        self.signals = symm.empty(2 * self.world, dtype=torch.int32, device=self.device)
        self.data.zero_()
        self.signals.zero_()
        self._data_handle = symm.rendezvous(self.data, group)
        self._signal_handle = symm.rendezvous(self.signals, group)
        self._data_ptrs = torch.tensor(list(self._data_handle.buffer_ptrs), dtype=torch.int64, device=self.device)
        self._signal_ptrs = torch.tensor(list(self._signal_handle.buffer_ptrs), dtype=torch.int64, device=self.device)
        self.epoch = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(group)        # nobody signals before everybody's words are zero

    def __call__(self, vector: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum of ``vector`` (float32, ``numel`` elements, on this rank's GPU) over the ranks."""
        if vector.numel() != self.numel:
            raise ValueError(f"expected {self.numel} elements, got {vector.numel()}")
        vector = vector.reshape(-1).contiguous()
        out = torch.empty_like(vector) if out is None else out
        self.epoch += 1
        self._lib.allreduce_oneshot(out, vector, self._data_ptrs, self._signal_ptrs, self.rank, self.world, self.epoch)
        return out

    def allreduce_gradients(self, params: Iterable[torch.nn.Parameter], average: bool = False) -> int:
        """The ``.grad`` of ``params`` (together ``numel`` floats) summed over the ranks, in place."""
        params = list(params)
        if not params:
            return 0
        flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).to(torch.float32)
                          for p in params]) if len(params) > 1 else \
            (params[0].grad if params[0].grad is not None else torch.zeros_like(params[0])).reshape(-1).to(torch.float32)
        total = self(flat)
        if average:
            total = total / self.world
        off = 0
        for p in params:
            n = p.numel()
            g = total[off:off + n].reshape(p.shape).to(p.dtype)
            if p.grad is None:
                p.grad = g.clone()
            else:
                p.grad.copy_(g)
            off += n
        return int(total.numel())
