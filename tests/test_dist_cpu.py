"""Batch sharding and the time-constant gradient allreduce with two gloo ranks on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sinabs_exodus_b200 import distributed as exd
from sinabs_exodus_b200 import layers as el


def test_shard_bounds_cover_batch():
    for batch in (1, 7, 8, 33):
        for world in (1, 2, 3, 8):
            spans = [exd.shard_bounds(batch, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        exd.shard_bounds(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        full = torch.arange(5 * 3 * 4, dtype=torch.float32).reshape(5, 3, 4)
        mine = exd.shard_batch(full)
        layer = el.LIF(tau_mem=torch.tensor([10.0, 20.0, 30.0, 40.0]), tau_syn=5.0, train_alphas=True)
        params = exd.time_constant_parameters(layer)
        assert [n for n, _ in layer.named_parameters()] == ["alpha_mem", "alpha_syn"] and len(params) == 2
        # pretend backward produced the partial sums over this rank's batch slice
        layer.alpha_mem.grad = mine.sum((0, 1))
        if rank == 0:
            layer.alpha_syn.grad = mine.sum().reshape(())
        n = exd.allreduce_time_constant_grads(layer)
        q.put((rank, tuple(mine.shape), n, layer.alpha_mem.grad.clone(), layer.alpha_syn.grad.clone(),
               full.sum((0, 1)), full[:3].sum()))
    finally:
        dist.destroy_process_group()


def test_allreduce_two_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    shapes = {r: s for r, s, *_ in results}
    assert shapes == {0: (3, 3, 4), 1: (2, 3, 4)}
    for rank, shape, n, g_mem, g_syn, want_mem, want_syn_rank0 in results:
        assert n == 5
        torch.testing.assert_close(g_mem, want_mem)          # sum over the whole batch on every rank
        torch.testing.assert_close(g_syn, want_syn_rank0)    # rank 1 had no gradient: contributes zeros


def test_single_process_is_noop():
    layer = el.ExpLeak(tau_mem=10.0)
    layer.tau_mem.grad = torch.tensor(1.5)
    assert exd.allreduce_time_constant_grads(layer) == 0
    assert float(layer.tau_mem.grad) == 1.5
