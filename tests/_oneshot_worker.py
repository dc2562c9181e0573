"""Worker of tests/test_gpu_multi.py: one rank of a small NCCL group that checks the one-shot peer-memory
allreduce against the NCCL collective.  Launched by torchrun, one process per GPU."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"]); local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import sinabs_exodus_b200 as ex
    from sinabs_exodus_b200.distributed import OneShotAllReduce, allreduce_gradients

    n = 2049                                     # the two time-constant vectors of a 1024-neuron layer, plus one
    red = OneShotAllReduce(n, dev)
    results = []
    for call in range(5):                        # both parities several times
        g = torch.Generator(device=dev).manual_seed(1000 * call + rank)
        v = torch.randn(n, device=dev, generator=g)
        got = red(v)
        want = v.clone()
        dist.all_reduce(want)
        torch.testing.assert_close(got, want, rtol=1e-6, atol=1e-6)
        results.append(got)
    # every rank holds the same bits
    gathered = [torch.empty_like(results[-1]) for _ in range(world)]
    dist.all_gather(gathered, results[-1])
    assert all(torch.equal(gathered[0], t) for t in gathered)
    # the gradient form: same result as the NCCL path
    torch.manual_seed(rank)
    pa = [torch.nn.Parameter(torch.zeros(1024, device=dev)), torch.nn.Parameter(torch.zeros(1, device=dev))]
    pb = [torch.nn.Parameter(torch.zeros(1024, device=dev)), torch.nn.Parameter(torch.zeros(1, device=dev))]
    for a, b in zip(pa, pb):
        a.grad = torch.randn_like(a); b.grad = a.grad.clone()
    red2 = OneShotAllReduce(1025, dev)
    red2.allreduce_gradients(pa)
    allreduce_gradients(pb)
    for a, b in zip(pa, pb):
        torch.testing.assert_close(a.grad, b.grad, rtol=1e-6, atol=1e-6)
    # the NCCL route with averaging, and with a rank that has no gradient for a parameter (it contributes zeros, so
    # that every rank issues the same collective)
    p1 = torch.nn.Parameter(torch.zeros(3, device=dev))
    p1.grad = torch.full((3,), float(rank + 1), device=dev)
    assert allreduce_gradients([p1], average=True) == 3
    torch.testing.assert_close(p1.grad, torch.full((3,), (world + 1) / 2.0, device=dev))
    p2 = [torch.nn.Parameter(torch.zeros(4, device=dev)), torch.nn.Parameter(torch.zeros(2, device=dev))]
    p2[0].grad = torch.ones(4, device=dev)
    p2[1].grad = None if rank == 0 else torch.ones(2, device=dev)
    assert allreduce_gradients(p2) == 6
    torch.testing.assert_close(p2[0].grad, torch.full((4,), float(world), device=dev))
    torch.testing.assert_close(p2[1].grad, torch.full((2,), float(world - 1), device=dev))
    ex.device_status()
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("ONESHOT_OK", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
