"""Times the REFERENCE's own CUDA kernels (oracle/_ref/libexodus_ref.so) next to this library's
Functions on the same [N, T] problem, forward + backward, on one GPU.  Measurement helper; needs a GPU.

    python oracle/bench_reference_gpu.py [--workload c2|c3|c5] [--batch B]

The reference path is what its autograd Functions do (``sinabs/exodus/spike.py:193-289``,
``leaky.py:43-72``): kernels from the reference headers plus the PyTorch glue around them
(surrogate evaluation, clip mask, products).  Prints one JSON line.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import ref_gpu  # noqa: E402


def timed(fn, n):
    fn(); torch.cuda.synchronize()
    s = torch.cuda.Event(enable_timing=True); e = torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(n):
        fn()
    e.record(); torch.cuda.synchronize()
    return s.elapsed_time(e) / n


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c5"])
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--reps", type=int, default=3)
    args = ap.parse_args()
    if not ref_gpu.available():
        print(json.dumps({"unavailable": "oracle/_ref/libexodus_ref.so not built"})); return
    import sinabs_exodus_b200 as ex
    from sinabs_exodus_b200.compat import activation as sa
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(1)
    if args.workload == "c2":
        B, T, M = args.batch or 8, 300, 32 * 34 * 34
        N = B * M
        x = 0.4 * torch.poisson(torch.full((N, T), 0.1, device=dev), generator=g)
        fn, alpha_v = sa.Heaviside(), 1.0
    elif args.workload == "c5":
        B, T, M = args.batch or 1, 500, 64 ** 3
        N = B * M
        x = 0.05 * torch.empty(N, T, device=dev).normal_(0.25, 0.5, generator=g)
        fn, alpha_v = sa.SingleExponential(), float(torch.exp(torch.tensor(-1 / 20.0)))
    else:
        B, T, M = args.batch or 64, 4000, 512
        N = B * M
        x = torch.empty(N, T, device=dev).normal_(0, 1, generator=g)
    go = torch.empty(N, T, device=dev).normal_(0, 1, generator=g)
    z = torch.zeros(N, device=dev); one = torch.ones(N, device=dev)
    res = {"workload": args.workload, "N": N, "T": T}
    if args.workload in ("c2", "c5"):
        alpha = torch.full((N,), alpha_v, device=dev)

        def ref_step():
            s, v = ref_gpu.lif_forward(x, z, alpha, one, one)
            ref_gpu.integrate_and_fire_backward(go, torch.zeros_like(go), v, s, z, alpha, one, one, None, fn, False)

        xg = x.clone().requires_grad_(True)

        def our_step():
            xg.grad = None
            s, v = ex.IntegrateAndFire.apply(xg, alpha, z, one, one, None, fn, None)
            s.backward(go)
    else:
        alpha = torch.full((N,), float(torch.exp(torch.tensor(-1 / 50.0))), device=dev)

        def ref_step():
            out = ref_gpu.leaky_forward(x, z, alpha)
            ref_gpu.leaky_backward(go, alpha)

        xg = x.clone().requires_grad_(True)

        def our_step():
            xg.grad = None
            ex.LeakyIntegrator.apply(xg, alpha, z).backward(go)
    t_ref = timed(ref_step, args.reps)
    t_our = timed(our_step, max(args.reps, 10))
    res.update(reference_ms=t_ref, ours_nt_layout_ms=t_our, reference_nts_per_s=N * T / t_ref * 1e3,
               ours_nt_layout_nts_per_s=N * T / t_our * 1e3, speedup=t_ref / t_our)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
