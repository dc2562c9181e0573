"""Generates the golden vectors in this directory.  Needs a CUDA GPU and
``oracle/_ref/libexodus_ref.so`` (the reference's own kernels, built by
``oracle/build.py`` from the reference checkout).

    python tests/golden/make_golden.py <output-dir>

Each ``.npz`` holds the seeded inputs and what the reference kernels returned
for them, so that the CPU checker can be pinned against the real reference
without a GPU.  Inputs are regenerated from the seed by ``tests/_cases.py``;
they are stored as well so that the files stand alone.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle as orc  # noqa: E402
from oracle import ref_gpu  # noqa: E402
from tests._cases import lif_case  # noqa: E402


def cu(a):
    return torch.tensor(a, device="cuda")


def lif_golden(name, seed, N, T, surrogate, max_spikes=None, **kw):
    cs = lif_case(seed, N, T, **kw)
    lo = cs["theta_low"]
    s, v = ref_gpu.lif_forward(cu(cs["inp"]), cu(cs["v_init"]), cu(cs["alpha"]), cu(cs["subtract"]),
                               cu(cs["theta"]), None if lo is None else cu(lo), max_spikes)
    rng = np.random.default_rng(seed + 1000)
    go = rng.standard_normal((N, T)).astype(np.float32)
    gv = (0.1 * rng.standard_normal((N, T))).astype(np.float32)
    # surrogate evaluated by the checker's numpy formula on the reference's v_mem
    surr = surrogate(v.cpu().numpy(), cs["theta"][:, None])
    nc = (v.cpu().numpy() > lo[:, None]).astype(np.float32) if lo is not None else np.ones_like(surr)
    g = (surr * go).astype(np.float32) + gv
    v_post = (v - cu(cs["subtract"]).unsqueeze(1) * s)
    gi, ga = ref_gpu.lif_backward_kernels(cu(g), cu(surr), cu(nc), cu(cs["alpha"]), cu(cs["subtract"]), v_post,
                                          cu(cs["v_init"]))
    return name, dict(
        kind="lif", seed=seed, inp=cs["inp"], v_init=cs["v_init"], alpha=cs["alpha"], subtract=cs["subtract"],
        theta=cs["theta"], theta_low=lo if lo is not None else np.zeros(N, np.float32),
        apply_theta_low=lo is not None, max_spikes=-1 if max_spikes is None else max_spikes,
        go=go, gv=gv, surr=surr, not_clipped=nc, g=g, v_post=v_post.cpu().numpy(),
        ref_spikes=s.cpu().numpy(), ref_v_mem=v.cpu().numpy(), ref_grad_input=gi.cpu().numpy(),
        ref_grad_alpha=ga.cpu().numpy())


def leaky_golden(name, seed, N, T):
    rng = np.random.default_rng(seed)
    inp = rng.standard_normal((N, T)).astype(np.float32)
    go = rng.standard_normal((N, T)).astype(np.float32)
    alpha = rng.uniform(0.3, 1.0, N).astype(np.float32)
    v0 = rng.standard_normal(N).astype(np.float32)
    out = ref_gpu.leaky_forward(cu(inp), cu(v0), cu(alpha))
    gi, ga, _ = ref_gpu.leaky_backward(cu(go), cu(alpha), out, cu(v0))
    return name, dict(kind="leaky", seed=seed, inp=inp, go=go, alpha=alpha, v_init=v0,
                      ref_out=out.cpu().numpy(), ref_grad_input=gi.cpu().numpy(), ref_grad_alpha=ga.cpu().numpy())


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    cases = [
        lif_golden("lif_multispike_clamp", 101, 24, 60, orc.surrogate_single_exponential),
        lif_golden("lif_maxspike2_noclamp", 102, 17, 45,
                   lambda v, th: orc.surrogate_periodic_exponential(v, th), max_spikes=2, clamp=False),
        lif_golden("lif_singlespike_heaviside", 103, 9, 33,
                   lambda v, th: orc.surrogate_heaviside(v, th, 0.5), max_spikes=1, per_neuron=False,
                   subtract_given=False),
        lif_golden("lif_strong_input", 104, 8, 40, orc.surrogate_single_exponential, in_mean=1.5, in_std=1.0),
        leaky_golden("leaky_basic", 201, 20, 70),
    ]
    for name, data in cases:
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **data)
        print("wrote", name)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden"))
