"""Benchmark of the neuron hot path: neuron-timesteps per second, forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5] [--impl ours|reference]

One "step" is one forward + backward pass of one layer over one batch of synthetic input.  The
headline workload is ``c5``, the largest configuration that fits one GPU: a LIF layer on
``(32, 500, 64, 64, 64)`` per GPU (16.8 GB per tensor); ``c1`` .. ``c4`` are the other configurations
and are measured in the same run as short extra legs.  With N > 1 the script is launched by torchrun,
one rank per GPU; every rank owns its own batch shard of the same size (weak scaling) and the only
collective is the allreduce of time-constant gradients.

Rank 0 prints ONE JSON line:
* ``value``           whole-job neuron-timesteps/s with inputs resident in HBM, device-timed
                      (CUDA events, max over ranks)
* ``roofline``        the dominant kernel's algorithmic bytes / its event-timed duration against
                      the measured HBM copy bandwidth
* ``e2e``             the same metric through the public layer API with pinned HOST buffers: input
                      and upstream gradient copied in, spikes and input gradient copied out, every
                      step, inside the timed region (streamed through a fixed pinned staging ring)
* ``other_configs``   the other configurations, device-timed, each with its dominant kernel and
                      fraction of the copy peak; with N > 1 the synaptic configuration includes the
                      allreduce of its time-constant gradients, timed separately as well
* ``reference_cuda``  the reference project's own CUDA kernels (built from its sources into the
                      checker directory, when present) with the tensor glue of its autograd
                      Functions, on a batch slice of the same seeded input
* ``cpu_baseline``    a time-stepped PyTorch layer loop (the stand-in for the CPU layers of the
                      package the reference plugs into, which is not installed) on the host cores,
                      on a fixed sample

``--impl reference`` times that CPU loop alone, on the same workload definition.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch

METRIC = "neuron_timesteps_per_s_fwd_bwd"
UNIT = "nts/s"


# --------------------------------------------------------------------------
# workloads (shapes are per GPU)
# --------------------------------------------------------------------------
WORKLOADS = {
    "c1": dict(desc="LIF tau_mem=20 thr=1 subtract MultiSpike SingleExponential(0.5) min_v_mem=-1, "
                    "input (8,100,128) N(0.3,0.5) seed 0, grad ones",
               shape=(8, 100, 128), kind="lif", bytes_fwd=12, bytes_bwd=12),
    "c2": dict(desc="IAF thr=1 subtract MultiSpike Heaviside, input (32,300,32,34,34) = 0.4*Poisson(0.1) seed 1, "
                    "grad N(0,1)",
               shape=(32, 300, 32, 34, 34), kind="iaf", bytes_fwd=12, bytes_bwd=12),
    "c3": dict(desc="ExpLeak tau_mem=50 shared, input (64,4000,512) N(0,1) seed 2, grad N(0,1)",
               shape=(64, 4000, 512), kind="expleak", bytes_fwd=8, bytes_bwd=8),
    "c4": dict(desc="LIF tau_syn=10 + per-neuron tau_mem~U(10,40), train_alphas, SingleSpike, reset to zero, "
                    "PeriodicExponential, input (128,500,1024) N(0.2,0.6) seed 3, grad N(0,1)",
               shape=(128, 500, 1024), kind="lif_syn", bytes_fwd=16, bytes_bwd=16),
    "c5": dict(desc="LIF tau_mem=20 subtract MultiSpike SingleExponential, input (32,500,64,64,64) per GPU "
                    "N(0.25,0.5), grad N(0,1)",
               shape=(32, 500, 64, 64, 64), kind="lif5", bytes_fwd=12, bytes_bwd=12),
}


def make_layer(kind: str, neurons_shape, device):
    import sinabs_exodus_b200.layers as el
    from sinabs_exodus_b200.compat import activation as sa

    if kind == "lif":
        layer = el.LIF(tau_mem=20.0, spike_threshold=1.0, surrogate_grad_fn=sa.SingleExponential(grad_width=0.5),
                       min_v_mem=-1.0)
    elif kind == "iaf":
        layer = el.IAF(spike_threshold=1.0, surrogate_grad_fn=sa.Heaviside())
    elif kind == "expleak":
        layer = el.ExpLeak(tau_mem=50.0)
    elif kind == "lif_syn":
        g = torch.Generator().manual_seed(3)
        tau = 10.0 + 30.0 * torch.rand(neurons_shape, generator=g)
        layer = el.LIF(tau_mem=tau, tau_syn=10.0, train_alphas=True, spike_fn=sa.SingleSpike,
                       reset_fn=sa.MembraneReset(0.0), surrogate_grad_fn=sa.PeriodicExponential())
    elif kind == "lif5":
        layer = el.LIF(tau_mem=20.0, surrogate_grad_fn=sa.SingleExponential())
    else:
        raise ValueError(kind)
    return layer.to(device)


class FunctionArm(torch.nn.Module):
    """The drop-in autograd Functions on the reference's own [N,T] layout (rows = batch x neurons), with the
    workload's neuron model and no layer glue: `IntegrateAndFire.apply` / `LeakyIntegrator.apply`."""

    def __init__(self, kind: str, rows: int, device):
        super().__init__()
        import math
        from sinabs_exodus_b200.compat import activation as sa
        if kind == "lif_syn":
            raise SystemExit("--layout nt: the synaptic workload has no single [N,T] Function")
        self.kind = kind
        alpha = {"iaf": 1.0, "lif": math.exp(-1.0 / 20.0), "lif5": math.exp(-1.0 / 20.0),
                 "expleak": math.exp(-1.0 / 50.0)}[kind]
        self.alpha = torch.full((rows,), alpha, device=device)
        self.v0 = torch.zeros(rows, device=device)
        self.theta = torch.ones(rows, device=device)
        self.low = torch.full((rows,), -1.0, device=device) if kind == "lif" else None
        self.surrogate = {"iaf": sa.Heaviside(), "lif": sa.SingleExponential(grad_width=0.5),
                          "lif5": sa.SingleExponential(), "expleak": None}[kind]

    def reset_states(self):
        pass

    def forward(self, x):
        import sinabs_exodus_b200 as ex
        if self.kind == "expleak":
            return ex.LeakyIntegrator.apply(x, self.alpha, self.v0)
        spikes, _ = ex.IntegrateAndFire.apply(x, self.alpha, self.v0, self.theta, self.theta, self.low,
                                              self.surrogate, None)
        return spikes


def make_input(name: str, shape, device, rank: int, batch=None):
    """Seeded synthetic input and upstream gradient with the configuration's value distribution."""
    seed = {"c1": 0, "c2": 1, "c3": 2, "c4": 3, "c5": 100}[name] + (rank if name != "c5" else rank)
    shape = tuple(shape) if batch is None else (batch,) + tuple(shape[1:])
    g = torch.Generator(device=device).manual_seed(seed)
    if name == "c2":
        x = torch.empty(shape, device=device)
        for b in range(shape[0]):      # per item: keeps the temporary small
            x[b] = 0.4 * torch.poisson(torch.full(shape[1:], 0.1, device=device), generator=g)
    else:
        mean, std = {"c1": (0.3, 0.5), "c3": (0.0, 1.0), "c4": (0.2, 0.6), "c5": (0.25, 0.5)}[name]
        x = torch.empty(shape, device=device).normal_(mean, std, generator=g)
    g2 = torch.Generator(device=device).manual_seed(seed + 1000)
    grad = torch.ones(shape, device=device) if name == "c1" else torch.empty(shape, device=device).normal_(0, 1, generator=g2)
    return x, grad


# --------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a region runs."""

    FIELDS = ("uuid,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows = []
        self.proc = None
        try:
            uuid = torch.cuda.get_device_properties(device_index).uuid
            self.uuid = "GPU-" + str(uuid) if not str(uuid).startswith("GPU-") else str(uuid)
        except Exception:
            self.uuid = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), line.strip()))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        return self.window(None, None)

    def window(self, t0, t1):
        """Statistics of the samples read between the host times t0 and t1 (time.monotonic; None = no bound)."""
        sm, smax, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for stamp, row in list(self.rows):
            if (t0 is not None and stamp < t0) or (t1 is not None and stamp > t1):
                continue
            parts = [p.strip() for p in row.split(",")]
            if len(parts) < 8 or (self.uuid and parts[0] != self.uuid):
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val == "Active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------
# kernel event timing: wraps the C-ABI calls with CUDA events on the launch stream
# --------------------------------------------------------------------------
class KernelTimer:
    NAMES = ("lif_forward", "lif_backward", "leaky_forward", "leaky_backward", "leaky_forward_scan",
             "leaky_backward_scan", "lif_syn_forward", "lif_syn_backward", "lif_forward_ckpt", "lif_backward_ckpt")

    COUNTED = ("acc_finish", "allreduce_oneshot")     # small kernels of the library: counted, not timed

    def __init__(self):
        from sinabs_exodus_b200 import _lib
        self.lib = _lib
        self.orig = {n: getattr(_lib, n) for n in self.NAMES + self.COUNTED}
        self.events = {n: [] for n in self.NAMES}
        self.counted = 0
        self.enabled = False
        for n in self.NAMES:
            setattr(_lib, n, self._wrap(n))
        for n in self.COUNTED:
            setattr(_lib, n, self._count(n))

    def _wrap(self, name):
        orig = self.orig[name]

        def call(*args, **kwargs):
            if not self.enabled:
                return orig(*args, **kwargs)
            s = torch.cuda.Event(enable_timing=True); e = torch.cuda.Event(enable_timing=True)
            s.record()                       # torch's current stream == the stream the kernel is launched on
            res = orig(*args, **kwargs)
            e.record()
            self.events[name].append((s, e))
            return res
        return call

    def _count(self, name):
        orig = self.orig[name]

        def call(*args, **kwargs):
            if self.enabled:
                self.counted += 1
            return orig(*args, **kwargs)
        return call

    def launches(self):
        return sum(len(v) for v in self.events.values()) + self.counted

    def summary(self):
        out = {}
        for n, evs in self.events.items():
            if evs:
                ms = [s.elapsed_time(e) for s, e in evs]
                out[n] = {"launches": len(ms), "avg_ms": sum(ms) / len(ms), "min_ms": min(ms)}
        return out

    def reset(self):
        self.events = {n: [] for n in self.NAMES}
        self.counted = 0


# --------------------------------------------------------------------------
# CPU arm: time-stepped PyTorch layer loop on the host cores
# --------------------------------------------------------------------------
def cpu_step(name: str, kind: str, x: torch.Tensor, grad: torch.Tensor):
    """One forward+backward of the time-stepped PyTorch loop on CPU tensors (layer semantics of `kind`)."""
    from oracle.torch_loop import lif_loop
    from sinabs_exodus_b200.compat import activation as sa

    B, T = x.shape[:2]
    xr = x.reshape(B, T, -1).clone().requires_grad_(True)
    M = xr.shape[2]
    zeros = torch.zeros(B, M)
    one = torch.tensor(1.0)
    if kind == "lif":
        tau = torch.tensor(20.0, requires_grad=True)
        res = lif_loop(xr, torch.exp(-1 / tau), zeros, one, one, torch.tensor(-1.0), sa.SingleExponential(0.5), None,
                       norm_input=True)
        out = res["spikes"]
    elif kind == "iaf":
        res = lif_loop(xr, torch.tensor(1.0), zeros, one, one, None, sa.Heaviside(), None)
        out = res["spikes"]
    elif kind == "expleak":
        tau = torch.tensor(50.0, requires_grad=True)
        res = lif_loop(xr, torch.exp(-1 / tau), zeros, spiking=False, decay_early=False)
        out = res["v_mem_pre"]
    elif kind == "lif_syn":
        g = torch.Generator().manual_seed(3)
        a_mem = torch.exp(-1 / (10.0 + 30.0 * torch.rand(M, generator=g))).requires_grad_(True)
        a_syn = torch.exp(torch.tensor(-1 / 10.0)).requires_grad_(True)
        res = lif_loop(xr, a_mem, zeros, one, None, None, sa.PeriodicExponential(), 1, reset_value=0.0,
                       alpha_syn=a_syn, i_syn_init=zeros, norm_input=True, decay_early=True)
        out = res["spikes"]
    else:
        tau = torch.tensor(20.0, requires_grad=True)
        res = lif_loop(xr, torch.exp(-1 / tau), zeros, one, one, None, sa.SingleExponential(), None, norm_input=True)
        out = res["spikes"]
    out.backward(grad.reshape(B, T, -1))
    return xr.grad


# Fixed sample of each workload for the CPU legs: (batch items, neurons) of the workload's own time length.
# Sized for a few seconds per step on 16 host cores; the same in every run.
CPU_SAMPLE = {"c1": (8, 128), "c2": (8, 36992), "c3": (16, 512), "c4": (16, 1024), "c5": (1, 65536)}


def cpu_sample(name: str, wl: dict, steps: int, warmup: int):
    """Times `steps` CPU steps on the workload's fixed sample.  Returns (nts_per_s, sample description, cores, ms_per_step)."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    shape = wl["shape"]
    T = shape[1]
    b, m = CPU_SAMPLE[name]
    b = min(b, shape[0]); m = min(m, int(np.prod(shape[2:])))
    x, g = make_input(name, (b, T, m), "cpu", 0)
    for _ in range(warmup):
        cpu_step(name, wl["kind"], x, g)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(name, wl["kind"], x, g)
    dt = time.perf_counter() - t0
    nts = b * m * T * steps
    sample = (f"{steps} fwd+bwd steps of a time-stepped PyTorch loop on a fixed sample of {name}: "
              f"batch {b} x {m} neurons x {T} steps")
    return nts / dt, sample, cores, dt / steps * 1e3


def cpu_c_kernels_sample(name: str, wl: dict, budget_s: float):
    """Second CPU point: the C restatement of the reference's kernel loops (OpenMP over neurons), with the
    Function glue of the reference in numpy, on an [N,T] sample of the workload.  None for the synaptic
    workload (the reference has no single Function for it)."""
    from oracle import oracle as orc
    kind = wl["kind"]
    if kind == "lif_syn":
        return None
    shape = wl["shape"]
    T = shape[1]
    rows_all = shape[0] * int(np.prod(shape[2:]))
    rng = np.random.default_rng(0)

    def run(rows):
        if name == "c2":
            x = (0.4 * rng.poisson(0.1, (rows, T))).astype(np.float32)
        else:
            mean, std = {"c1": (0.3, 0.5), "c3": (0.0, 1.0), "c5": (0.25, 0.5)}[name]
            x = rng.normal(mean, std, (rows, T)).astype(np.float32)
        go = np.ones((rows, T), np.float32) if name == "c1" else rng.standard_normal((rows, T)).astype(np.float32)
        z = np.zeros(rows, np.float32)
        one = np.ones(rows, np.float32)
        t0 = time.perf_counter()
        if kind == "expleak":
            a = np.full(rows, np.exp(-1 / 50.0), np.float32)
            out = orc.leaky_forward(x, z, a)
            orc.leaky_integrator_backward(go, out, z, a, True)
        else:
            a = one if kind == "iaf" else np.full(rows, np.exp(-1 / 20.0), np.float32)
            low = np.full(rows, -1.0, np.float32) if kind == "lif" else None
            surr = {"iaf": lambda v, th: orc.surrogate_heaviside(v, th),
                    "lif": lambda v, th: orc.surrogate_single_exponential(v, th, 0.5),
                    "lif5": lambda v, th: orc.surrogate_single_exponential(v, th)}[kind]
            spikes, v = orc.lif_forward(x, z, a, one, one, low, None)
            orc.integrate_and_fire_backward(go, np.zeros_like(go), v, spikes, z, a, one, one, low, surr, kind != "iaf")
        return time.perf_counter() - t0

    rows = min(rows_all, 4096)
    dt = min(run(rows), run(rows))
    rows_fit = int(min(rows_all, max(rows, rows * (budget_s / 4.0) / dt)))
    dt = run(rows_fit)
    return {"value": rows_fit * T / dt, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
            "sample": f"C restatement of the reference kernel loops (OpenMP) + numpy Function glue, forward+backward "
                      f"on {rows_fit} rows x {T} steps of {name} in the reference's [N,T] layout"}


def stream_mix_ceilings(dev) -> dict:
    """What plain streaming kernels reach on this GPU for the read/write mixes of the two passes: one read and two
    writes per element (the forward: in -> spikes, v_mem) and two reads and one write (the backward: grad, v_mem ->
    grad_in).  Calibration only, with library elementwise kernels on 512 MB tensors: `torch.frexp` (one fp32 in, one
    fp32 and one int32 out) and `torch.add`.  DRAM turns around between reads and writes, so the ceiling of a mix is
    not that of a copy; the kernels' GB/s should be read against these as well as against the copy peak."""
    n = 1 << 27
    a = torch.randn(n, device=dev)
    b = torch.randn(n, device=dev)
    o1 = torch.empty(n, device=dev)
    o2 = torch.empty(n, device=dev, dtype=torch.int32)

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / reps * 1e-3

    t12 = timed(lambda: torch.frexp(a, out=(o1, o2)))
    t21 = timed(lambda: torch.add(a, b, out=o1))
    t11 = timed(lambda: o1.copy_(a))
    return {"1r2w_gbs": 12.0 * n / t12 / 1e9, "2r1w_gbs": 12.0 * n / t21 / 1e9, "copy_gbs": 8.0 * n / t11 / 1e9,
            "how": "torch.frexp / torch.add / copy_ on 2^27 fp32 elements, CUDA events, 20 repetitions"}


# --------------------------------------------------------------------------
def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (earlier pool measurement)"


def config_dict(name: str, wl: dict, world: int) -> dict:
    """The `config` object of the JSON line; the same for both arms."""
    shape = wl["shape"]
    nts = int(np.prod(shape))
    return {"workload": f"{name}: {wl['desc']}", "per_gpu_shape": list(shape),
            "l2": f"each tensor is {nts * 4 / 1e6:.0f} MB (L2 is 126 MB); no flush between steps",
            "parallelism": f"batch-sharded x{world}"}


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, sample, cores, ms = cpu_sample(args.workload, wl, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.workload, wl, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def kernel_bytes(kind: str) -> dict:
    """Algorithmic bytes per neuron-step of each entry point for a workload kind."""
    b = {"lif_forward": 12, "lif_backward": 12, "leaky_forward": 8, "leaky_backward": 8,
         "leaky_forward_scan": 8, "leaky_backward_scan": 8,
         # fused LIF + synapse: read in, write i_syn/spikes/v_mem; read grad, v_mem, i_syn, write grad_in
         "lif_syn_forward": 16, "lif_syn_backward": 16,
         # checkpointed pair: read in, write spikes + 1/8 state; read grad, in, 1/8 state, write grad_in
         "lif_forward_ckpt": 8.5, "lif_backward_ckpt": 12.5}
    if kind == "expleak":              # trainable tau: the alpha gradient reads the forward output
        b["leaky_backward"] = 12
        b["leaky_backward_scan"] = 12
    if kind == "lif_syn":              # two-stage route: alpha gradient reads i_syn, decay_early scale gradient reads the input
        b["leaky_backward"] = 16
    return b


def roofline_of(name: str, kind: str, kernels: dict, nts_step: int, peak: float, peak_src: str):
    """Roofline object for the dominant kernel (largest total time) of a timed region."""
    if not kernels:
        return None
    per = kernel_bytes(kind)
    dom = max(kernels, key=lambda k: kernels[k]["avg_ms"] * kernels[k]["launches"])
    bts = per[dom] * nts_step
    ach = bts / (kernels[dom]["avg_ms"] * 1e-3) / 1e9
    traffic = None
    try:      # DRAM bytes per neuron-step from the committed ncu capture of a small case, scaled to this launch
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            traffic = float(json.load(f)[name][dom]) * nts_step
    except Exception:
        traffic = None
    return {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
            "traffic": traffic, "peak_source": peak_src, "algorithmic_bytes_per_launch": bts,
            "avg_launch_ms": kernels[dom]["avg_ms"],
            "all_kernels": {k: dict(v, gbs=per[k] * nts_step / (v["avg_ms"] * 1e-3) / 1e9) for k, v in kernels.items()}}


class Workload:
    """Layer, resident input and upstream gradient of one configuration on this rank's GPU."""

    def __init__(self, name: str, wl: dict, dev, rank: int, layout: str = "btm"):
        import sinabs_exodus_b200 as ex
        from sinabs_exodus_b200 import distributed as exd
        self.name, self.wl, self.dev = name, wl, dev
        shape = wl["shape"]
        self.B, self.T = shape[0], shape[1]
        self.M = int(np.prod(shape[2:]))
        self.nts = self.B * self.T * self.M
        self.layer = make_layer(wl["kind"], shape[2:], dev)
        x, grad = make_input(name, shape, dev, rank)
        if layout == "nt":      # same values, rows = (batch item, neuron), time contiguous
            B, T, M = self.B, self.T, self.M
            x = x.reshape(B, T, M).transpose(1, 2).reshape(B * M, T).contiguous()
            grad = grad.reshape(B, T, M).transpose(1, 2).reshape(B * M, T).contiguous()
            self.layer = FunctionArm(wl["kind"], B * M, dev)
        self.x = x.requires_grad_(True)
        self.grad = grad
        self.tc_params = exd.time_constant_parameters(self.layer)
        self.collective_events = []

    def step(self, world: int = 1, time_collective: bool = False):
        from sinabs_exodus_b200 import distributed as exd
        self.layer.zero_grad(set_to_none=True)
        self.x.grad = None
        self.layer.reset_states()
        out = self.layer(self.x)
        out.backward(self.grad)
        if world > 1 and self.tc_params:
            if time_collective:
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                e0.record()
                exd.allreduce_gradients(self.tc_params)
                e1.record()
                self.collective_events.append((e0, e1))
            else:
                exd.allreduce_gradients(self.tc_params)
        return out


def timed_steps(fn, steps: int, world: int, dev):
    """K calls of fn between barrier + synchronize on both sides, CUDA events, max over ranks.  Returns ms in total."""
    import torch.distributed as dist
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev0 = torch.cuda.Event(enable_timing=True); ev1 = torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        fn()
    ev1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def measure_other(name: str, timer: KernelTimer, dev, rank: int, world: int, steps: int, warmup: int, peak: float,
                  peak_src: str):
    """Short device-timed run of another configuration (eager layer API; c1 also as one CUDA graph)."""
    import sinabs_exodus_b200 as ex
    wl = dict(WORKLOADS[name])
    w = Workload(name, wl, dev, rank)
    for _ in range(warmup):
        w.step(world)
    torch.cuda.synchronize()
    # Step time first, with nothing else on the stream: sub-millisecond steps are bound by the host's launch path, and
    # the two event records around every kernel of the second pass would add to exactly that.  Such steps are also
    # timed over more repetitions.
    small = w.nts < (1 << 28)
    ksteps = steps
    if small:
        steps = max(steps, 50)
        for _ in range(10):
            w.step(world)
    ms = timed_steps(lambda: w.step(world), steps, world, dev)
    timer.reset()
    timer.enabled = True
    timed_steps(lambda: w.step(world, time_collective=True), ksteps, world, dev)
    timer.enabled = False
    kernels = timer.summary()
    launches = timer.launches()
    step_bytes = (wl["bytes_fwd"] + wl["bytes_bwd"]) * w.nts
    res = {"workload": f"{name}: {wl['desc']}", "per_gpu_shape": list(wl["shape"]), "steps": steps, "warmup": warmup,
           "ms_per_step": ms / steps, "value": w.nts * world * steps / (ms * 1e-3), "unit": UNIT,
           "launches_per_step": launches / ksteps,
           "step_fraction_of_hbm_roofline": (step_bytes / (ms / steps * 1e-3) / 1e9) / peak,
           "roofline": roofline_of(name, wl["kind"], kernels, w.nts, peak, peak_src)}
    if w.collective_events:
        c_ms = [a.elapsed_time(b) for a, b in w.collective_events]
        res["collective"] = {"what": "sum-allreduce of the time-constant gradients (NCCL, one flat buffer), inside the timed region",
                             "floats": int(sum(p.numel() for p in w.tc_params)), "avg_ms": sum(c_ms) / len(c_ms),
                             "calls": len(c_ms)}
        # The exchange alone, GPU otherwise idle, both ways on equal footing (these small calls are bound by their
        # host path, which is what they cost a step that is itself host-bound): the NCCL route of
        # distributed.allreduce_gradients (flatten, collective, scatter) and the one-kernel route over peer-mapped
        # memory (exb_allreduce_oneshot).
        def alone(fn, reps=20):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            import torch.distributed as dist
            dist.barrier()
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / reps
        from sinabs_exodus_b200 import distributed as exd
        res["collective"]["nccl_alone_avg_ms"] = alone(lambda: exd.allreduce_gradients(w.tc_params))
        one, why = None, ""
        try:
            one = exd.OneShotAllReduce(int(sum(p.numel() for p in w.tc_params)), dev)
        except Exception as exc:
            why = f"{type(exc).__name__}: {str(exc)[:160]}"
        import torch.distributed as dist
        agreed = torch.tensor([1 if one is not None else 0], device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)        # every rank times it, or none does (the calls are collective)
        if int(agreed.item()) == 1:
            try:
                res["collective"]["one_shot_alone_avg_ms"] = alone(lambda: one.allreduce_gradients(w.tc_params))
                ex._lib.device_status(dev)
            except Exception as exc:
                res["collective"]["one_shot_unavailable"] = f"{type(exc).__name__}: {str(exc)[:160]}"
        else:
            res["collective"]["one_shot_unavailable"] = why or "not available on another rank"
    if name == "c1":
        # backward in the calling thread: no hand-over to PyTorch's autograd thread
        prev = torch.autograd.is_multithreading_enabled()
        torch.autograd.set_multithreading_enabled(False)
        try:
            for _ in range(10):
                w.step(world)
            sms = timed_steps(lambda: w.step(world), steps, world, dev)
            res["single_thread_autograd"] = {"ms_per_step": sms / steps, "value": w.nts * world * steps / (sms * 1e-3)}
        finally:
            torch.autograd.set_multithreading_enabled(prev)
    if name in ("c1", "c3", "c4") and not (world > 1 and w.tc_params):
        # the same step captured once as a CUDA graph: what is left when the per-step host work is taken out
        try:
            graphed = ex.GraphedStep(w.layer, w.x.detach(), w.grad, carry_state=False, input_grad=True)
            for _ in range(3):
                graphed.replay()
            gms = timed_steps(graphed.replay, steps, world, dev)
            res["cuda_graph"] = {"ms_per_step": gms / steps, "value": w.nts * world * steps / (gms * 1e-3),
                                 "step_fraction_of_hbm_roofline": (step_bytes / (gms / steps * 1e-3) / 1e9) / peak}
            del graphed
        except Exception as exc:
            res["cuda_graph"] = {"unavailable": str(exc)[:200]}
    del w
    torch.cuda.empty_cache()
    return res


# Batch items of each workload given to the reference's kernels (its backward is O(T^2) per neuron and its
# Function glue keeps about ten [N,T] tensors alive).
REFERENCE_CUDA_BATCH = {"c2": 8, "c3": 64, "c5": 4}


def reference_cuda(name: str, wl: dict, dev, reps: int = 3):
    """The reference project's own CUDA kernels (oracle/_ref, built from its sources where they are present) with
    the tensor glue of its autograd Functions (sinabs/exodus/spike.py:193-289, leaky.py:43-72), forward + backward
    in its [N,T] layout, on a batch slice of the workload's seeded input.  A baseline, never the product path."""
    from oracle import ref_gpu
    from sinabs_exodus_b200.compat import activation as sa
    if not ref_gpu.available():
        return {"unavailable": "the reference kernels are not built here (no reference checkout at build time)"}
    if name not in REFERENCE_CUDA_BATCH:
        return {"unavailable": "the reference has no kernel for this configuration (reset to zero; fused synapse)"
                if name == "c4" else "not measured"}
    kind = wl["kind"]
    shape = wl["shape"]
    B = min(REFERENCE_CUDA_BATCH[name], shape[0])
    T = shape[1]
    M = int(np.prod(shape[2:]))
    N = B * M
    x, go = make_input(name, shape, dev, 0, batch=B)
    to_nt = lambda t: t.reshape(B, T, M).transpose(1, 2).reshape(N, T).contiguous()
    x, go = to_nt(x), to_nt(go)
    z = torch.zeros(N, device=dev); one = torch.ones(N, device=dev)
    note = ""
    if kind == "expleak":
        alpha = torch.full((N,), float(np.exp(-1 / 50.0)), device=dev)

        def step():
            out = ref_gpu.leaky_forward(x, z, alpha)
            ref_gpu.leaky_backward(go, alpha, out, z)          # tau is trainable: alpha gradient included
    else:
        if kind == "iaf":
            alpha, fn, low = one, sa.Heaviside(), None
        else:
            a = float(np.exp(-1 / 20.0))
            alpha = torch.full((N,), a, device=dev)
            x = (1.0 - a) * x                                  # layers/lif.py:206-209 (norm_input), done by the layer
            fn = sa.SingleExponential(0.5) if kind == "lif" else sa.SingleExponential()
            low = -one if kind == "lif" else None
            note = "; input pre-multiplied by 1 - alpha as the reference layer's norm_input does"
        gv = torch.zeros_like(go)

        def step():
            s, v = ref_gpu.lif_forward(x, z, alpha, one, one, low)
            ref_gpu.integrate_and_fire_backward(go, gv, v, s, z, alpha, one, one, low, fn, kind != "iaf")
    step()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    return {"value": N * T / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "batch": B, "rows": N, "steps_timed": reps,
            "what": "reference CUDA kernels (lifForward/lifBackward/lifBackwardAlpha or leakyForward/leakyBackward/"
                    "leakyBackwardAlpha, compiled for sm_100a from the reference sources) + the PyTorch glue of the "
                    f"reference Functions, [N,T] layout, batch {B} of {name}" + note}


def run_e2e(w: Workload, world: int, args, timer: KernelTimer):
    """The metric through the public layer API with pinned host buffers.  Every step copies the whole input and the
    whole upstream gradient from host memory and the whole output and input gradient back, in micro-batches of batch
    items through a FIXED pinned staging ring (a few slots per direction, reused round robin: every byte still crosses
    the bus every step, but a rank pins a few GB instead of four full tensors).  Copy-in of micro-batch i+1, the layer
    call on i and the copy-out of i-1 run on three streams."""
    from sinabs_exodus_b200 import distributed as exd
    import torch.distributed as dist
    dev = w.dev
    shape = w.wl["shape"]
    B = w.B
    item_bytes = w.T * w.M * 4
    # micro-batches of whole batch items, about 128 MB per tensor each (one item if an item is larger)
    per_mb = max(1, min(B, int((128 << 20) // item_bytes)))
    nmb = (B + per_mb - 1) // per_mb
    if args.e2e_microbatches:
        nmb = max(1, min(args.e2e_microbatches, B))
    bounds = [exd.shard_bounds(B, i, nmb) for i in range(nmb)]
    mb_items = max(hi - lo for lo, hi in bounds)
    host_slots = max(2, min(nmb, args.e2e_host_slots))
    dev_slots = max(2, min(nmb, 3))
    mb_shape = (mb_items,) + tuple(shape[1:])
    pin = lambda: torch.empty(mb_shape, pin_memory=True)
    xh = [pin() for _ in range(host_slots)]; gh = [pin() for _ in range(host_slots)]
    oh = [pin() for _ in range(host_slots)]; gih = [pin() for _ in range(host_slots)]
    gen = torch.Generator().manual_seed(1234)
    for t in xh:
        t.copy_(w.x.detach()[:mb_items].reshape(mb_shape) if w.x.shape[0] >= mb_items else torch.randn(mb_shape, generator=gen))
    for t in gh:
        t.copy_(w.grad[:mb_items].reshape(mb_shape))
    xd = [torch.empty(mb_shape, device=dev, requires_grad=True) for _ in range(dev_slots)]
    gd = [torch.empty(mb_shape, device=dev) for _ in range(dev_slots)]
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_main = torch.cuda.current_stream(dev)
    layer = w.layer
    done = [None] * dev_slots          # event: the layer call that used device slot s has finished

    def e2e_step():
        layer.zero_grad(set_to_none=True)
        s_in.wait_stream(s_out)             # host slots of the previous step are free again
        for i, (lo, hi) in enumerate(bounds):
            n = hi - lo
            ds, hs = i % dev_slots, i % host_slots
            with torch.cuda.stream(s_in), torch.no_grad():
                if done[ds] is not None:
                    s_in.wait_event(done[ds])
                xd[ds].grad = None
                xd[ds][:n].copy_(xh[hs][:n], non_blocking=True)
                gd[ds][:n].copy_(gh[hs][:n], non_blocking=True)
                ev = torch.cuda.Event(); ev.record(s_in)
            s_main.wait_event(ev)
            layer.reset_states()
            xin = xd[ds] if n == mb_items else xd[ds][:n]
            out = layer(xin)
            out.backward(gd[ds][:n])
            gin = xd[ds].grad
            ev2 = torch.cuda.Event(); ev2.record(s_main)
            done[ds] = ev2
            s_out.wait_event(ev2)
            with torch.cuda.stream(s_out):
                oh[hs][:n].copy_(out.detach(), non_blocking=True)
                gih[hs][:n].copy_(gin[:n], non_blocking=True)
            out.record_stream(s_out); gin.record_stream(s_out)
        if world > 1 and w.tc_params:
            exd.allreduce_gradients(w.tc_params)
        s_main.wait_stream(s_out)           # the step ends when its results are in host memory

    k_e2e = max(3, min(args.steps, args.e2e_steps))
    for _ in range(2):
        e2e_step()
    ms = timed_steps(e2e_step, k_e2e, world, dev)
    bytes_t = w.nts * 4
    pinned = 4 * host_slots * int(np.prod(mb_shape)) * 4
    return {"value": w.nts * world * k_e2e / (ms * 1e-3), "unit": UNIT,
            "h2d_bytes_per_step": 2 * bytes_t, "d2h_bytes_per_step": 2 * bytes_t, "steps": k_e2e,
            "ms_per_step": ms / k_e2e, "microbatches": nmb, "pinned_staging_bytes": pinned,
            "what": "layer forward+backward; input and upstream gradient copied from pinned host memory, "
                    "spikes/output and input gradient copied back, every step; the batch is streamed in "
                    "micro-batches through a fixed pinned staging ring so that copy-in, kernels and copy-out overlap"}


def run_ours(args, wl):
    import torch.distributed as dist
    import sinabs_exodus_b200 as ex

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ex._lib.load()
    peak, peak_src = measured_peak_gbs()

    name = args.workload
    w = Workload(name, wl, dev, rank, args.layout)
    if args.layout == "nt":
        args.no_e2e = True
    if args.recompute:
        w.layer.set_backward_recompute(True, always=True)
    timer = KernelTimer()
    sampler = ClockSampler(local) if rank == 0 else None      # started early: nvidia-smi takes a moment to deliver
    if sampler:
        sampler.start()
    for _ in range(args.warmup):
        w.step(world)
    torch.cuda.synchronize()
    timer.enabled = True            # the library's launches in one eager step (a captured step replays the same ones)
    w.step(world)
    timer.enabled = False
    launches_per_step = timer.launches()
    timer.reset()
    torch.cuda.synchronize()

    run_step = lambda: w.step(world)
    if args.cuda_graph:
        # Whole step (state reset, forward, backward) captured once and replayed: removes the per-step
        # host work, which dominates when the kernels take only tens of microseconds.
        if world > 1 and w.tc_params:
            raise SystemExit("--cuda-graph is for single-process runs (the allreduce is issued from the host)")
        graphed = ex.GraphedStep(w.layer, w.x.detach(), w.grad, carry_state=False, input_grad=True)
        run_step = graphed.replay
        for _ in range(3):
            run_step()
        torch.cuda.synchronize()

    # ---- timed region: K steps, device-timed, barrier + synchronize on both sides
    t_region0 = time.monotonic()
    if w.nts >= (1 << 28):
        timer.enabled = True
        ms_total = timed_steps(run_step, args.steps, world, dev)
        timer.enabled = False
        launches = timer.launches()
    else:
        # A sub-millisecond step is bound by the host's launch path: the two event records around every kernel
        # would add to exactly that, so the kernels are timed in a second pass of the same steps and the launch
        # count of that pass stands for the timed one (the same calls are made).
        ms_total = timed_steps(run_step, args.steps, world, dev)
        timer.enabled = True
        timed_steps(run_step, args.steps, world, dev)
        timer.enabled = False
        launches = timer.launches()
    kernels = timer.summary()
    t_region1 = time.monotonic()
    if args.cuda_graph:
        launches = launches_per_step * args.steps      # replays do not pass through the wrappers
    value = w.nts * world * args.steps / (ms_total * 1e-3)

    # ---- the same step without the v_mem tensor (layer.set_backward_recompute): extra key, not the headline
    recompute = None
    if (not args.lean and not args.cuda_graph and args.layout == "btm" and wl["kind"] in ("lif", "iaf", "lif5")
            and hasattr(w.layer, "set_backward_recompute") and w.nts >= (1 << 28)):
        w.layer.set_backward_recompute(True, always=True)
        try:
            for _ in range(3):
                w.step(world)
            timer.reset()
            timer.enabled = True
            rsteps = max(3, min(args.steps, 10))
            rms = timed_steps(run_step, rsteps, world, dev)
            timer.enabled = False
            rk = timer.summary()
            per = kernel_bytes(wl["kind"])
            recompute = {
                "what": "layer.set_backward_recompute(True): the forward writes spikes and one checkpoint of the state per "
                        "8 steps instead of v_mem, the backward rebuilds v_mem from the input and the checkpoints "
                        "(bit-identical gradients); 8.5 + 12.5 = 21 bytes per neuron-step instead of 24",
                "steps": rsteps, "ms_per_step": rms / rsteps, "value": w.nts * world * rsteps / (rms * 1e-3), "unit": UNIT,
                "kernels": {k: dict(v, gbs=per[k] * w.nts / (v["avg_ms"] * 1e-3) / 1e9,
                                    bytes_per_neuron_step=per[k]) for k, v in rk.items()}}
        finally:
            w.layer.set_backward_recompute(False)
            timer.reset()

    # ---- forward passes that nobody differentiates (torch.no_grad, no recording): spikes only, as float and as bytes
    inference = None
    if (not args.lean and not args.cuda_graph and args.layout == "btm" and wl["kind"] in ("lif", "iaf", "lif5")):
        xin = w.x.detach()

        def infer():
            w.layer.reset_states()
            w.layer(xin)
        inference = {"what": "layer forward under torch.no_grad() without record_states: no v_mem tensor is written"}
        isteps = max(3, min(args.steps, 10))
        with torch.no_grad():
            for key, dtype, bytes_nts in (("float32_spikes", torch.float32, 8), ("uint8_spikes", torch.uint8, 5)):
                w.layer.set_spike_output(dtype, saturate=True)
                try:
                    for _ in range(3):
                        infer()
                    ims = timed_steps(infer, isteps, world, dev)
                    inference[key] = {"ms_per_forward": ims / isteps, "value": w.nts * world * isteps / (ims * 1e-3),
                                      "unit": "nts/s (forward only)", "bytes_per_neuron_step": bytes_nts,
                                      "gbs": bytes_nts * w.nts / (ims / isteps * 1e-3) / 1e9}
                finally:
                    w.layer.set_spike_output(torch.float32)
        torch.cuda.empty_cache()

    # ---- end to end with host buffers (public layer API; copies inside the timed region)
    e2e = None
    if not args.no_e2e:
        timer.reset()
        t_e2e0 = time.monotonic()
        e2e = run_e2e(w, world, args, timer)
        if sampler:
            e2e["clocks"] = sampler.window(t_e2e0, time.monotonic())
    # Clocks: the samples that fell into the timed region; a region too short for the 100 ms sampling period to
    # give at least three (the default run of the largest configuration lasts 0.3 s) takes the whole run instead
    # -- warm-up, timed region and the extra measurements, all of them kernels of this library under load.
    clocks = None
    if sampler:
        whole = sampler.stop()
        clocks = sampler.window(t_region0, t_region1)
        clocks["window"] = "timed region"
        if (clocks.get("samples") or 0) < 3:
            clocks = dict(whole, window="whole run (the timed region held fewer than 3 samples)")

    roof = roofline_of(name, wl["kind"], kernels, w.nts, peak, peak_src) if rank == 0 else None
    step_bytes = (wl["bytes_fwd"] + wl["bytes_bwd"]) * w.nts
    nts_step = w.nts
    del w
    torch.cuda.empty_cache()

    # ---- the other configurations, device-timed (every rank takes part: c4 has a collective)
    others = None
    if not args.no_others:
        others = {}
        for other in ("c1", "c2", "c3", "c4", "c5"):
            if other == name or (other == "c5" and name != "c5"):
                continue
            try:
                others[other] = measure_other(other, timer, dev, rank, world, args.other_steps, 3, peak, peak_src)
            except Exception as exc:      # an extra leg must not take the headline down
                others[other] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
                torch.cuda.empty_cache()

    mix = ref_cuda = cpu = None
    if rank == 0:
        if not args.no_mix:
            try:
                mix = stream_mix_ceilings(dev)
            except Exception as exc:
                mix = {"unavailable": str(exc)[:200]}
        if world == 1 and not args.no_reference_cuda:
            ref_cuda = {}
            for n in dict.fromkeys([name, "c2", "c3"]):
                try:
                    ref_cuda[n] = reference_cuda(n, dict(WORKLOADS[n]) if n != name else wl, dev)
                except Exception as exc:
                    ref_cuda[n] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
                torch.cuda.empty_cache()
        if world == 1 and not args.no_cpu:
            v, sample, cores, _ = cpu_sample(name, wl, 3, 1)
            cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
            try:
                cpu["c_kernels"] = cpu_c_kernels_sample(name, wl, 6.0)
            except Exception as exc:      # the checker library is optional for this extra figure
                cpu["c_kernels"] = {"unavailable": str(exc)[:200]}
        config = config_dict(name, wl, world)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config,
            "run": {"api": "sinabs_exodus_b200.layers" if args.layout == "btm"
                    else "IntegrateAndFire / LeakyIntegrator Functions on [N,T] (no layer glue)",
                    "cuda_graph": bool(args.cuda_graph),
                    "autograd": "single-threaded" if args.single_thread_autograd else "default (backward on PyTorch's autograd thread)"},
            "step_fraction_of_hbm_roofline": (step_bytes / (ms_total / args.steps * 1e-3) / 1e9) / peak,
            "roofline": roof, "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "recompute": recompute, "inference": inference,
            "cpu_baseline": cpu, "other_configs": others, "reference_cuda": ref_cuda, "stream_mix_ceilings": mix,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=None, help="override the per-GPU batch size (profiling small cases)")
    ap.add_argument("--shape", default=None,
                    help="override the per-GPU input shape, e.g. 32,300,36991 (same layer and value distribution)")
    ap.add_argument("--layout", default="btm", choices=["btm", "nt"],
                    help="btm: the layers (time-major kernels); nt: the drop-in Functions on the reference's [N,T] layout")
    ap.add_argument("--single-thread-autograd", action="store_true",
                    help="run backward in the calling thread (torch.autograd.set_multithreading_enabled(False)): "
                         "saves the hand-over to PyTorch's autograd thread, 60-120 us per step, which shows on small problems")
    ap.add_argument("--cuda-graph", action="store_true", help="capture the step in a CUDA graph and time replays")
    ap.add_argument("--recompute", action="store_true",
                    help="time the step with layer.set_backward_recompute(True) as the main measurement (profiling aid; "
                         "the default run reports it as the extra key `recompute`)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-mix", action="store_true", help="skip the streaming-mix calibration (1 read : 2 writes, 2 : 1)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="skip the short runs of the other configurations")
    ap.add_argument("--no-reference-cuda", action="store_true", help="skip timing the reference project's CUDA kernels")
    ap.add_argument("--lean", action="store_true", help="headline timing only (profiling): no e2e, mix, cpu, others, reference")
    ap.add_argument("--other-steps", type=int, default=10)
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-microbatches", type=int, default=0, help="0: micro-batches of about 128 MB per tensor")
    ap.add_argument("--e2e-host-slots", type=int, default=2, help="pinned staging slots per direction and tensor")
    args = ap.parse_args()
    if args.recompute:
        args.lean = True
    if args.lean:
        args.no_e2e = args.no_mix = args.no_cpu = args.no_others = args.no_reference_cuda = True
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    wl = dict(WORKLOADS[args.workload])
    if args.shape is not None:
        wl["shape"] = tuple(int(v) for v in args.shape.split(","))
        if len(wl["shape"]) < 3:
            raise SystemExit("--shape needs at least batch,time,neurons")
        wl["desc"] += f" [shape overridden to {wl['shape']}]"
    if args.batch is not None:
        wl["shape"] = (args.batch,) + tuple(wl["shape"][1:])
        wl["desc"] += f" [batch overridden to {args.batch}]"
    if args.impl == "reference":
        run_reference(args, wl)
    elif args.single_thread_autograd:
        with torch.autograd.set_multithreading_enabled(False):
            run_ours(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
