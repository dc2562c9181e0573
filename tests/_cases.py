"""Seeded problem generators shared by CPU and GPU tests (numpy, float32, [N, T] layout)."""
from __future__ import annotations

import numpy as np


def lif_case(seed, N, T, per_neuron=True, clamp=True, v_init_random=True, subtract_given=True,
             in_mean=0.3, in_std=0.5):
    """Random LIF problem.  Thresholds stay well above the lower bound."""
    rng = np.random.default_rng(seed)
    inp = (in_mean + in_std * rng.standard_normal((N, T))).astype(np.float32)
    if per_neuron:
        alpha = rng.uniform(0.5, 1.0, N).astype(np.float32)
        theta = rng.uniform(0.3, 1.2, N).astype(np.float32)
        subtract = (theta * rng.uniform(0.5, 1.0, N)).astype(np.float32) if subtract_given else theta.copy()
        theta_low = (-rng.uniform(0.2, 1.0, N)).astype(np.float32) if clamp else None
    else:
        alpha = np.full(N, np.float32(np.exp(-1 / 20.0)), np.float32)
        theta = np.ones(N, np.float32)
        subtract = np.full(N, 0.8 if subtract_given else 1.0, np.float32)
        theta_low = np.full(N, -1.0, np.float32) if clamp else None
    v_init = (rng.uniform(-0.5, 0.5, N)).astype(np.float32) if v_init_random else np.zeros(N, np.float32)
    return dict(inp=inp, alpha=alpha, theta=theta, subtract=subtract, theta_low=theta_low, v_init=v_init)


def near_threshold_rows(v_mem, theta, rel=1e-5):
    """Rows in which some step's membrane potential lies within rel*theta of a positive multiple of theta."""
    th = theta[:, None]
    k = np.maximum(np.round(v_mem / th), 1.0)
    return (np.abs(v_mem - k * th) <= rel * np.abs(th)).any(axis=1)


def rel_err(a, ref):
    """max |a - ref| / max(|ref|, rms(ref)) -- the 1e-5 criterion used for v_mem and gradients."""
    ref = np.asarray(ref, np.float64)
    a = np.asarray(a, np.float64)
    scale = np.sqrt(np.mean(ref ** 2)) if ref.size else 1.0
    denom = np.maximum(np.abs(ref), max(scale, 1e-30))
    return float(np.max(np.abs(a - ref) / denom)) if ref.size else 0.0
