"""The scan entry point that brings its own scratch memory (``exb_leaky_forward_scan_static``).  Needs a GPU.

Some hosts may not allocate device memory once they are running -- a service with a fixed memory
budget, or code living inside another framework's memory pool -- so they cannot provide the
scratch buffer the time-parallel leaky scan needs.  For them the library carries a fixed 1 MiB
array.  These tests call that entry point through the C ABI and compare it with the entry point
that takes a caller-provided workspace.

This file sorts last on purpose: a run that stops at the first failure has then already been
through every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-5
DEV = "cuda:0"


def _problem(seed, B, T, M):
    rng = np.random.default_rng(seed)
    x = torch.tensor(rng.standard_normal((B, T, M)).astype(np.float32), device=DEV)
    alpha = torch.tensor(rng.uniform(0.8, 1.0, B * M).astype(np.float32), device=DEV)
    v0 = torch.tensor(rng.standard_normal(B * M).astype(np.float32), device=DEV)
    return x, alpha, v0


def _with_workspace(x, alpha, v0):
    from sinabs_exodus_b200 import _lib
    B, T, M = x.shape
    ws = torch.empty((_lib.leaky_scan_workspace_bytes(B, T, M) + 3) // 4, dtype=torch.int32, device=DEV)
    out = torch.full_like(x, float("nan")); v_last = torch.empty(B * M, device=DEV)
    _lib.leaky_forward_scan(out, x, v0, (alpha, _lib.PARAM_PER_N), (None, 0), v_last, ws, B, T, M)
    return out, v_last


def _static(x, alpha, v0):
    from sinabs_exodus_b200 import _lib
    B, T, M = x.shape
    out = torch.full_like(x, float("nan")); v_last = torch.empty(B * M, device=DEV)
    _lib.leaky_forward_scan_static(out, x, v0, (alpha, _lib.PARAM_PER_N), (None, 0), v_last, B, T, M)
    return out, v_last


def test_static_scratch_matches_workspace_entry_point_twice_in_a_row():
    """Two calls back to back on the shared array (different data, different shapes): each must
    equal the workspace version, i.e. nothing of the first call leaks into the second."""
    from sinabs_exodus_b200 import _lib
    for seed, (B, T, M) in enumerate([(1, 4000, 128), (2, 3001, 36)]):
        x, alpha, v0 = _problem(seed, B, T, M)
        assert 0 < _lib.leaky_scan_workspace_bytes(B, T, M) <= _lib.STATIC_SCRATCH_BYTES
        got, got_last = _static(x, alpha, v0)
        want, want_last = _with_workspace(x, alpha, v0)
        torch.cuda.synchronize()
        scale = float(want.pow(2).mean().sqrt())
        err = float(((got - want).abs() / torch.clamp(want.abs(), min=scale)).max())
        assert err < TOL, (B, T, M, err)
        assert not torch.isnan(got).any()
        torch.testing.assert_close(got_last, want_last, rtol=TOL, atol=TOL * scale)
    _lib.device_status()


def test_static_scratch_rejects_oversized_and_inapplicable_shapes():
    from sinabs_exodus_b200 import _lib
    # 1100 tiles x 2 segments x 512 B of aggregates: more than the built-in array holds
    B, T, M = 1100, 256, 128
    assert _lib.leaky_scan_workspace_bytes(B, T, M) > _lib.STATIC_SCRATCH_BYTES
    x = torch.zeros(B, T, M, device=DEV); a = torch.full((1,), 0.9, device=DEV)
    out = torch.empty_like(x)
    with pytest.raises(_lib.ExodusLibraryError, match="bytes of scratch"):
        _lib.leaky_forward_scan_static(out, x, None, (a, _lib.PARAM_SCALAR), (None, 0), None, B, T, M)
    # too short to split at all
    x2 = torch.zeros(1, 40, 128, device=DEV)
    with pytest.raises(_lib.ExodusLibraryError, match="does not apply"):
        _lib.leaky_forward_scan_static(torch.empty_like(x2), x2, None, (a, _lib.PARAM_SCALAR), (None, 0), None, 1, 40, 128)


def test_static_scratch_call_takes_no_device_memory():
    """What the entry point promises: once the first call on the device has been made (it looks up the array and
    makes the runtime load the kernel), a call takes no device memory at all.  Free device memory as the driver
    reports it is the same before and after a call on preallocated tensors."""
    from sinabs_exodus_b200 import _lib
    B, T, M = 2, 2048, 64
    x, alpha, v0 = _problem(5, B, T, M)
    out = torch.empty_like(x); v_last = torch.empty(B * M, device=DEV)
    args = (out, x, v0, (alpha, _lib.PARAM_PER_N), (None, 0), v_last, B, T, M)
    _lib.leaky_forward_scan_static(*args)          # first call: set-up happens here
    torch.cuda.synchronize()
    unchanged = False
    for _ in range(3):                             # the figure is device-wide; allow for an unrelated blip
        free_before, _total = torch.cuda.mem_get_info()
        _lib.leaky_forward_scan_static(*args)
        torch.cuda.synchronize()
        free_after, _total = torch.cuda.mem_get_info()
        if free_after == free_before:
            unchanged = True
            break
    assert unchanged, (free_before, free_after)
    want, _ = _with_workspace(x, alpha, v0)
    torch.testing.assert_close(out, want, rtol=TOL, atol=TOL)
