"""The give-up path of the kernels' bounded waits, exercised without any fault.  Needs a GPU.

``exb_set_wait_limit`` shortens the poll limit and keeps the time-parallel scan's ready flags down, so the
segments that wait for an earlier segment run out of polls.  The kernel must return normally, the device status
must report the time-out exactly once, the state that depended on the wait must be NaN, and the next call (with
the defaults restored) must be correct.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_scan_wait_runs_out_and_the_kernel_returns():
    from sinabs_exodus_b200 import _lib
    B, T, M = 1, 256, 128                                  # one tile, four segments: four CTAs, all resident at once
    nbytes = _lib.leaky_scan_workspace_bytes(B, T, M)
    assert nbytes > 0
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(B, T, M, device=DEV, generator=g)
    alpha = torch.full((1,), 0.9, device=DEV)
    ws = torch.empty((nbytes + 3) // 4, dtype=torch.int32, device=DEV)

    def run():
        out = torch.full_like(x, float("nan")); v_last = torch.zeros(B * M, device=DEV)
        total = torch.zeros(1, dtype=torch.float64, device=DEV)
        _lib.leaky_forward_scan(out, x, None, (alpha, _lib.PARAM_SCALAR), (None, 0), v_last, ws, B, T, M, out_sum=total)
        torch.cuda.synchronize()                           # the kernel has returned
        return out, v_last, total

    _lib.device_status()                                   # nothing pending
    try:
        _lib.set_wait_limit(1024, withhold_scan_flags=True)
        out, v_last, total = run()
        with pytest.raises(_lib.ExodusLibraryError, match="wait ran out"):
            _lib.device_status()
        _lib.device_status()                               # reported once, then clear
        assert torch.isnan(v_last).all() and torch.isnan(total).all()
        assert not torch.isnan(out[:, :16]).any()          # the first segment waits for nobody
        assert torch.isnan(out[:, -1]).all()               # the last one gave up before writing
    finally:
        _lib.set_wait_limit(0, withhold_scan_flags=False)
    out, v_last, total = run()
    _lib.device_status()
    want = torch.empty_like(x); want_last = torch.empty(B * M, device=DEV)
    _lib.leaky_forward(want, x, None, (alpha, _lib.PARAM_SCALAR), (None, 0), want_last, B, T, M, _lib.LAYOUT_BTM)
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(v_last, want_last, rtol=1e-5, atol=1e-5)
