"""The compact spike raster (one byte per neuron-step) against the CPU checker and against the float raster.  Needs a GPU."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from sinabs_exodus_b200 import _lib
from tests import _gpu
from tests._cases import lif_case
from tests.test_gpu_lif_syn import reference_forward, synaptic_case

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _u8_forward(cs, B, M, mode, max_spikes, reset_mode, with_v_mem, saturate=True, in_scale=None):
    N, T = cs["inp"].shape
    x = _gpu.to_dev(cs["inp"], B, M, _lib.LAYOUT_BTM)
    spikes = torch.full((B, T, M), 77, dtype=torch.uint8, device=DEV)
    v_mem = torch.full_like(x, float("nan")) if with_v_mem else None
    v_post = torch.full((N,), float("nan"), device=DEV)
    count = torch.zeros(1, dtype=torch.int64, device=DEV)
    ok = _lib.lif_forward_u8(spikes, v_mem, x, _gpu.vec(cs["v_init"]), _gpu.param(in_scale, mode, B, M),
                             _gpu.param(cs["alpha"], mode, B, M), _gpu.param(cs["subtract"], mode, B, M),
                             _gpu.param(cs["theta"], mode, B, M), _gpu.param(cs["theta_low"], mode, B, M), max_spikes,
                             reset_mode, saturate, v_post, count, B, T, M)
    if not ok:
        return None
    torch.cuda.synchronize()
    s = spikes.permute(0, 2, 1).reshape(N, T).cpu().numpy()
    v = None if v_mem is None else _gpu.from_dev(v_mem, B, M, _lib.LAYOUT_BTM)
    return s, v, v_post.cpu().numpy(), int(count.item())


@pytest.mark.parametrize("B,T,M", [(3, 50, 64), (2, 33, 132), (37, 9, 4096), (75, 7, 2052)])
@pytest.mark.parametrize("with_v_mem", [True, False])
@pytest.mark.parametrize("max_spikes", [None, 1, 3])
def test_lif_forward_u8_equals_float_raster(B, T, M, with_v_mem, max_spikes):
    cs = lif_case(B * 31 + M, B * M, T, clamp=True, in_mean=0.6, in_std=1.0)
    got = _u8_forward(cs, B, M, _lib.PARAM_PER_N, max_spikes, _lib.RESET_SUBTRACT, with_v_mem)
    assert got is not None
    s, v, v_post, count = got
    s_ref, v_ref = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"], max_spikes)
    assert s.dtype == np.uint8
    np.testing.assert_array_equal(s, np.minimum(s_ref, 255).astype(np.uint8))
    if with_v_mem:
        np.testing.assert_array_equal(v, v_ref)
    assert count == int(s_ref.sum(dtype=np.float64))
    post = (v_ref[:, -1].astype(np.float64) - cs["subtract"].astype(np.float64) * s_ref[:, -1]).astype(np.float32)
    np.testing.assert_array_equal(v_post, post)


def test_lif_forward_u8_saturates_and_says_so():
    """A neuron driven to more than 255 spikes per step: the byte is 255, the count and the reset use the true number;
    without the caller's consent the call is refused."""
    B, T, M = 1, 6, 8
    N = B * M
    cs = dict(inp=np.full((N, T), 300.5, np.float32), alpha=np.ones(N, np.float32), theta=np.ones(N, np.float32),
              subtract=np.ones(N, np.float32), theta_low=None, v_init=np.zeros(N, np.float32))
    s, v, v_post, count = _u8_forward(cs, B, M, _lib.PARAM_SCALAR, None, _lib.RESET_SUBTRACT, True, saturate=True)
    s_ref, v_ref = orc.lif_forward(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"])
    assert s_ref.max() > 255 and (s == 255).all()
    np.testing.assert_array_equal(v, v_ref)
    assert count == int(s_ref.sum(dtype=np.float64))
    with pytest.raises(_lib.ExodusLibraryError, match="255"):
        _u8_forward(cs, B, M, _lib.PARAM_SCALAR, None, _lib.RESET_SUBTRACT, True, saturate=False)
    with pytest.raises(_lib.ExodusLibraryError, match="255"):
        _u8_forward(cs, B, M, _lib.PARAM_SCALAR, 1000, _lib.RESET_SUBTRACT, True, saturate=False)
    assert _u8_forward(cs, B, M, _lib.PARAM_SCALAR, 255, _lib.RESET_SUBTRACT, True, saturate=False) is not None


def test_lif_forward_u8_says_when_a_shape_is_not_eligible():
    cs = lif_case(3, 2 * 30, 12, clamp=False)                 # 30 neurons: not a multiple of 4
    assert _u8_forward(cs, 2, 30, _lib.PARAM_PER_N, 1, _lib.RESET_SUBTRACT, True) is None


@pytest.mark.parametrize("shape", ["narrow_per_n", "wide_per_m"])
@pytest.mark.parametrize("keep", [True, False])
def test_lif_syn_forward_u8(shape, keep):
    from tests.test_gpu_lif_syn import SHAPES
    B, T, M, mode = SHAPES[shape]
    cs = synaptic_case(99, B, T, M, mode, clamp=True, reset_to_value=False)
    N = B * M
    x = _gpu.to_dev(cs["inp"], B, M, _lib.LAYOUT_BTM)
    spikes = torch.full((B, T, M), 77, dtype=torch.uint8, device=DEV)
    v_mem = torch.full_like(x, float("nan")) if keep else None
    i_syn = torch.full_like(x, float("nan")) if keep else None
    v_post = torch.empty(N, device=DEV); i_last = torch.empty(N, device=DEV)
    count = torch.zeros(1, dtype=torch.int64, device=DEV)
    p = lambda k: _gpu.param(cs[k], mode, B, M)
    ok = _lib.lif_syn_forward_u8(spikes, v_mem, i_syn, x, _gpu.vec(cs["v_init"]), _gpu.vec(cs["i_init"]), p("a_syn"), p("s_syn"),
                                 p("s_mem"), p("a_mem"), p("subtract"), p("theta"), p("theta_low"), None, _lib.RESET_SUBTRACT,
                                 True, v_post, i_last, count, B, T, M)
    assert ok
    torch.cuda.synchronize()
    s_ref, v_ref, i_ref = reference_forward(cs, None, False)
    np.testing.assert_array_equal(spikes.permute(0, 2, 1).reshape(N, T).cpu().numpy(), np.minimum(s_ref, 255).astype(np.uint8))
    np.testing.assert_array_equal(i_last.cpu().numpy(), i_ref[:, -1])
    assert count.item() == int(s_ref.sum(dtype=np.float64))
    if keep:
        np.testing.assert_array_equal(_gpu.from_dev(v_mem, B, M, _lib.LAYOUT_BTM), v_ref)
        np.testing.assert_array_equal(_gpu.from_dev(i_syn, B, M, _lib.LAYOUT_BTM), i_ref)


@pytest.mark.parametrize("kwargs", [dict(tau_mem=15.0, min_v_mem=-0.5), dict(tau_mem=15.0, tau_syn=6.0), dict(tau_mem=15.0, record_states=True)])
@pytest.mark.parametrize("neurons", [24, 30])
def test_layer_uint8_output_equals_float_output(kwargs, neurons):
    """`set_spike_output(torch.uint8)`: same raster, state, recordings and firing rate as the float layer under
    no_grad, also for a neuron count the byte kernels do not take (converted); refused while autograd records."""
    from sinabs_exodus_b200.layers import LIF
    from sinabs_exodus_b200.compat.activation import SingleSpike
    torch.manual_seed(3)
    x = 0.5 + 0.8 * torch.randn(3, 40, neurons, device=DEV)
    a = LIF(spike_fn=SingleSpike, **kwargs).to(DEV)
    b = LIF(spike_fn=SingleSpike, **kwargs).to(DEV).set_spike_output(torch.uint8)
    with torch.no_grad():
        for _ in range(2):                                  # the second call starts from the carried state
            out_a, out_b = a(x), b(x)
            assert out_b.dtype == torch.uint8 and out_b.shape == out_a.shape
            torch.testing.assert_close(out_b.float(), out_a, rtol=0, atol=0)
            torch.testing.assert_close(b.v_mem, a.v_mem, rtol=0, atol=0)
            torch.testing.assert_close(b.firing_rate, a.firing_rate, rtol=1e-6, atol=0)
            for key in a.recordings:
                torch.testing.assert_close(b.recordings[key], a.recordings[key], rtol=0, atol=0)
    with pytest.raises(ValueError, match="no gradient"):
        b(x.clone().requires_grad_(True))
    from sinabs_exodus_b200.layers import IAF
    with pytest.raises(ValueError, match="255"):
        IAF().to(DEV).set_spike_output(torch.uint8)          # MultiSpike: more than 255 possible
    IAF().to(DEV).set_spike_output(torch.uint8, saturate=True)
