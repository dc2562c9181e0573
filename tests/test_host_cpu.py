"""Host-side logic that needs no GPU: surrogate classification, parameter handling, layers' bookkeeping, conversion."""
import numpy as np
import pytest
import torch

from sinabs_exodus_b200 import _lib, conversion, layers as el
from sinabs_exodus_b200.compat import activation as sa
from sinabs_exodus_b200.compat import layers as sl
from sinabs_exodus_b200.layers.lif import _flat_param, expand_to_1d_contiguous
from sinabs_exodus_b200.spike import _mode_of, _reduce_to_param
from sinabs_exodus_b200.surrogate import classify


def test_surrogate_classification():
    assert classify(sa.SingleExponential(0.3, 2.0)) == (_lib.SURR_SINGLE_EXPONENTIAL, 0.3, 2.0)
    assert classify(sa.Heaviside(0.25)) == (_lib.SURR_HEAVISIDE, 0.25, 0.0)
    assert classify(sa.PeriodicExponential())[0] == _lib.SURR_PERIODIC_EXPONENTIAL
    assert classify(lambda v, th: v * 0)[0] == _lib.SURR_GENERIC

    class SingleExponential:            # same name, different function: must not be fused
        grad_width = 0.5
        grad_scale = 1.0

        def __call__(self, v, th):
            return torch.exp(-torch.abs(v - th))

    assert classify(SingleExponential())[0] == _lib.SURR_GENERIC


def test_surrogate_formulas_match_checker():
    from oracle import oracle as orc
    v = torch.linspace(-2, 5, 141).reshape(1, -1).repeat(2, 1)
    th = torch.tensor([[0.7], [1.0]])
    for fn, ref in ((sa.SingleExponential(), orc.surrogate_single_exponential),
                    (sa.Heaviside(), orc.surrogate_heaviside),
                    (sa.PeriodicExponential(), orc.surrogate_periodic_exponential)):
        np.testing.assert_allclose(fn(v, th).numpy(), ref(v.numpy(), th.numpy()), rtol=1e-5, atol=1e-7)


def test_param_modes_and_reduction():
    assert _mode_of(torch.zeros(1), 4, 12, "p") == _lib.PARAM_SCALAR
    assert _mode_of(torch.zeros(4), 4, 12, "p") == _lib.PARAM_PER_M
    assert _mode_of(torch.zeros(12), 4, 12, "p") == _lib.PARAM_PER_N
    with pytest.raises(ValueError):
        _mode_of(torch.zeros(5), 4, 12, "p")
    g = torch.arange(12.0)
    assert _reduce_to_param(g, (), _lib.PARAM_SCALAR, 3, 4).item() == 66
    torch.testing.assert_close(_reduce_to_param(g, (2, 2), _lib.PARAM_PER_M, 3, 4), torch.tensor([[12., 15.], [18., 21.]]))
    assert _reduce_to_param(g, (3, 4), _lib.PARAM_PER_N, 3, 4).shape == (3, 4)


def test_flat_param_keeps_graph():
    p = torch.nn.Parameter(torch.rand(3, 1, 1))
    flat = _flat_param(p, (3, 2, 2), 5, "cpu")
    assert flat.shape == (12,)
    flat.sum().backward()
    torch.testing.assert_close(p.grad, torch.full((3, 1, 1), 4.0))
    assert _flat_param(2.0, (3,), 1, "cpu").shape == (1,)
    assert _flat_param(torch.rand(5, 3), (3,), 5, "cpu").shape == (15,)
    assert expand_to_1d_contiguous(1.5, (2, 3)).shape == (6,)


def test_layer_bookkeeping():
    lyr = el.LIF(tau_mem=20.0, tau_syn=5.0, train_alphas=True, shape=(2, 3))
    assert lyr.does_spike and lyr.is_state_initialised() and lyr.state_has_shape((2, 3))
    assert set(dict(lyr.named_parameters())) == {"alpha_mem", "alpha_syn"}
    assert set(dict(lyr.named_buffers())) == {"v_mem", "i_syn"}
    assert repr(lyr).startswith("EXODUS ")
    lyr2 = el.LIF(tau_mem=20.0)
    assert set(dict(lyr2.named_parameters())) == {"tau_mem"} and not lyr2.is_state_initialised()
    assert lyr2.max_num_spikes_per_bin is None
    assert el.LIF(tau_mem=1.0, spike_fn=sa.SingleSpike).max_num_spikes_per_bin == 1
    assert el.LIF(tau_mem=1.0, spike_fn=sa.MaxSpike(3)).max_num_spikes_per_bin == 3
    with pytest.raises(NotImplementedError):
        el.LIF(tau_mem=1.0, reset_fn=lambda *a: None)
    iaf = el.IAF()
    assert iaf.tau_mem is None and float(iaf.alpha_mem_calculated) == 1.0
    assert "tau_mem" not in iaf._param_dict and "norm_input" not in iaf._param_dict
    leak = el.ExpLeak(tau_mem=10.0)
    assert not leak.does_spike and "spike_fn" not in leak._param_dict
    assert leak.decay_early is False and leak.norm_input is False
    with pytest.raises(TypeError):
        el.LIFSqueeze(tau_mem=10.0)
    sq = el.LIFSqueeze(tau_mem=10.0, num_timesteps=7)
    assert sq._param_dict["num_timesteps"] == 7 and sq._param_dict["batch_size"] == -1


def test_state_dict_interchange():
    """Parameter and buffer names agree between the PyTorch-side class and the EXODUS class."""
    for kwargs in (dict(tau_mem=20.0), dict(tau_mem=20.0, tau_syn=10.0, train_alphas=True)):
        a = sl.LIF(shape=(2, 4), **kwargs)
        b = el.LIF(shape=(2, 4), **kwargs)
        assert set(a.state_dict()) == set(b.state_dict())
        b.load_state_dict(a.state_dict())
        a.load_state_dict(b.state_dict())


def test_conversion_roundtrip():
    model = torch.nn.Sequential(
        torch.nn.Linear(4, 4), sl.LIF(tau_mem=15.0, min_v_mem=-0.5), torch.nn.Linear(4, 4),
        sl.IAFSqueeze(batch_size=3, min_v_mem=-1.0), sl.ExpLeak(tau_mem=7.0))
    ex = conversion.sinabs_to_exodus(model)
    assert type(ex[1]) is el.LIF and type(ex[3]) is el.IAFSqueeze and type(ex[4]) is el.ExpLeak
    assert ex[1].min_v_mem == -0.5 and ex[3].batch_size == 3 and ex[3].min_v_mem == -1.0
    assert float(ex[1].tau_mem) == 15.0
    back = conversion.exodus_to_sinabs(ex)
    assert type(back[1]) is sl.LIF and type(back[3]) is sl.IAFSqueeze and type(back[4]) is sl.ExpLeak
    assert back[3].batch_size == 3 and float(back[4].tau_mem) == 7.0
    assert set(conversion.module_map.values()) == {el.IAF, el.IAFSqueeze, el.LIF, el.LIFSqueeze, el.ExpLeak, el.ExpLeakSqueeze}


def test_function_validation_on_cpu_tensors():
    """Shape/contiguity errors are ValueErrors raised before the library is touched."""
    from sinabs_exodus_b200 import IntegrateAndFire, LeakyIntegrator
    x = torch.rand(2, 10); a = torch.full((2,), 0.9); z = torch.zeros(2); th = torch.ones(2)
    with pytest.raises(ValueError):
        IntegrateAndFire.apply(x[0], a, z, th, th, None, sa.Heaviside())
    with pytest.raises(ValueError):
        IntegrateAndFire.apply(x, a.reshape(2, 1), z, th, th, None, sa.Heaviside())
    with pytest.raises(ValueError):
        IntegrateAndFire.apply(x, a, z, th, th, torch.tensor([1.2, 0.0]), sa.Heaviside())
    with pytest.raises(ValueError):
        LeakyIntegrator.apply(x.t(), a, z)
    with pytest.raises(_lib.ExodusLibraryError):
        LeakyIntegrator.apply(x, a, z)          # valid arguments, CPU tensors: no CPU implementation


def test_decay_from_tau_matches_autograd():
    """The one-node decay Function: same values and gradients as exp(-1/tau) and 1 - exp(-1/tau) through autograd."""
    from sinabs_exodus_b200.layers.lif import _DecayFromTau
    tau = torch.tensor([2.0, 10.0, 37.5], dtype=torch.float32, requires_grad=True)
    w1, w2 = torch.tensor([0.3, -1.2, 2.0]), torch.tensor([1.5, 0.4, -0.7])
    alpha, comp = _DecayFromTau.apply(tau, True)
    torch.testing.assert_close(alpha, torch.exp(-1.0 / tau.detach()), rtol=0, atol=0)
    torch.testing.assert_close(comp, 1.0 - torch.exp(-1.0 / tau.detach()), rtol=0, atol=0)
    ((alpha * w1).sum() + (comp * w2).sum()).backward()
    got = tau.grad.clone()
    tau.grad = None
    a = torch.exp(-1.0 / tau)
    ((a * w1).sum() + ((1.0 - a) * w2).sum()).backward()
    torch.testing.assert_close(got, tau.grad, rtol=1e-6, atol=1e-9)
    # one output unused, and the variant without the complement
    tau.grad = None
    alpha, comp = _DecayFromTau.apply(tau, True)
    comp.sum().backward()
    torch.testing.assert_close(tau.grad, -(torch.exp(-1.0 / tau.detach()) / tau.detach() ** 2), rtol=1e-6, atol=1e-9)
    alpha, none = _DecayFromTau.apply(tau, False)
    assert none is None
    assert torch.autograd.gradcheck(lambda t: _DecayFromTau.apply(t, True), (torch.tensor([3.0, 8.0], dtype=torch.float64,
                                    requires_grad=True),))


def test_scalar_constants_are_cached():
    from sinabs_exodus_b200.layers.lif import _scalar_constant
    a = _scalar_constant(0.75, "cpu")
    assert a is _scalar_constant(0.75, "cpu") and a.item() == 0.75 and a.shape == (1,)
    assert _scalar_constant(0.5, "cpu") is not a


def test_firing_rate_is_formed_on_read():
    layer = el.IAF()
    assert layer.firing_rate is None
    layer._set_rate_source(torch.tensor([30], dtype=torch.int64), 120)
    assert abs(layer.firing_rate.item() - 0.25) < 1e-7
    layer.firing_rate = torch.tensor(0.5)          # plain assignment still works (sinabs sets it that way)
    assert layer.firing_rate.item() == 0.5


def test_variant_layers_are_ordinary_classes():
    import pickle
    for cls, kwargs in ((el.IAFSqueeze, dict(batch_size=2, spike_threshold=0.5)),
                        (el.ExpLeakSqueeze, dict(num_timesteps=5, tau_mem=12.0)),
                        (el.LIFSqueeze, dict(batch_size=3, tau_mem=20.0, tau_syn=5.0))):
        layer = cls(**kwargs)
        assert repr(layer).startswith("EXODUS " + cls.__name__)
        clone = pickle.loads(pickle.dumps(layer))
        assert type(clone) is cls and clone.arg_dict.keys() == layer.arg_dict.keys()
        rebuilt = cls(**layer.arg_dict)
        assert type(rebuilt) is cls
    assert "tau_mem" not in el.IAF().arg_dict and "spike_fn" not in el.ExpLeak(tau_mem=5.0).arg_dict


def test_value_checks_are_remembered_per_tensor():
    """The alpha / threshold checks read back from the device once per (live tensor, version), not per call,
    and still fire when a tensor is modified in place or replaced by another one."""
    from sinabs_exodus_b200.spike import _CHECKED, _check_values
    a, th, lo = torch.rand(6), torch.ones(6), -torch.ones(6)
    _check_values(a, th, lo)
    entries = len(_CHECKED)
    _check_values(a, th, lo)
    assert len(_CHECKED) == entries
    a.mul_(5.0)                                   # same object, new version
    with pytest.raises(ValueError):
        _check_values(a, th, lo)
    for _ in range(4):                            # short-lived tensors may reuse ids: never trusted blindly
        with pytest.raises(ValueError):
            _check_values(torch.full((6,), 1.5), th, None)
    with pytest.raises(ValueError):
        _check_values(torch.rand(6), th, torch.full((6,), 2.0))


def test_nvtx_ranges_wrap_and_unwrap_the_launching_calls():
    from sinabs_exodus_b200 import _lib
    plain = _lib.lif_forward
    _lib.set_nvtx_ranges(True)
    try:
        assert _lib.lif_forward is not plain and _lib.lif_forward.__wrapped__ is plain
        assert _lib.acc_finish.__wrapped__.__name__ == "acc_finish"
        _lib.set_nvtx_ranges(True)                        # idempotent
        assert _lib.lif_forward.__wrapped__ is plain
    finally:
        _lib.set_nvtx_ranges(False)
    assert _lib.lif_forward is plain
