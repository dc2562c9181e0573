"""The training pair that never materialises v_mem (``exb_lif_forward_ckpt`` / ``exb_lif_backward_ckpt``), through
the C ABI.  Needs a GPU.

The forward must give the spikes of the checker bit for bit and checkpoints that equal the checker's post-reset
potential at every eighth step; the backward rebuilds v_mem with the forward's own arithmetic, so its gradients must
equal those of ``exb_lif_backward`` on the materialised v_mem BIT FOR BIT, whatever the tile shape and pipeline.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from tests._cases import lif_case

pytestmark = pytest.mark.gpu

# narrow tiles, ragged in time and neurons, fewer steps than one checkpoint interval, wide tiles (last two)
SHAPES = [(3, 50, 36), (2, 64, 128), (1, 100, 260), (4, 7, 8), (2, 8, 4), (5, 17, 132), (300, 21, 516), (150, 40, 1024)]


def _case(seed, B, T, M, mode, clamp):
    from sinabs_exodus_b200 import _lib
    N = B * M
    cs = lif_case(seed, N, T, clamp=clamp)
    for k in ("alpha", "theta", "subtract", "theta_low"):
        if cs[k] is None:
            continue
        if mode == _lib.PARAM_SCALAR:
            cs[k] = np.full(N, cs[k][0], np.float32)
        elif mode == _lib.PARAM_PER_M:
            cs[k] = np.tile(cs[k][:M], B)
    return cs


@pytest.mark.parametrize("B,T,M", SHAPES)
@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("reset_mode", [0, 1])
def test_checkpointed_pair_equals_the_materialised_one(B, T, M, mode, reset_mode):
    from sinabs_exodus_b200 import _lib
    from tests import _gpu
    for clamp, max_spikes, kind, p0, p1 in ((True, None, _lib.SURR_SINGLE_EXPONENTIAL, 0.5, 1.0),
                                            (False, 1, _lib.SURR_PERIODIC_EXPONENTIAL, 0.5, 1.0),
                                            (True, 2, _lib.SURR_HEAVISIDE, 0.6, 0.0)):
        cs = _case(40 + B + T + M, B, T, M, mode, clamp)
        if reset_mode == 1:
            cs["subtract"] = (0.25 * cs["theta"]).astype(np.float32)
        N = B * M
        s_ref, v_ref = orc.lif_forward_ext(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"],
                                           cs["theta_low"], max_spikes, reset_to_value=bool(reset_mode))
        res = _gpu.lif_forward_ckpt(cs, B, M, mode, max_spikes, reset_mode=reset_mode)
        assert res is not None
        s, ckpt, v_post, count, dev_tensors = res
        np.testing.assert_array_equal(s, s_ref)
        assert count == int(s_ref.sum())
        # the state that enters step 8j: the initial state, or the potential of step 8j-1 after its reset
        if reset_mode == 0:
            post = (v_ref.astype(np.float64) - cs["subtract"].astype(np.float64)[:, None] * s_ref).astype(np.float32)
        else:
            post = np.where(s_ref > 0, cs["subtract"][:, None], v_ref).astype(np.float32)
        want = np.concatenate([cs["v_init"][:, None], post[:, 7::8]], axis=1)[:, :ckpt.shape[1]]
        np.testing.assert_array_equal(ckpt, want)
        np.testing.assert_array_equal(v_post, post[:, -1])

        _, v_gpu, _, _ = _gpu.lif_forward(cs, B, M, _lib.LAYOUT_BTM, mode, max_spikes, reset_mode=reset_mode)
        rng = np.random.default_rng(B * 31 + T)
        go = rng.standard_normal((N, T)).astype(np.float32)
        G = rng.standard_normal(N).astype(np.float32)
        for want_alpha in (True, False):
            a = _gpu.lif_backward(cs, v_gpu, go, B, M, _lib.LAYOUT_BTM, mode=mode, g_last=G, kind=kind, p0=p0, p1=p1,
                                  max_spikes=max_spikes, reset_mode=reset_mode, want_alpha=want_alpha)
            b = _gpu.lif_backward_ckpt(cs, dev_tensors, go, B, M, mode=mode, g_last=G, kind=kind, p0=p0, p1=p1,
                                       max_spikes=max_spikes, reset_mode=reset_mode, want_alpha=want_alpha)
            for x, y in zip(a[:3], b[:3]):
                if x is None:
                    assert y is None
                else:
                    assert np.isfinite(y).all()
                    np.testing.assert_array_equal(y, x)


@pytest.mark.parametrize("B,T,M", [(3, 40, 20), (300, 21, 516)])
def test_checkpointed_pair_with_input_scale(B, T, M):
    """Fused input scale and its gradient (rebuilt from the state in both routes)."""
    from sinabs_exodus_b200 import _lib
    from tests import _gpu
    N = B * M
    cs = lif_case(77, N, T, clamp=True)
    cs["alpha"] = np.minimum(cs["alpha"], np.float32(0.97))
    scale = (1.0 - cs["alpha"]).astype(np.float32)
    scaled = dict(cs, inp=(scale[:, None] * cs["inp"]).astype(np.float32))
    s_ref, v_ref = orc.lif_forward(scaled["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"])
    res = _gpu.lif_forward_ckpt(cs, B, M, 2, in_scale=scale)
    assert res is not None
    s, ckpt, v_post, count, dev_tensors = res
    np.testing.assert_array_equal(s, s_ref)
    go = np.random.default_rng(9).standard_normal((N, T)).astype(np.float32)
    G = np.random.default_rng(10).standard_normal(N).astype(np.float32)
    a = _gpu.lif_backward(cs, v_ref, go, B, M, _lib.LAYOUT_BTM, g_last=G, kind=_lib.SURR_SINGLE_EXPONENTIAL, p0=0.5, p1=1.0,
                          in_scale=scale, want_scale=True, scale_from_state=True, want_alpha=True)
    b = _gpu.lif_backward_ckpt(cs, dev_tensors, go, B, M, g_last=G, in_scale=scale, want_scale=True, want_alpha=True)
    for x, y in zip(a, b):
        np.testing.assert_array_equal(y, x)


def test_checkpointed_pair_refuses_what_it_cannot_do():
    import torch
    from sinabs_exodus_b200 import _lib
    from tests import _gpu
    cs = lif_case(3, 2 * 6, 20, clamp=True)          # 6 neurons: not a multiple of 4
    assert _gpu.lif_forward_ckpt(cs, 2, 6) is None
    cs = lif_case(3, 2 * 8, 20, clamp=True)
    res = _gpu.lif_forward_ckpt(cs, 2, 8)
    go = np.ones((16, 20), np.float32)
    with pytest.raises(_lib.ExodusLibraryError, match="built-in surrogates"):
        _gpu.lif_backward_ckpt(cs, res[4], go, 2, 8, kind=_lib.SURR_GENERIC)
    bad = torch.empty(2, 2, 8, device="cuda:0")
    with pytest.raises(_lib.ExodusLibraryError, match="ckpt must be"):
        _lib.lif_forward_ckpt(torch.empty(2, 20, 8, device="cuda:0"), bad, torch.empty(2, 20, 8, device="cuda:0"), None,
                              (None, 0), (torch.ones(1, device="cuda:0"), 0), (None, 0), (torch.ones(1, device="cuda:0"), 0),
                              (None, 0), None, 0, None, None, 2, 20, 8)


@pytest.mark.parametrize("norm_input", [True, False])
@pytest.mark.parametrize("shape", [(8, 100, 128), (3, 37, 4, 6, 6), (300, 12, 516)])
def test_layer_with_backward_recompute_equals_the_layer_without(shape, norm_input):
    """``layer.set_backward_recompute(True, always=True)``: same spikes, same state, bit-identical input gradient; the tau gradient
    comes out of the same per-neuron values through an atomic reduction, so it is compared to 1e-6."""
    import torch
    import sinabs_exodus_b200 as ex
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(5)
    x = (0.6 * torch.randn(shape, device=dev, generator=g) + 0.3)
    if norm_input:
        x = 4.0 * x
    grad = torch.randn(shape, device=dev, generator=g)
    results = []
    for recompute in (False, True):
        layer = ex.layers.LIF(tau_mem=20.0, min_v_mem=-1.0, norm_input=norm_input).to(dev)
        layer.set_backward_recompute(recompute, always=True)
        xin = x.clone().requires_grad_(True)
        before = torch.cuda.memory_allocated()
        out = layer(xin)
        held = torch.cuda.memory_allocated() - before
        out.backward(grad)
        results.append((out.detach(), xin.grad, layer.tau_mem.grad.clone(), layer.v_mem.detach().clone(), held,
                        float(layer.firing_rate)))
    a, b = results
    assert a[0].sum() > 0
    torch.testing.assert_close(b[0], a[0], rtol=0, atol=0)
    torch.testing.assert_close(b[1], a[1], rtol=0, atol=0)
    torch.testing.assert_close(b[2], a[2], rtol=1e-6, atol=0)
    torch.testing.assert_close(b[3], a[3], rtol=0, atol=0)
    assert b[5] == a[5]
    if x.numel() * 4 > (1 << 20):
        assert b[4] < a[4] - 0.8 * x.numel() * 4      # most of a v_mem-sized tensor less is held after the forward


def test_layer_with_backward_recompute_falls_back():
    """Recorded states, a surrogate the kernels do not know and neuron counts the TMA kernels do not take run as before."""
    import torch
    import sinabs_exodus_b200 as ex
    dev = "cuda:0"
    x = torch.rand(2, 30, 10, device=dev) * 2
    for kw in (dict(record_states=True), dict(surrogate_grad_fn=lambda v, th: torch.exp(-(v - th).abs())), dict()):
        layer = ex.layers.LIF(tau_mem=10.0, norm_input=False, **kw).to(dev)
        ref = ex.layers.LIF(tau_mem=10.0, norm_input=False, **kw).to(dev)
        layer.set_backward_recompute(True, always=True)
        xa = x.clone().requires_grad_(True); xb = x.clone().requires_grad_(True)
        layer(xa).sum().backward(); ref(xb).sum().backward()
        torch.testing.assert_close(xa.grad, xb.grad, rtol=0, atol=0)
        if kw.get("record_states"):
            assert "v_mem" in layer.recordings


@pytest.mark.parametrize("B,T,M", [(3, 50, 36), (300, 21, 516), (2, 33, 10)])
@pytest.mark.parametrize("reset_mode", [0, 1])
def test_forward_without_v_mem(B, T, M, reset_mode):
    """``exb_lif_forward`` with v_mem == NULL: the same spikes, final state and count; refused (nothing launched) for
    shapes the TMA-staged kernels do not take (10 neurons)."""
    import torch
    from sinabs_exodus_b200 import _lib
    from tests import _gpu
    cs = _case(60 + B + T, B, T, M, 2, True)
    if reset_mode == 1:
        cs["subtract"] = (0.25 * cs["theta"]).astype(np.float32)
    s_ref, v_ref = orc.lif_forward_ext(cs["inp"], cs["v_init"], cs["alpha"], cs["subtract"], cs["theta"], cs["theta_low"],
                                       None, reset_to_value=bool(reset_mode))
    x = _gpu.to_dev(cs["inp"], B, M, _lib.LAYOUT_BTM)
    spikes = torch.full_like(x, float("nan"))
    v_post = torch.full((B * M,), float("nan"), device=_gpu.DEV)
    count = torch.zeros(1, dtype=torch.int64, device=_gpu.DEV)
    P = lambda k: _gpu.param(cs[k], 2, B, M)
    ok = _lib.lif_forward(spikes, None, x, _gpu.vec(cs["v_init"]), (None, 0), P("alpha"), P("subtract"), P("theta"),
                          P("theta_low"), None, reset_mode, v_post, count, B, T, M, _lib.LAYOUT_BTM)
    torch.cuda.synchronize()
    if M % 4:
        assert ok is False and bool(torch.isnan(spikes).all())
        return
    assert ok is True
    np.testing.assert_array_equal(_gpu.from_dev(spikes, B, M, _lib.LAYOUT_BTM), s_ref)
    assert int(count.item()) == int(s_ref.sum())
    _, _, v_post_ref, _ = _gpu.lif_forward(cs, B, M, _lib.LAYOUT_BTM, 2, None, reset_mode=reset_mode)
    np.testing.assert_array_equal(v_post.cpu().numpy(), v_post_ref)


def test_layer_inference_writes_no_v_mem():
    """Under ``torch.no_grad()`` and without ``record_states`` the layer's forward launch writes the spikes only."""
    import torch
    import sinabs_exodus_b200 as ex
    dev = "cuda:0"
    x = torch.rand(16, 200, 2048, device=dev) * 0.6
    a = ex.layers.LIF(tau_mem=20.0, norm_input=False).to(dev)
    b = ex.layers.LIF(tau_mem=20.0, norm_input=False).to(dev)
    out_a = a(x)
    torch.cuda.synchronize(); torch.cuda.reset_peak_memory_stats(); base = torch.cuda.memory_allocated()
    with torch.no_grad():
        out_b = b(x)
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    assert out_a.sum() > 0
    torch.testing.assert_close(out_b, out_a.detach(), rtol=0, atol=0)
    torch.testing.assert_close(b.v_mem, a.v_mem.detach(), rtol=0, atol=0)
    assert float(b.firing_rate) == float(a.firing_rate)
    assert peak < 1.5 * x.numel() * 4          # one output tensor, not two
    rec = ex.layers.LIF(tau_mem=20.0, norm_input=False, record_states=True).to(dev)
    with torch.no_grad():
        rec(x[:2])
    assert rec.recordings["v_mem"].shape == x[:2].shape


def test_synaptic_layer_inference_writes_no_states():
    """The fused synaptic forward under ``torch.no_grad()`` without ``record_states``: spikes only."""
    import torch
    import sinabs_exodus_b200 as ex
    dev = "cuda:0"
    x = torch.rand(16, 200, 2048, device=dev) * 3.0
    mk = lambda **kw: ex.layers.LIF(tau_mem=20.0, tau_syn=8.0, **kw).to(dev)
    a, b = mk(), mk()
    out_a = a(x)
    torch.cuda.synchronize(); torch.cuda.reset_peak_memory_stats(); base = torch.cuda.memory_allocated()
    with torch.no_grad():
        out_b = b(x)
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated() - base
    assert out_a.sum() > 0
    torch.testing.assert_close(out_b, out_a.detach(), rtol=0, atol=0)
    torch.testing.assert_close(b.v_mem, a.v_mem.detach(), rtol=0, atol=0)
    torch.testing.assert_close(b.i_syn, a.i_syn.detach(), rtol=0, atol=0)
    assert peak < 1.5 * x.numel() * 4          # one output tensor, not three
    rec = mk(record_states=True)
    with torch.no_grad():
        rec(x[:2])
    assert rec.recordings["v_mem"].shape == x[:2].shape and rec.recordings["i_syn"].shape == x[:2].shape


def test_backward_recompute_in_a_captured_step():
    """``GraphedStep`` over a layer that trains without the v_mem tensor replays to the eager results."""
    import torch
    import sinabs_exodus_b200 as ex
    dev = "cuda:0"
    layer = ex.layers.LIF(tau_mem=15.0, norm_input=False).to(dev)
    layer.set_backward_recompute(True, always=True)
    g = torch.Generator(device=dev).manual_seed(8)
    xs = [torch.randn(4, 40, 64, device=dev, generator=g) + 0.4 for _ in range(3)]
    gos = [torch.randn(4, 40, 64, device=dev, generator=g) for _ in range(3)]

    def eager(x, go):
        layer.reset_states(); layer.zero_grad(set_to_none=True)
        x = x.clone().requires_grad_(True)
        out = layer(x)
        out.backward(go)
        return out.detach().clone(), x.grad.clone(), layer.tau_mem.grad.clone()

    want = [eager(x, go) for x, go in zip(xs, gos)]
    step = ex.GraphedStep(layer, xs[0], gos[0], carry_state=False, input_grad=True)
    for (out_w, gx_w, gt_w), x, go in zip(want, xs, gos):
        out = step(x, go)
        assert out_w.sum() > 0
        torch.testing.assert_close(out, out_w, rtol=0, atol=0)
        torch.testing.assert_close(step.input_grad, gx_w, rtol=0, atol=0)
        torch.testing.assert_close(layer.tau_mem.grad, gt_w, rtol=1e-6, atol=0)


def test_layer_step_with_nvtx_ranges_on():
    """The tracing aid changes nothing but the timeline."""
    import torch
    import sinabs_exodus_b200 as ex
    dev = "cuda:0"
    x = torch.rand(2, 30, 16, device=dev) * 2
    ref = ex.layers.LIF(tau_mem=10.0, norm_input=False).to(dev)
    want = ref(x)
    ex.set_nvtx_ranges(True)
    try:
        layer = ex.layers.LIF(tau_mem=10.0, norm_input=False).to(dev)
        xin = x.clone().requires_grad_(True)
        out = layer(xin)
        out.sum().backward()
    finally:
        ex.set_nvtx_ranges(False)
    torch.testing.assert_close(out.detach(), want.detach(), rtol=0, atol=0)
    assert xin.grad is not None and layer.tau_mem.grad is not None


def test_backward_recompute_is_used_only_where_it_pays_by_default():
    """Without ``always`` the switch leaves small problems on the ordinary pair (the rebuild costs more than the
    traffic it saves there): the v_mem tensor is still held after the forward; with ``always`` it is not."""
    import torch
    import sinabs_exodus_b200 as ex
    dev = "cuda:0"
    x = torch.rand(8, 100, 4096, device=dev) * 0.4       # 64 tiles of 512 neurons: far below eight per SM
    held = {}
    for key, kw in (("default", dict()), ("always", dict(always=True))):
        layer = ex.layers.LIF(tau_mem=20.0, norm_input=False).to(dev)
        layer.set_backward_recompute(True, **kw)
        xin = x.clone().requires_grad_(True)
        torch.cuda.synchronize(); before = torch.cuda.memory_allocated()
        out = layer(xin)
        held[key] = torch.cuda.memory_allocated() - before
        out.sum().backward()
    assert held["default"] > 1.9 * x.numel() * 4          # spikes + v_mem
    assert held["always"] < 1.3 * x.numel() * 4           # spikes + checkpoints
