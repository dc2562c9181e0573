"""numpy-in / numpy-out helpers that call the C-ABI of libexodus_b200.so on cuda:0.

Problems are given in the [N, T] layout with N = B*M (row n = b*M + m); the
helpers rearrange them to the requested device layout, call the entry point
through ``sinabs_exodus_b200._lib`` (ctypes), and bring the results back to [N, T].
"""
from __future__ import annotations

import numpy as np
import torch

from sinabs_exodus_b200 import _lib

DEV = "cuda:0"


def to_dev(a_nt, B, M, layout):
    """[N,T] numpy -> device tensor in `layout`."""
    if a_nt is None:
        return None
    N, T = a_nt.shape
    t = torch.tensor(np.ascontiguousarray(a_nt, np.float32), device=DEV)
    if layout == _lib.LAYOUT_BTM:
        t = t.view(B, M, T).permute(0, 2, 1).contiguous()
    return t


def from_dev(t, B, M, layout):
    if layout == _lib.LAYOUT_BTM:
        t = t.permute(0, 2, 1).contiguous().view(B * M, -1)
    return t.cpu().numpy()


def param(vec_n, mode, B, M):
    """Pick the representation of a per-neuron vector for `mode`; vec_n has N entries that
    must already be consistent with the mode (constant / periodic in M / free)."""
    if vec_n is None:
        return (None, _lib.PARAM_SCALAR)
    v = np.asarray(vec_n, np.float32)
    if mode == _lib.PARAM_SCALAR:
        v = v[:1]
    elif mode == _lib.PARAM_PER_M:
        v = v[:M]
    return (torch.tensor(np.ascontiguousarray(v), device=DEV), mode)


def vec(a):
    return None if a is None else torch.tensor(np.ascontiguousarray(a, np.float32), device=DEV)


def lif_forward(cs, B, M, layout, mode=_lib.PARAM_PER_N, max_spikes=None, reset_mode=_lib.RESET_SUBTRACT,
                in_scale=None, want_count=True, elem_offset=0):
    """``elem_offset`` ([N,T] layout): the three tensors start that many floats into their allocations, which are
    filled with a sentinel around them; the sentinel must survive the call."""
    N, T = cs["inp"].shape
    x = to_dev(cs["inp"], B, M, layout)
    guards = []
    if elem_offset:
        assert layout == _lib.LAYOUT_NT
        def carve(fill):
            buf = torch.full((elem_offset + N * T + 64,), -12345.0, device=DEV)
            guards.append(buf)
            view = buf[elem_offset:elem_offset + N * T].view(N, T)
            view.fill_(fill)
            return view
        xs = carve(0.0); xs.copy_(x); x = xs
        spikes = carve(float("nan")); v_mem = carve(float("nan"))
    else:
        spikes = torch.full_like(x, float("nan")); v_mem = torch.full_like(x, float("nan"))
    v_post = torch.empty(N, device=DEV)
    count = torch.zeros(1, dtype=torch.int64, device=DEV) if want_count else None
    _lib.lif_forward(spikes, v_mem, x, vec(cs["v_init"]), param(in_scale, mode, B, M), param(cs["alpha"], mode, B, M),
                     param(cs["subtract"], mode, B, M), param(cs["theta"], mode, B, M),
                     param(cs["theta_low"], mode, B, M), max_spikes, reset_mode, v_post, count, B, T, M, layout)
    torch.cuda.synchronize()
    for buf in guards:
        assert bool((buf[:elem_offset] == -12345.0).all()) and bool((buf[elem_offset + N * T:] == -12345.0).all()), \
            "the kernel wrote outside its tensors"
    return (from_dev(spikes, B, M, layout), from_dev(v_mem, B, M, layout), v_post.cpu().numpy(),
            int(count.item()) if want_count else None)


def lif_backward(cs, v_mem, go, B, M, layout, mode=_lib.PARAM_PER_N, gv=None, g_last=None, surr=None,
                 kind=_lib.SURR_GENERIC, p0=0.0, p1=0.0, max_spikes=None, reset_mode=_lib.RESET_SUBTRACT,
                 want_alpha=False, in_scale=None, want_scale=False, want_init=True, scale_from_state=False):
    N, T = v_mem.shape
    gi = torch.full((N, T), float("nan"), device=DEV)
    gi = to_dev(gi.cpu().numpy(), B, M, layout)
    ga = torch.empty(N, device=DEV) if want_alpha else None
    g0 = torch.empty(N, device=DEV) if want_init else None
    gs = torch.empty(N, device=DEV) if want_scale else None
    _lib.lif_backward(gi, ga, g0, gs, to_dev(go, B, M, layout), to_dev(gv, B, M, layout), vec(g_last),
                      to_dev(v_mem, B, M, layout), to_dev(surr, B, M, layout), vec(cs["v_init"]),
                      to_dev(cs["inp"], B, M, layout) if (want_scale and not scale_from_state) else None,
                      param(in_scale, mode, B, M), param(cs["alpha"], mode, B, M), param(cs["subtract"], mode, B, M),
                      param(cs["theta"], mode, B, M), param(cs["theta_low"], mode, B, M), max_spikes, reset_mode,
                      kind, p0, p1, B, T, M, layout)
    torch.cuda.synchronize()
    cpu = lambda t: None if t is None else t.cpu().numpy()
    return from_dev(gi, B, M, layout), cpu(ga), cpu(g0), cpu(gs)


def lif_forward_ckpt(cs, B, M, mode=_lib.PARAM_PER_N, max_spikes=None, reset_mode=_lib.RESET_SUBTRACT, in_scale=None):
    """exb_lif_forward_ckpt on the time-major layout.  Returns (spikes [N,T], ckpt [N, ceil(T/8)], v_post_last, count,
    device tensors (x, ckpt) for the backward) or None when the shape is not eligible."""
    N, T = cs["inp"].shape
    x = to_dev(cs["inp"], B, M, _lib.LAYOUT_BTM)
    spikes = torch.full_like(x, float("nan"))
    ckpt = torch.full(_lib.ckpt_shape(B, T, M), float("nan"), device=DEV)
    v_post = torch.empty(N, device=DEV)
    count = torch.zeros(1, dtype=torch.int64, device=DEV)
    ok = _lib.lif_forward_ckpt(spikes, ckpt, x, vec(cs["v_init"]), param(in_scale, mode, B, M), param(cs["alpha"], mode, B, M),
                               param(cs["subtract"], mode, B, M), param(cs["theta"], mode, B, M),
                               param(cs["theta_low"], mode, B, M), max_spikes, reset_mode, v_post, count, B, T, M)
    if not ok:
        return None
    torch.cuda.synchronize()
    return (from_dev(spikes, B, M, _lib.LAYOUT_BTM), from_dev(ckpt, B, M, _lib.LAYOUT_BTM), v_post.cpu().numpy(),
            int(count.item()), (x, ckpt))


def lif_backward_ckpt(cs, dev_tensors, go, B, M, mode=_lib.PARAM_PER_N, g_last=None, kind=_lib.SURR_SINGLE_EXPONENTIAL,
                      p0=0.5, p1=1.0, max_spikes=None, reset_mode=_lib.RESET_SUBTRACT, want_alpha=False, in_scale=None,
                      want_scale=False, want_init=True):
    x, ckpt = dev_tensors
    N, T = go.shape
    gi = torch.full_like(x, float("nan"))
    ga = torch.empty(N, device=DEV) if want_alpha else None
    g0 = torch.empty(N, device=DEV) if want_init else None
    gs = torch.empty(N, device=DEV) if want_scale else None
    _lib.lif_backward_ckpt(gi, ga, g0, gs, to_dev(go, B, M, _lib.LAYOUT_BTM), vec(g_last), x, ckpt, vec(cs["v_init"]),
                           param(in_scale, mode, B, M), param(cs["alpha"], mode, B, M), param(cs["subtract"], mode, B, M),
                           param(cs["theta"], mode, B, M), param(cs["theta_low"], mode, B, M), max_spikes, reset_mode,
                           kind, p0, p1, B, T, M)
    torch.cuda.synchronize()
    cpu = lambda t: None if t is None else t.cpu().numpy()
    return from_dev(gi, B, M, _lib.LAYOUT_BTM), cpu(ga), cpu(g0), cpu(gs)


def _check_total(total, out):
    """The sum of the outputs that the forward kernel accumulates on the side."""
    ref = out.double().sum().item()
    scale = out.double().abs().sum().item() + 1e-30
    assert abs(total.item() - ref) <= 1e-6 * scale, (total.item(), ref)


def leaky_forward(inp, v_init, alpha, B, M, layout, mode=_lib.PARAM_PER_N, in_scale=None):
    N, T = inp.shape
    x = to_dev(inp, B, M, layout)
    out = torch.full_like(x, float("nan"))
    v_last = torch.empty(N, device=DEV)
    total = torch.zeros(1, dtype=torch.float64, device=DEV)
    _lib.leaky_forward(out, x, vec(v_init), param(alpha, mode, B, M), param(in_scale, mode, B, M), v_last,
                       B, T, M, layout, out_sum=total)
    torch.cuda.synchronize()
    _check_total(total, out)
    return from_dev(out, B, M, layout), v_last.cpu().numpy()


def leaky_backward(go, alpha, B, M, layout, mode=_lib.PARAM_PER_N, out=None, inp=None, v_init=None, g_last=None,
                   in_scale=None, want_alpha=False, want_scale=False):
    N, T = go.shape
    g = to_dev(go, B, M, layout)
    gi = torch.full_like(g, float("nan"))
    ga = torch.empty(N, device=DEV) if want_alpha else None
    g0 = torch.empty(N, device=DEV)
    gs = torch.empty(N, device=DEV) if want_scale else None
    _lib.leaky_backward(gi, ga, g0, gs, g, vec(g_last), to_dev(out, B, M, layout) if want_alpha else None,
                        to_dev(inp, B, M, layout) if want_scale else None, vec(v_init),
                        param(alpha, mode, B, M), param(in_scale, mode, B, M), B, T, M, layout)
    torch.cuda.synchronize()
    cpu = lambda t: None if t is None else t.cpu().numpy()
    return from_dev(gi, B, M, layout), cpu(ga), cpu(g0), cpu(gs)


def leaky_forward_scan(inp, v_init, alpha, B, M, mode=_lib.PARAM_PER_N, in_scale=None):
    """Time-parallel variant; returns None when the library says the shape is not eligible."""
    N, T = inp.shape
    nbytes = _lib.leaky_scan_workspace_bytes(B, T, M)
    if nbytes == 0:
        return None
    ws = torch.empty((nbytes + 3) // 4, dtype=torch.int32, device=DEV)
    x = to_dev(inp, B, M, _lib.LAYOUT_BTM)
    out = torch.full_like(x, float("nan"))
    v_last = torch.empty(N, device=DEV)
    total = torch.zeros(1, dtype=torch.float64, device=DEV)
    _lib.leaky_forward_scan(out, x, vec(v_init), param(alpha, mode, B, M), param(in_scale, mode, B, M), v_last, ws,
                            B, T, M, out_sum=total)
    torch.cuda.synchronize()
    _check_total(total, out)
    return from_dev(out, B, M, _lib.LAYOUT_BTM), v_last.cpu().numpy()


def leaky_backward_scan(go, alpha, B, M, mode=_lib.PARAM_PER_N, out=None, inp=None, v_init=None, g_last=None,
                        in_scale=None, want_alpha=False, want_scale=False):
    N, T = go.shape
    nbytes = _lib.leaky_scan_workspace_bytes(B, T, M)
    if nbytes == 0:
        return None
    ws = torch.empty((nbytes + 3) // 4, dtype=torch.int32, device=DEV)
    L = _lib.LAYOUT_BTM
    g = to_dev(go, B, M, L)
    gi = torch.full_like(g, float("nan"))
    ga = torch.full((N,), float("nan"), device=DEV) if want_alpha else None
    g0 = torch.empty(N, device=DEV)
    gs = torch.full((N,), float("nan"), device=DEV) if want_scale else None
    _lib.leaky_backward_scan(gi, ga, g0, gs, g, vec(g_last), to_dev(out, B, M, L) if want_alpha else None,
                             to_dev(inp, B, M, L) if want_scale else None, vec(v_init),
                             param(alpha, mode, B, M), param(in_scale, mode, B, M), ws, B, T, M)
    torch.cuda.synchronize()
    cpu = lambda t: None if t is None else t.cpu().numpy()
    return from_dev(gi, B, M, L), cpu(ga), cpu(g0), cpu(gs)


def lif_syn_forward(inp, v_init, i_init, a_syn, s_syn, s_mem, a_mem, subtract, theta, theta_low, B, M,
                    mode=_lib.PARAM_PER_N, max_spikes=None, reset_mode=_lib.RESET_SUBTRACT):
    """exb_lif_syn_forward on an [N,T] problem (time-major on the device).  Per-neuron arguments hold N values
    consistent with `mode`.  Returns (spikes, v_mem, i_syn) as [N,T], v_post_last, i_last, spike count; None when
    the library says the shape is not eligible for the fused kernel."""
    N, T = inp.shape
    L = _lib.LAYOUT_BTM
    x = to_dev(inp, B, M, L)
    spikes = torch.full_like(x, float("nan")); v_mem = torch.full_like(x, float("nan")); i_syn = torch.full_like(x, float("nan"))
    v_post = torch.full((N,), float("nan"), device=DEV); i_last = torch.full((N,), float("nan"), device=DEV)
    count = torch.zeros(1, dtype=torch.int64, device=DEV)
    ok = _lib.lif_syn_forward(spikes, v_mem, i_syn, x, vec(v_init), vec(i_init), param(a_syn, mode, B, M),
                              param(s_syn, mode, B, M), param(s_mem, mode, B, M), param(a_mem, mode, B, M),
                              param(subtract, mode, B, M), param(theta, mode, B, M), param(theta_low, mode, B, M),
                              max_spikes, reset_mode, v_post, i_last, count, B, T, M)
    if not ok:
        return None
    torch.cuda.synchronize()
    return (from_dev(spikes, B, M, L), from_dev(v_mem, B, M, L), from_dev(i_syn, B, M, L), v_post.cpu().numpy(),
            i_last.cpu().numpy(), int(count.item()))


def lif_syn_backward(go, v_mem, i_syn, v_init, i_init, a_syn, s_syn, s_mem, a_mem, subtract, theta, theta_low, B, M,
                     mode=_lib.PARAM_PER_N, max_spikes=None, reset_mode=_lib.RESET_SUBTRACT, kind=_lib.SURR_GENERIC,
                     p0=0.0, p1=0.0, surr=None, gv=None, g_vlast=None, g_isyn=None, g_ilast=None, want_params=True,
                     want_init=True):
    """exb_lif_syn_backward; [N,T] numpy in and out.  Returns dict of numpy arrays (absent outputs are None)."""
    N, T = v_mem.shape
    L = _lib.LAYOUT_BTM
    nan_n = lambda: torch.full((N,), float("nan"), device=DEV)
    gi = torch.full((B, T, M), float("nan"), device=DEV)
    gam, gsm, gas, gss = (nan_n(), nan_n(), nan_n(), nan_n()) if want_params else (None,) * 4
    gv0, gi0 = (nan_n(), nan_n()) if want_init else (None, None)
    _lib.lif_syn_backward(gi, gam, gsm, gas, gss, gv0, gi0, to_dev(go, B, M, L), to_dev(gv, B, M, L), vec(g_vlast),
                          to_dev(g_isyn, B, M, L), vec(g_ilast), to_dev(v_mem, B, M, L),
                          to_dev(i_syn, B, M, L) if want_params else None, to_dev(surr, B, M, L), vec(v_init),
                          vec(i_init), param(a_syn, mode, B, M), param(s_syn, mode, B, M), param(s_mem, mode, B, M),
                          param(a_mem, mode, B, M), param(subtract, mode, B, M), param(theta, mode, B, M),
                          param(theta_low, mode, B, M), max_spikes, reset_mode, kind, p0, p1, B, T, M)
    torch.cuda.synchronize()
    cpu = lambda t: None if t is None else t.cpu().numpy()
    return dict(grad_input=from_dev(gi, B, M, L), grad_alpha_mem=cpu(gam), grad_scale_mem=cpu(gsm),
                grad_alpha_syn=cpu(gas), grad_scale_syn=cpu(gss), grad_v_init=cpu(gv0), grad_i_init=cpu(gi0))
