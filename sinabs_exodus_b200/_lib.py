"""ctypes binding of ``libexodus_b200.so`` (declared in ``include/exodus_b200.h``).

The library is the only compute path.  If it is missing or a call fails, an
exception is raised; there is no PyTorch or CPU substitute.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libexodus_b200.so")

LAYOUT_NT = 0
LAYOUT_BTM = 1
PARAM_SCALAR = 0
PARAM_PER_M = 1
PARAM_PER_N = 2
PARAM_SHAPE_MASK = 3
PARAM_IS_TAU = 0x10                # on a decay argument: the values are time constants, alpha = exp(-1/tau)
SCALE_ONE_MINUS_ALPHA = 0x20       # on a scale argument (pointer None): scale = 1 - alpha of the same stage
SCALE_TIMES_ALPHA = 0x40           # on a scale argument: the scale is multiplied by alpha
RESET_SUBTRACT = 0
RESET_TO_VALUE = 1
SURR_GENERIC = 0
SURR_SINGLE_EXPONENTIAL = 1
SURR_HEAVISIDE = 2
SURR_PERIODIC_EXPONENTIAL = 3
MAX_SPIKES_UNLIMITED = 0xFFFFFFFF

_vp = ctypes.c_void_p
_i = ctypes.c_int
_i64 = ctypes.c_int64
_u32 = ctypes.c_uint32
_f = ctypes.c_float

_lib: Optional[ctypes.CDLL] = None

EXPORTS = (
    "exb_version", "exb_last_error", "exb_status_string", "exb_device_status", "exb_set_wait_limit", "exb_acc_finish", "exb_allreduce_oneshot",
    "exb_lif_forward", "exb_lif_forward_record", "exb_lif_forward_u8", "exb_lif_syn_forward_u8", "exb_lif_backward", "exb_lif_forward_ckpt", "exb_lif_backward_ckpt", "exb_leaky_forward", "exb_leaky_backward",
    "exb_leaky_scan_workspace_bytes", "exb_leaky_forward_scan", "exb_leaky_backward_scan",
    "exb_leaky_forward_scan_static", "exb_static_scratch_bytes", "exb_lif_syn_forward", "exb_lif_syn_backward",
)


class ExodusLibraryError(RuntimeError):
    """The CUDA library is missing or one of its entry points reported a failure."""


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ExodusLibraryError(
            f"{LIB_PATH} not found. Build it with `python -m sinabs_exodus_b200.build` "
            "(needs nvcc). There is no fallback implementation.")
    lib = ctypes.CDLL(LIB_PATH)
    lib.exb_version.restype = ctypes.c_char_p
    lib.exb_last_error.restype = ctypes.c_char_p
    lib.exb_status_string.restype = ctypes.c_char_p
    lib.exb_status_string.argtypes = [_i]
    lib.exb_device_status.restype = _i
    lib.exb_device_status.argtypes = [_i, _vp]
    lib.exb_set_wait_limit.restype = _i
    lib.exb_set_wait_limit.argtypes = [_i, _u32, _i]
    geometry = [_i64, _i64, _i64, _i, _i, _vp]
    lib.exb_lif_forward.restype = _i
    lib.exb_lif_forward.argtypes = [_vp, _vp, _vp, _vp,
                                    _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _i,
                                    _u32, _i, _vp, _vp] + geometry
    lib.exb_lif_forward_record.restype = _i
    lib.exb_lif_forward_record.argtypes = [_vp, _vp, _vp, _vp, _vp,
                                           _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _i,
                                           _u32, _i, _vp, _vp] + geometry
    lib.exb_lif_forward_u8.restype = _i
    lib.exb_lif_forward_u8.argtypes = [_vp, _vp, _vp, _vp,
                                       _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _i,
                                       _u32, _i, _i, _vp, _vp, _i64, _i64, _i64, _i, _vp]
    lib.exb_lif_forward_ckpt.restype = _i
    lib.exb_lif_forward_ckpt.argtypes = [_vp, _vp, _vp, _vp,
                                         _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _i,
                                         _u32, _i, _vp, _vp, _i64, _i64, _i64, _i, _vp]
    lib.exb_lif_backward_ckpt.restype = _i
    lib.exb_lif_backward_ckpt.argtypes = [_vp, _vp, _vp, _vp,
                                          _vp, _vp,
                                          _vp, _vp, _vp,
                                          _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _i,
                                          _u32, _i, _i, _f, _f, _vp, _i64, _i64, _i64, _i, _vp]
    lib.exb_lif_backward.restype = _i
    lib.exb_lif_backward.argtypes = [_vp, _vp, _vp, _vp,
                                     _vp, _vp, _vp,
                                     _vp, _vp, _vp, _vp,
                                     _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _i,
                                     _u32, _i, _i, _f, _f, _vp] + geometry
    lib.exb_allreduce_oneshot.restype = _i
    lib.exb_allreduce_oneshot.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i64, _u32, _i, _vp]
    lib.exb_acc_finish.restype = _i
    lib.exb_acc_finish.argtypes = [_vp, _vp, _i64, _i, _vp]
    lib.exb_leaky_forward.restype = _i
    lib.exb_leaky_forward.argtypes = [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _vp] + geometry
    lib.exb_leaky_backward.restype = _i
    lib.exb_leaky_backward.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                       _vp, _i, _vp, _i, _vp] + geometry
    lib.exb_leaky_scan_workspace_bytes.restype = _i64
    lib.exb_leaky_scan_workspace_bytes.argtypes = [_i64, _i64, _i64]
    scan_tail = [_vp, _i64, _i, _i64, _i64, _i64, _i, _vp]
    lib.exb_leaky_forward_scan.restype = _i
    lib.exb_leaky_forward_scan.argtypes = [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _vp] + scan_tail
    lib.exb_leaky_backward_scan.restype = _i
    lib.exb_leaky_backward_scan.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp] + scan_tail
    syn_params = [_vp, _i] * 7
    lib.exb_lif_syn_forward.restype = _i
    lib.exb_lif_syn_forward.argtypes = [_vp] * 6 + syn_params + [_u32, _i, _vp, _vp, _vp, _i64, _i64, _i64, _i, _vp]
    lib.exb_lif_syn_forward_u8.restype = _i
    lib.exb_lif_syn_forward_u8.argtypes = [_vp] * 6 + syn_params + [_u32, _i, _i, _vp, _vp, _vp, _i64, _i64, _i64, _i, _vp]
    lib.exb_lif_syn_backward.restype = _i
    lib.exb_lif_syn_backward.argtypes = ([_vp] * 17 + syn_params + [_u32, _i, _i, _f, _f, _vp, _vp, _i64, _i64, _i64, _i, _vp])
    lib.exb_static_scratch_bytes.restype = _i64
    lib.exb_static_scratch_bytes.argtypes = []
    lib.exb_leaky_forward_scan_static.restype = _i
    lib.exb_leaky_forward_scan_static.argtypes = [_vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _i64, _i64, _i64, _i, _vp]
    _lib = lib
    return lib


def version() -> str:
    return load().exb_version().decode()


def _check(status: int, what: str) -> None:
    if status != 0:
        lib = load()
        raise ExodusLibraryError(
            f"{what} failed: {lib.exb_status_string(status).decode()} -- {lib.exb_last_error().decode()}")


# Opt-in: query the device status after every launch.  Each query waits for the stream, so this is for
# debugging and for hosts that prefer a loud failure to speed; off unless EXODUS_B200_CHECK_STATUS=1 or
# set_status_checks(True).  Without it a wait that ran out shows as NaN in the layer state and in the
# per-neuron gradients, and in device_status() whenever the caller polls it.
_check_every_call = os.environ.get("EXODUS_B200_CHECK_STATUS", "0") == "1"


def set_status_checks(enabled: bool) -> None:
    """Poll ``exb_device_status`` after every kernel launch (synchronises the stream each time)."""
    global _check_every_call
    _check_every_call = bool(enabled)


def _after_launch(dev: torch.device) -> None:
    if _check_every_call and not torch.cuda.is_current_stream_capturing():
        device_status(dev)


def device_status(device: Optional[torch.device] = None) -> None:
    """Wait for the current stream of ``device`` and raise if a bounded device-side wait ran out."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _check(load().exb_device_status(dev.index, _stream(dev)), "exb_device_status")


def set_wait_limit(polls: int = 0, withhold_scan_flags: bool = False, device: Optional[torch.device] = None) -> None:
    """``exb_set_wait_limit``: poll limit of the kernels' bounded waits (0 = default) and the diagnostic switch
    that keeps the time-parallel scan's ready flags down (so that its waits run out)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _check(load().exb_set_wait_limit(dev.index, int(polls), int(bool(withhold_scan_flags))), "exb_set_wait_limit")


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _ptr_f64(t: Optional[torch.Tensor]):
    """Address of a one-element float64 CUDA accumulator (or None)."""
    if t is None:
        return None
    if not t.is_cuda or t.dtype != torch.float64 or t.numel() < 1:
        raise ExodusLibraryError("the sum accumulator must be a float64 CUDA tensor with one element")
    return t.data_ptr()


def _require_cuda(*tensors: Optional[torch.Tensor]) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise ExodusLibraryError(
                "exodus_b200 kernels only run on CUDA tensors; got a tensor on "
                f"{t.device}. There is no CPU implementation in this package.")
        if t.dtype != torch.float32:
            raise ExodusLibraryError(f"exodus_b200 kernels are float32 only; got {t.dtype}")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ExodusLibraryError(f"tensors on different devices: {dev} and {t.device}")
    assert dev is not None
    return dev


try:      # raw handle of the current stream without building a Stream object (a few microseconds per call less)
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:      # pragma: no cover - older PyTorch
    _raw_stream = None


def _stream(dev: torch.device):
    if _raw_stream is not None:
        return _raw_stream(dev.index)
    return torch.cuda.current_stream(dev).cuda_stream


class ParamSpec(tuple):
    """(tensor | None, mode) pair for a per-neuron parameter."""

    def __new__(cls, tensor: Optional[torch.Tensor], mode: int = PARAM_SCALAR):
        return super().__new__(cls, (tensor, mode))


def lif_forward(spikes, v_mem, inp, v_init, in_scale: Tuple, alpha: Tuple, subtract: Tuple, theta: Tuple,
                theta_low: Tuple, max_spikes: Optional[int], reset_mode: int, v_post_last, spike_count,
                B: int, T: int, M: int, layout: int, v_post=None) -> bool:
    """``v_post``: optional tensor like ``v_mem`` that receives the potential after each step's reset
    (time-major layout only).  ``v_mem`` may be None (spikes only); the call then returns False, without having
    launched anything, when the shape is not one the spikes-only kernels take."""
    if B * T * M == 0:      # empty problem: nothing to launch (empty tensors have no storage to point at)
        return True
    dev = _require_cuda(spikes, v_mem, inp, v_init, in_scale[0], alpha[0], subtract[0], theta[0], theta_low[0],
                        v_post_last, v_post)
    ms = MAX_SPIKES_UNLIMITED if max_spikes is None else int(max_spikes)
    tail = (ptr(in_scale[0]), in_scale[1], ptr(alpha[0]), alpha[1], ptr(subtract[0]), subtract[1],
            ptr(theta[0]), theta[1], ptr(theta_low[0]), theta_low[1],
            ms, reset_mode, ptr(v_post_last), ptr(spike_count),
            B, T, M, layout, dev.index, _stream(dev))
    if v_post is None:
        st = load().exb_lif_forward(ptr(spikes), ptr(v_mem), ptr(inp), ptr(v_init), *tail)
        if st == 4 and v_mem is None:
            return False        # spikes-only is for shapes the TMA-staged kernels take: the caller passes a v_mem tensor
        _check(st, "exb_lif_forward")
        _after_launch(dev)
    else:
        st = load().exb_lif_forward_record(ptr(spikes), ptr(v_mem), ptr(v_post), ptr(inp), ptr(v_init), *tail)
        _check(st, "exb_lif_forward_record")
        _after_launch(dev)
    return True


def _require_u8(t: torch.Tensor) -> None:
    if not t.is_cuda or t.dtype != torch.uint8 or not t.is_contiguous():
        raise ExodusLibraryError("the compact spike raster must be a contiguous uint8 CUDA tensor")


def lif_forward_u8(spikes_u8, v_mem, inp, v_init, in_scale: Tuple, alpha: Tuple, subtract: Tuple, theta: Tuple,
                   theta_low: Tuple, max_spikes: Optional[int], reset_mode: int, saturate: bool, v_post_last, spike_count,
                   B: int, T: int, M: int) -> bool:
    """``exb_lif_forward_u8``: spikes as one byte per neuron-step (``v_mem`` may be None).  Returns False when the
    shape is not eligible (the caller then uses :func:`lif_forward`)."""
    if B * T * M == 0:
        return True
    _require_u8(spikes_u8)
    dev = _require_cuda(v_mem, inp, v_init, in_scale[0], alpha[0], subtract[0], theta[0], theta_low[0], v_post_last)
    ms = MAX_SPIKES_UNLIMITED if max_spikes is None else int(max_spikes)
    st = load().exb_lif_forward_u8(
        ptr(spikes_u8), ptr(v_mem), ptr(inp), ptr(v_init), ptr(in_scale[0]), in_scale[1], ptr(alpha[0]), alpha[1],
        ptr(subtract[0]), subtract[1], ptr(theta[0]), theta[1], ptr(theta_low[0]), theta_low[1],
        ms, reset_mode, int(bool(saturate)), ptr(v_post_last), ptr(spike_count), B, T, M, dev.index, _stream(dev))
    if st == 4:
        return False
    _check(st, "exb_lif_forward_u8")
    _after_launch(dev)
    return True


def lif_backward(grad_input, grad_alpha, grad_init, grad_scale, grad_spikes, grad_v_mem, grad_v_last,
                 v_mem, surr, v_init, inp, in_scale: Tuple, alpha: Tuple, subtract: Tuple, theta: Tuple,
                 theta_low: Tuple, max_spikes: Optional[int], reset_mode: int,
                 surr_kind: int, p0: float, p1: float, B: int, T: int, M: int, layout: int, acc_decay=None) -> bool:
    """``acc_decay``: float64 accumulator shaped like the alpha argument (see the header).  Returns False when it was
    given and the shape is not one the reducing kernels take (nothing was launched)."""
    if B * T * M == 0:      # empty problem: nothing to launch (empty tensors have no storage to point at)
        return True
    dev = _require_cuda(grad_input, grad_alpha, grad_init, grad_scale, grad_spikes, grad_v_mem, grad_v_last,
                        v_mem, surr, v_init, inp, in_scale[0], alpha[0], subtract[0], theta[0], theta_low[0])
    ms = MAX_SPIKES_UNLIMITED if max_spikes is None else int(max_spikes)
    st = load().exb_lif_backward(
        ptr(grad_input), ptr(grad_alpha), ptr(grad_init), ptr(grad_scale),
        ptr(grad_spikes), ptr(grad_v_mem), ptr(grad_v_last),
        ptr(v_mem), ptr(surr), ptr(v_init), ptr(inp),
        ptr(in_scale[0]), in_scale[1], ptr(alpha[0]), alpha[1], ptr(subtract[0]), subtract[1],
        ptr(theta[0]), theta[1], ptr(theta_low[0]), theta_low[1],
        ms, reset_mode, surr_kind, float(p0), float(p1), _ptr_f64(acc_decay),
        B, T, M, layout, dev.index, _stream(dev))
    if st == 4 and acc_decay is not None:
        return False
    _check(st, "exb_lif_backward")
    _after_launch(dev)
    return True


CKPT_EVERY = 8      # EXB_CKPT_EVERY of the header


def ckpt_shape(B: int, T: int, M: int) -> Tuple[int, int, int]:
    """Shape of the checkpoint tensor of :func:`lif_forward_ckpt`."""
    return (B, (T + CKPT_EVERY - 1) // CKPT_EVERY, M)


def lif_forward_ckpt(spikes, ckpt, inp, v_init, in_scale: Tuple, alpha: Tuple, subtract: Tuple, theta: Tuple,
                     theta_low: Tuple, max_spikes: Optional[int], reset_mode: int, v_post_last, spike_count,
                     B: int, T: int, M: int) -> bool:
    """``exb_lif_forward_ckpt``: spikes and, instead of ``v_mem``, the state entering every ``CKPT_EVERY``-th step
    (``ckpt``: float32 tensor of :func:`ckpt_shape`).  Returns False when the shape is not eligible (the caller then
    uses :func:`lif_forward`)."""
    if B * T * M == 0:
        return False
    dev = _require_cuda(spikes, ckpt, inp, v_init, in_scale[0], alpha[0], subtract[0], theta[0], theta_low[0], v_post_last)
    if tuple(ckpt.shape) != ckpt_shape(B, T, M) or not ckpt.is_contiguous():
        raise ExodusLibraryError(f"ckpt must be a contiguous float32 tensor of shape {ckpt_shape(B, T, M)}")
    ms = MAX_SPIKES_UNLIMITED if max_spikes is None else int(max_spikes)
    st = load().exb_lif_forward_ckpt(
        ptr(spikes), ptr(ckpt), ptr(inp), ptr(v_init), ptr(in_scale[0]), in_scale[1], ptr(alpha[0]), alpha[1],
        ptr(subtract[0]), subtract[1], ptr(theta[0]), theta[1], ptr(theta_low[0]), theta_low[1],
        ms, reset_mode, ptr(v_post_last), ptr(spike_count), B, T, M, dev.index, _stream(dev))
    if st == 4:
        return False
    _check(st, "exb_lif_forward_ckpt")
    _after_launch(dev)
    return True


def lif_backward_ckpt(grad_input, grad_alpha, grad_init, grad_scale, grad_spikes, grad_v_last, inp, ckpt, v_init,
                      in_scale: Tuple, alpha: Tuple, subtract: Tuple, theta: Tuple, theta_low: Tuple,
                      max_spikes: Optional[int], reset_mode: int, surr_kind: int, p0: float, p1: float,
                      B: int, T: int, M: int, acc_decay=None) -> None:
    """``exb_lif_backward_ckpt``: the backward pass of :func:`lif_forward_ckpt` (same shapes are eligible)."""
    if B * T * M == 0:
        return
    dev = _require_cuda(grad_input, grad_alpha, grad_init, grad_scale, grad_spikes, grad_v_last, inp, ckpt, v_init,
                        in_scale[0], alpha[0], subtract[0], theta[0], theta_low[0])
    ms = MAX_SPIKES_UNLIMITED if max_spikes is None else int(max_spikes)
    st = load().exb_lif_backward_ckpt(
        ptr(grad_input), ptr(grad_alpha), ptr(grad_init), ptr(grad_scale), ptr(grad_spikes), ptr(grad_v_last),
        ptr(inp), ptr(ckpt), ptr(v_init),
        ptr(in_scale[0]), in_scale[1], ptr(alpha[0]), alpha[1], ptr(subtract[0]), subtract[1],
        ptr(theta[0]), theta[1], ptr(theta_low[0]), theta_low[1],
        ms, reset_mode, surr_kind, float(p0), float(p1), _ptr_f64(acc_decay), B, T, M, dev.index, _stream(dev))
    _check(st, "exb_lif_backward_ckpt")
    _after_launch(dev)


def allreduce_oneshot(out: torch.Tensor, inp: torch.Tensor, buffers: torch.Tensor, signals: torch.Tensor, rank: int,
                      world: int, epoch: int) -> None:
    """``exb_allreduce_oneshot``; ``buffers`` / ``signals``: int64 CUDA tensors holding the ``world`` peer addresses."""
    dev = _require_cuda(out, inp)
    n = inp.numel()
    if out.numel() != n or not (out.is_contiguous() and inp.is_contiguous()):
        raise ExodusLibraryError("allreduce_oneshot needs contiguous float32 vectors of equal length")
    st = load().exb_allreduce_oneshot(out.data_ptr(), inp.data_ptr(), buffers.data_ptr(), signals.data_ptr(), rank, world,
                                      n, epoch, dev.index, _stream(dev))
    _check(st, "exb_allreduce_oneshot")


def acc_finish(out: torch.Tensor, acc: torch.Tensor) -> None:
    """``exb_acc_finish``: ``out[i] = float(acc[i]); acc[i] = 0`` (float64 accumulators -> float32 gradients)."""
    n = out.numel()
    if n == 0:
        return
    if not (out.is_cuda and out.dtype == torch.float32 and out.is_contiguous() and acc.is_cuda
            and acc.dtype == torch.float64 and acc.is_contiguous() and acc.numel() >= n):
        raise ExodusLibraryError("acc_finish needs a contiguous float32 output and a float64 accumulator of at least its size")
    dev = out.device
    _check(load().exb_acc_finish(out.data_ptr(), acc.data_ptr(), n, dev.index, _stream(dev)), "exb_acc_finish")


def leaky_forward(out, inp, v_init, alpha: Tuple, in_scale: Tuple, v_last, B: int, T: int, M: int,
                  layout: int, out_sum=None) -> None:
    """``out_sum``: optional float64 tensor of one element (zeroed by the caller) that receives sum(out)."""
    if B * T * M == 0:      # empty problem: nothing to launch (empty tensors have no storage to point at)
        return
    dev = _require_cuda(out, inp, v_init, alpha[0], in_scale[0], v_last)
    st = load().exb_leaky_forward(ptr(out), ptr(inp), ptr(v_init), ptr(alpha[0]), alpha[1],
                                  ptr(in_scale[0]), in_scale[1], ptr(v_last), _ptr_f64(out_sum),
                                  B, T, M, layout, dev.index, _stream(dev))
    _check(st, "exb_leaky_forward")
    _after_launch(dev)


def leaky_backward(grad_input, grad_alpha, grad_init, grad_scale, grad_out, grad_v_last, out, inp, v_init,
                   alpha: Tuple, in_scale: Tuple, B: int, T: int, M: int, layout: int, acc_decay=None) -> bool:
    if B * T * M == 0:      # empty problem: nothing to launch (empty tensors have no storage to point at)
        return True
    dev = _require_cuda(grad_input, grad_alpha, grad_init, grad_scale, grad_out, grad_v_last, out, inp, v_init,
                        alpha[0], in_scale[0])
    st = load().exb_leaky_backward(ptr(grad_input), ptr(grad_alpha), ptr(grad_init), ptr(grad_scale),
                                   ptr(grad_out), ptr(grad_v_last), ptr(out), ptr(inp), ptr(v_init),
                                   ptr(alpha[0]), alpha[1], ptr(in_scale[0]), in_scale[1], _ptr_f64(acc_decay),
                                   B, T, M, layout, dev.index, _stream(dev))
    if st == 4 and acc_decay is not None:
        return False
    _check(st, "exb_leaky_backward")
    _after_launch(dev)
    return True


def leaky_scan_workspace_bytes(B: int, T: int, M: int) -> int:
    """Scratch bytes the time-parallel leaky scan needs for this shape; 0 when it does not apply."""
    return int(load().exb_leaky_scan_workspace_bytes(B, T, M))


def leaky_forward_scan(out, inp, v_init, alpha: Tuple, in_scale: Tuple, v_last, workspace, B: int, T: int,
                       M: int, out_sum=None, clean: bool = False) -> None:
    dev = _require_cuda(out, inp, v_init, alpha[0], in_scale[0], v_last)
    st = load().exb_leaky_forward_scan(ptr(out), ptr(inp), ptr(v_init), ptr(alpha[0]), alpha[1],
                                       ptr(in_scale[0]), in_scale[1], ptr(v_last), _ptr_f64(out_sum),
                                       workspace.data_ptr(), workspace.numel() * workspace.element_size(), int(clean),
                                       B, T, M, dev.index, _stream(dev))
    _check(st, "exb_leaky_forward_scan")
    _after_launch(dev)


def leaky_backward_scan(grad_input, grad_alpha, grad_init, grad_scale, grad_out, grad_v_last, out, inp, v_init,
                        alpha: Tuple, in_scale: Tuple, workspace, B: int, T: int, M: int, acc_decay=None,
                        clean: bool = False) -> None:
    dev = _require_cuda(grad_input, grad_alpha, grad_init, grad_scale, grad_out, grad_v_last, out, inp, v_init,
                        alpha[0], in_scale[0])
    st = load().exb_leaky_backward_scan(ptr(grad_input), ptr(grad_alpha), ptr(grad_init), ptr(grad_scale),
                                        ptr(grad_out), ptr(grad_v_last), ptr(out), ptr(inp), ptr(v_init),
                                        ptr(alpha[0]), alpha[1], ptr(in_scale[0]), in_scale[1], _ptr_f64(acc_decay),
                                        workspace.data_ptr(), workspace.numel() * workspace.element_size(), int(clean),
                                        B, T, M, dev.index, _stream(dev))
    _check(st, "exb_leaky_backward_scan")
    _after_launch(dev)


def static_scratch_bytes() -> int:
    """Size of the library's built-in scratch array (``EXB_STATIC_SCRATCH_BYTES``), asked from the library."""
    return int(load().exb_static_scratch_bytes())


def __getattr__(name: str):
    if name == "STATIC_SCRATCH_BYTES":      # kept as a module attribute; the value lives in the library
        return static_scratch_bytes()
    raise AttributeError(name)


def leaky_forward_scan_static(out, inp, v_init, alpha: Tuple, in_scale: Tuple, v_last, B: int, T: int, M: int) -> None:
    """``exb_leaky_forward_scan_static``: the forward scan on the library's built-in scratch array.

    For hosts that must not allocate device memory once they are running (fixed memory budget,
    foreign memory pool).  Shapes that need more than ``STATIC_SCRATCH_BYTES`` raise.  Calls share
    the array: do not let two of them run on the GPU at the same time.
    """
    dev = _require_cuda(out, inp, v_init, alpha[0], in_scale[0], v_last)
    st = load().exb_leaky_forward_scan_static(ptr(out), ptr(inp), ptr(v_init), ptr(alpha[0]), alpha[1],
                                              ptr(in_scale[0]), in_scale[1], ptr(v_last),
                                              B, T, M, dev.index, _stream(dev))
    _check(st, "exb_leaky_forward_scan_static")
    _after_launch(dev)


def _pm(spec):
    return ptr(spec[0]), spec[1]


def lif_syn_forward(spikes, v_mem, i_syn, inp, v_init, i_init, alpha_syn: Tuple, scale_syn: Tuple, scale_mem: Tuple,
                    alpha_mem: Tuple, subtract: Tuple, theta: Tuple, theta_low: Tuple, max_spikes: Optional[int],
                    reset_mode: int, v_post_last, i_last, spike_count, B: int, T: int, M: int) -> bool:
    """``exb_lif_syn_forward``.  Returns False when the shape is not eligible for the fused kernel."""
    dev = _require_cuda(spikes, v_mem, i_syn, inp, v_init, i_init, alpha_syn[0], scale_syn[0], scale_mem[0],
                        alpha_mem[0], subtract[0], theta[0], theta_low[0], v_post_last, i_last)
    ms = MAX_SPIKES_UNLIMITED if max_spikes is None else int(max_spikes)
    st = load().exb_lif_syn_forward(
        ptr(spikes), ptr(v_mem), ptr(i_syn), ptr(inp), ptr(v_init), ptr(i_init),
        *_pm(alpha_syn), *_pm(scale_syn), *_pm(scale_mem), *_pm(alpha_mem), *_pm(subtract), *_pm(theta), *_pm(theta_low),
        ms, reset_mode, ptr(v_post_last), ptr(i_last), ptr(spike_count), B, T, M, dev.index, _stream(dev))
    if st == 4:
        return False
    _check(st, "exb_lif_syn_forward")
    _after_launch(dev)
    return True


def lif_syn_forward_u8(spikes_u8, v_mem, i_syn, inp, v_init, i_init, alpha_syn: Tuple, scale_syn: Tuple, scale_mem: Tuple,
                       alpha_mem: Tuple, subtract: Tuple, theta: Tuple, theta_low: Tuple, max_spikes: Optional[int],
                       reset_mode: int, saturate: bool, v_post_last, i_last, spike_count, B: int, T: int, M: int) -> bool:
    """``exb_lif_syn_forward_u8`` (``v_mem`` and ``i_syn`` both given or both None).  False when not eligible."""
    if B * T * M == 0:
        return True
    _require_u8(spikes_u8)
    dev = _require_cuda(v_mem, i_syn, inp, v_init, i_init, alpha_syn[0], scale_syn[0], scale_mem[0], alpha_mem[0],
                        subtract[0], theta[0], theta_low[0], v_post_last, i_last)
    ms = MAX_SPIKES_UNLIMITED if max_spikes is None else int(max_spikes)
    st = load().exb_lif_syn_forward_u8(
        ptr(spikes_u8), ptr(v_mem), ptr(i_syn), ptr(inp), ptr(v_init), ptr(i_init),
        *_pm(alpha_syn), *_pm(scale_syn), *_pm(scale_mem), *_pm(alpha_mem), *_pm(subtract), *_pm(theta), *_pm(theta_low),
        ms, reset_mode, int(bool(saturate)), ptr(v_post_last), ptr(i_last), ptr(spike_count), B, T, M, dev.index, _stream(dev))
    if st == 4:
        return False
    _check(st, "exb_lif_syn_forward_u8")
    _after_launch(dev)
    return True


def lif_syn_backward(grad_input, grad_alpha_mem, grad_scale_mem, grad_alpha_syn, grad_scale_syn, grad_v_init,
                     grad_i_init, grad_spikes, grad_v_mem, grad_v_last, grad_i_syn, grad_i_last, v_mem, i_syn, surr,
                     v_init, i_init, alpha_syn: Tuple, scale_syn: Tuple, scale_mem: Tuple, alpha_mem: Tuple,
                     subtract: Tuple, theta: Tuple, theta_low: Tuple, max_spikes: Optional[int], reset_mode: int,
                     surr_kind: int, p0: float, p1: float, B: int, T: int, M: int, acc_decay_mem=None,
                     acc_decay_syn=None) -> None:
    dev = _require_cuda(grad_input, grad_alpha_mem, grad_scale_mem, grad_alpha_syn, grad_scale_syn, grad_v_init,
                        grad_i_init, grad_spikes, grad_v_mem, grad_v_last, grad_i_syn, grad_i_last, v_mem, i_syn, surr,
                        v_init, i_init, alpha_syn[0], scale_syn[0], scale_mem[0], alpha_mem[0], subtract[0], theta[0],
                        theta_low[0])
    ms = MAX_SPIKES_UNLIMITED if max_spikes is None else int(max_spikes)
    st = load().exb_lif_syn_backward(
        ptr(grad_input), ptr(grad_alpha_mem), ptr(grad_scale_mem), ptr(grad_alpha_syn), ptr(grad_scale_syn),
        ptr(grad_v_init), ptr(grad_i_init), ptr(grad_spikes), ptr(grad_v_mem), ptr(grad_v_last), ptr(grad_i_syn),
        ptr(grad_i_last), ptr(v_mem), ptr(i_syn), ptr(surr), ptr(v_init), ptr(i_init),
        *_pm(alpha_syn), *_pm(scale_syn), *_pm(scale_mem), *_pm(alpha_mem), *_pm(subtract), *_pm(theta), *_pm(theta_low),
        ms, reset_mode, surr_kind, float(p0), float(p1), _ptr_f64(acc_decay_mem), _ptr_f64(acc_decay_syn),
        B, T, M, dev.index, _stream(dev))
    _check(st, "exb_lif_syn_backward")
    _after_launch(dev)


# Tracing aid: NVTX ranges around the calls that launch kernels, named after the entry point, so that a timeline
# shows which layer call a kernel belongs to.  Off unless asked for (a range costs a few microseconds per call).
_LAUNCHERS = ("lif_forward", "lif_forward_u8", "lif_forward_ckpt", "lif_backward", "lif_backward_ckpt", "leaky_forward",
              "leaky_backward", "leaky_forward_scan", "leaky_backward_scan", "leaky_forward_scan_static",
              "lif_syn_forward", "lif_syn_forward_u8", "lif_syn_backward", "acc_finish", "allreduce_oneshot")
_nvtx_on = False


def set_nvtx_ranges(enabled: bool = True) -> None:
    """Wrap every launching call of this module in an NVTX range ``exb.<name>`` (``EXODUS_B200_NVTX=1`` in the
    environment does the same at import)."""
    global _nvtx_on
    if bool(enabled) == _nvtx_on:
        return
    module = globals()
    for name in _LAUNCHERS:
        fn = module[name]
        if enabled:
            def ranged(*args, __fn=fn, __label="exb." + name, **kwargs):
                torch.cuda.nvtx.range_push(__label)
                try:
                    return __fn(*args, **kwargs)
                finally:
                    torch.cuda.nvtx.range_pop()
            ranged.__wrapped__ = fn
            ranged.__doc__ = fn.__doc__
            module[name] = ranged
        else:
            module[name] = getattr(fn, "__wrapped__", fn)
    _nvtx_on = bool(enabled)


if os.environ.get("EXODUS_B200_NVTX", "0") == "1":
    set_nvtx_ranges(True)
