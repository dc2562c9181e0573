"""The C-ABI library loads and exports everything ``include/exodus_b200.h`` declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from sinabs_exodus_b200 import build, _lib
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "exodus_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(exb_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 7
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/exodus_b200.h but not exported"


def test_python_binding_covers_header(lib):
    from sinabs_exodus_b200 import _lib
    assert set(declared_symbols()) == set(_lib.EXPORTS)


def test_version_and_status_strings(lib):
    assert b"sm_100a" in lib.exb_version()
    assert lib.exb_status_string(0) == b"ok"
    assert lib.exb_status_string(1) == b"invalid argument"


def test_argument_validation_without_gpu(lib):
    """Bad arguments are rejected before any CUDA call is made."""
    null = None
    one = ctypes.c_void_p(16)   # never dereferenced: validation fails first
    st = lib.exb_leaky_forward(null, one, null, one, 0, null, 0, null, null, 1, 1, 1, 0, 0, null)
    assert st == 1 and b"required" in lib.exb_last_error()
    st = lib.exb_leaky_forward(one, one, null, one, 0, null, 0, null, null, -1, 1, 1, 0, 0, null)
    assert st == 1 and b"negative" in lib.exb_last_error()
    st = lib.exb_leaky_forward(one, one, null, one, 7, null, 0, null, null, 1, 1, 1, 0, 0, null)
    assert st == 1 and b"mode" in lib.exb_last_error()
    st = lib.exb_leaky_forward(one, one, null, one, 0, null, 0, null, null, 1, 1, 1, 9, 0, null)
    assert st == 1 and b"layout" in lib.exb_last_error()
    # empty problems are a successful no-op
    assert lib.exb_leaky_forward(one, one, null, one, 0, null, 0, null, null, 0, 5, 3, 0, 0, null) == 0


def test_missing_library_is_loud(monkeypatch, tmp_path):
    from sinabs_exodus_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.ExodusLibraryError):
        _lib.load()


def test_misaligned_pointers_are_rejected(lib):
    """A float32 tensor cannot start at an address that is not a multiple of 4: EXB_ERR_ALIGN, before any launch."""
    null = None
    ok, odd = ctypes.c_void_p(64), ctypes.c_void_p(66)
    st = lib.exb_leaky_forward(ok, odd, null, ok, 0, null, 0, null, null, 1, 1, 1, 0, 0, null)
    assert st == 2 and b"aligned" in lib.exb_last_error()
    assert lib.exb_status_string(2) == b"misaligned pointer"
    st = lib.exb_leaky_forward(ok, ok, null, ok, 0, null, 0, null, ctypes.c_void_p(68), 1, 1, 1, 0, 0, null)
    assert st == 2      # the float64 sum accumulator needs 8 bytes


def test_static_scratch_size_has_one_source(lib):
    """The size of the built-in scratch array is set in the public header; the library reports the value it was
    built with and the Python constant is that report."""
    from sinabs_exodus_b200 import _lib
    text = open(os.path.join(ROOT, "include", "exodus_b200.h")).read()
    m = re.search(r"#define\s+EXB_STATIC_SCRATCH_BYTES\s+\((\d+)u\s*<<\s*(\d+)\)", text)
    assert m and _lib.STATIC_SCRATCH_BYTES == lib.exb_static_scratch_bytes() == int(m.group(1)) << int(m.group(2)) == 1 << 20
    src = open(os.path.join(ROOT, "sinabs_exodus_b200", "csrc", "exb_tma_kernels.cu")).read()
    assert "g_static_scratch[EXB_STATIC_SCRATCH_BYTES]" in src and "1u << 20" not in src


def test_checkpoint_pair_validates_before_any_cuda_call(lib):
    """exb_lif_forward_ckpt / exb_lif_backward_ckpt and the spikes-only form of exb_lif_forward: bad arguments come
    back as EXB_ERR_ARG / EXB_ERR_UNSUPPORTED without a device being touched."""
    null = None
    p = ctypes.c_void_p(64)        # never dereferenced
    pairs = (null, 0, p, 0, null, 0, p, 0, null, 0)          # in_scale, alpha, subtract, theta, theta_low
    geom = (1, 8, 4, 0, null)                                 # B, T, M, device, stream
    # forward: ckpt is required
    st = lib.exb_lif_forward_ckpt(p, null, p, null, *pairs, 1, 0, null, null, *geom)
    assert st == 1 and b"ckpt" in lib.exb_last_error()
    # backward: the generic surrogate cannot be served, and input + ckpt are required
    st = lib.exb_lif_backward_ckpt(p, null, null, null, p, null, p, p, null, *pairs, 1, 0, 0, 0.0, 0.0, null, *geom)
    assert st == 1 and b"built-in surrogates" in lib.exb_last_error()
    st = lib.exb_lif_backward_ckpt(p, null, null, null, p, null, null, p, null, *pairs, 1, 0, 1, 0.5, 1.0, null, *geom)
    assert st == 1 and b"required" in lib.exb_last_error()
    # reset to a value needs the value
    st = lib.exb_lif_forward_ckpt(p, p, p, null, *pairs, 1, 1, null, null, *geom)
    assert st == 1 and b"reset-to-value" in lib.exb_last_error()
    # spikes-only forward: only in the time-major layout (layout 0 is [N,T])
    st = lib.exb_lif_forward(p, null, p, null, *pairs, 1, 0, null, null, 1, 8, 4, 0, 0, null)
    assert st == 4 and b"v_mem may be omitted" in lib.exb_last_error()
    # empty problems are a successful no-op
    assert lib.exb_lif_forward_ckpt(p, p, p, null, *pairs, 1, 0, null, null, 0, 8, 4, 0, null) == 0
