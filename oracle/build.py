"""Build recipe for the checker libraries (test infrastructure, never shipped).

* ``oracle/_build/liboracle.so``       : the C restatement, fused-multiply-add association
* ``oracle/_build/liboracle_nofma.so`` : same source with ``-DORC_NO_FMA``
* ``oracle/_ref/libexodus_ref.so``     : the reference's own CUDA kernels, compiled for
  sm_100a from the reference checkout (only when that checkout is present; its
  sources are included from where they lie and never copied)

Run ``python oracle/build.py`` or call :func:`build_all`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
REF_DIR = os.path.join(HERE, "_ref")
# Checkout of the reference project (read-only): the EXODUS_REFERENCE_ROOT environment variable, else a
# directory named `reference` beside this repository.  Absent -> the reference kernels are simply not built.
REFERENCE_ROOT = os.environ.get("EXODUS_REFERENCE_ROOT",
                                os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    os.makedirs(BUILD_DIR, exist_ok=True)
    src = os.path.join(HERE, "exodus_oracle.c")
    out = os.path.join(BUILD_DIR, "liboracle.so")
    out_nofma = os.path.join(BUILD_DIR, "liboracle_nofma.so")
    base = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math",
            "-fopenmp", src, "-lm"]
    if force or not _newer(out, src):
        subprocess.check_call(base + ["-o", out])
    if force or not _newer(out_nofma, src):
        subprocess.check_call(base + ["-DORC_NO_FMA", "-o", out_nofma])
    return out


def reference_available() -> bool:
    return os.path.isfile(os.path.join(REFERENCE_ROOT, "cuda", "lif_kernels.h"))


def build_reference_kernels(force: bool = False) -> str | None:
    """Compile the reference kernels (from the reference checkout) behind the shim."""
    if not reference_available():
        return None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(REF_DIR, exist_ok=True)
    src = os.path.join(HERE, "ref_kernels.cu")
    out = os.path.join(REF_DIR, "libexodus_ref.so")
    deps = [src, os.path.join(REFERENCE_ROOT, "cuda", "lif_kernels.h"),
            os.path.join(REFERENCE_ROOT, "cuda", "leaky_kernels.h")]
    if force or not _newer(out, *deps):
        # Same code generation defaults as the reference's own build (setup.py
        # passes no nvcc flags): -O3 host default, fmad on, IEEE division.
        subprocess.check_call([
            nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC",
            "-I", os.path.join(REFERENCE_ROOT, "cuda"), src, "-o", out, "-lcudart",
        ])
    return out


def build_all(force: bool = False) -> None:
    build_oracle(force)
    build_reference_kernels(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("oracle libraries built")
