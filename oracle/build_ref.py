"""Test infrastructure: builds oracle/_ref/libflashomni_ref.so, a C-ABI harness (oracle/ref_harness.cu)
around the reference's own CUDA kernels, compiled from the reference headers where they lie.

    python oracle/build_ref.py [--force]

Needs the reference checkout (FLASHOMNI_REFERENCE_DIR, else a directory `reference` beside this repository) and the
CUTLASS / CuTe headers the reference's GEMMs include (taken from the installed flashinfer wheel; the
reference's own 3rdparty/cutlass submodule is empty). Nothing is copied from the reference; the only
output is the shared library under oracle/_ref/, which is git-ignored. Does nothing (exit 0) when the
reference or the headers are absent.
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "libflashomni_ref.so")
SRC = os.path.join(HERE, "ref_harness.cu")


def reference_dir() -> str:
    """The reference checkout: FLASHOMNI_REFERENCE_DIR, else `reference` beside the repository; "" if neither exists."""
    env = os.environ.get("FLASHOMNI_REFERENCE_DIR", "")
    if env:
        return env if os.path.isdir(env) else ""
    sibling = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return sibling if os.path.isdir(sibling) else ""


def _cutlass_root():
    try:
        import flashinfer
        root = os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass")
        if os.path.isdir(os.path.join(root, "include", "cute")):
            return root
    except Exception:
        pass
    return None


def build(force: bool = False) -> str | None:
    ref = reference_dir()
    inc = os.path.join(ref, "include")
    if not os.path.isdir(os.path.join(inc, "flashomni")):
        print("build_ref: reference headers not found, skipping")
        return None
    cut = _cutlass_root()
    if cut is None:
        print("build_ref: CUTLASS headers not found, skipping")
        return None
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    # flags of the reference's own build (setup.py:229-238): -O3 -std=c++17 -use_fast_math
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
           "-use_fast_math", "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared", f"-I{inc}", f"-I{cut}/include",
           f"-I{cut}/tools/util/include", "-o", OUT, SRC]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build_ref: nvcc failed")
    return OUT


if __name__ == "__main__":
    print(build("--force" in sys.argv))
