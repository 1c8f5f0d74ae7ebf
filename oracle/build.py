"""Builds the checker libraries under oracle/. Test and baseline infrastructure only.

  libmoe_oracle.so   the plain-C restatement (moe_oracle.c), gcc + OpenMP
  _ref/libdrama_ref.so   the reference's own kernels/drama.cu compiled unchanged for sm_100 from the
                     reference checkout when one is present (never copied into this repository);
                     used to cross-check results and as the same-hardware baseline
"""

from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
C_LIB = os.path.join(HERE, "libmoe_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_LIB = os.path.join(REF_DIR, "libdrama_ref.so")


def build_c(force: bool = False) -> str:
    src = os.path.join(HERE, "moe_oracle.c")
    if force or not os.path.exists(C_LIB) or os.path.getmtime(src) > os.path.getmtime(C_LIB):
        cmd = ["gcc", "-O3", "-fopenmp", "-shared", "-fPIC", "-o", C_LIB, src, "-lm"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("gcc failed:\n" + r.stderr)
    return C_LIB


def build_ref(reference_root: str, force: bool = False) -> str | None:
    """Compiles <reference_root>/kernels/drama.cu where it lies; output only into oracle/_ref/."""
    src = os.path.join(reference_root, "kernels", "drama.cu")
    if not os.path.exists(src):
        return REF_LIB if os.path.exists(REF_LIB) else None
    if not force and os.path.exists(REF_LIB) and os.path.getmtime(REF_LIB) > os.path.getmtime(src):
        return REF_LIB
    os.makedirs(REF_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-O3", "-std=c++17", "-arch=sm_100", "-Xcompiler", "-fPIC", "-shared", "-o", REF_LIB, src, "-lcublas"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on the reference kernels:\n" + r.stderr)
    return REF_LIB


if __name__ == "__main__":
    import sys

    print(build_c(force=True))
    if len(sys.argv) > 1:
        print(build_ref(sys.argv[1], force=True))
