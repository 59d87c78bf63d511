"""Builds the plain-C oracle into oracle/_build/libfp8mm_oracle.so with gcc.

(The reference's own dequantise kernels are compiled by build_ref.py into oracle/_ref/. Its
GEMM kernels are HIP C++ for gfx942 built on MFMA builtins and cannot be compiled here.)"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "fp8_mm_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libfp8mm_oracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    subprocess.check_call(["gcc", "-O2", "-fno-fast-math", "-shared", "-fPIC", "-o", OUT, SRC, "-lm"])
    return OUT


if __name__ == "__main__":
    print(build(force=True))
