"""Ahead-of-time build of lib/libb200fp8mm.so with nvcc for sm_100a.

Replaces the reference's import-time JIT (`load_inline` with hipcc for gfx942,
1-amd-fp8-mm/amd-fp8-mm-submission.py:582-592)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
INCLUDE = os.path.join(ROOT, "include")
SRC = os.path.join(HERE, "csrc", "fp8_mm_sm100.cu")
SOURCES = [SRC, os.path.join(HERE, "csrc", "mla_consumers_sm100.cu")]
HEADERS = [os.path.join(INCLUDE, "b200_fp8_mm.h"), os.path.join(INCLUDE, "b200_mla_consumers.h")]
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libb200fp8mm.so")


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    newest = max(os.path.getmtime(p) for p in SOURCES + HEADERS)
    return os.path.getmtime(LIB) < newest


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [
        _nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
        "-I", INCLUDE, "-shared", "-Xcompiler", "-fPIC", "-o", LIB, *SOURCES,
    ]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
