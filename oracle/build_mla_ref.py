"""Compiles the reference's RoPE kernels for the host CPU: oracle/_ref/libmla_ref.so.

Test infrastructure, same scheme as build_ref.py. The reference's MLA-decode submission
(3-amd-mla-decode/amd-mla-submission.py) carries its device code as a Python string; its four RoPE
kernels (lines 17-108: rope_3d_kernel, rope_3d_kernel_d0aligned2, rope_3d_kernel_d0aligned16_d2is64,
rope_3d_kernel_d0is128_d2is64) are plain loops over bf16 values with no shared memory and no barrier,
so they compile unmodified with g++ against mla_ref_shim.h (bf16 modelled as round-to-nearest-even).
The recipe reads the file where it lies in the reference checkout, cuts the kernels' text out of the
string, pipes shim + kernels + mla_ref_driver.inc to g++ through standard input and writes only the
shared library. The dispatch between the kernels (same file, 110-125) is restated in the driver.

The scaled-softmax kernel (same file, 127-225) is NOT compiled: its block-wide reduction relies on
64 threads running in lockstep between two barriers, which separate host threads cannot reproduce; it
is restated in mla_oracle.py instead."""
from __future__ import annotations

import os
import re
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libmla_ref.so")
SHIM = os.path.join(HERE, "mla_ref_shim.h")
DRIVER = os.path.join(HERE, "mla_ref_driver.inc")
REL_SOURCE = os.path.join("3-amd-mla-decode", "amd-mla-submission.py")
KERNELS = ("rope_3d_kernel", "rope_3d_kernel_d0aligned2", "rope_3d_kernel_d0is128_d2is64")


def reference_root() -> str:
    return os.environ.get("FP8MM_REFERENCE_ROOT", "/root/reference")


def reference_source() -> str | None:
    path = os.path.join(reference_root(), REL_SOURCE)
    return path if os.path.isfile(path) else None


def extract_kernels(py_text: str) -> str:
    m = re.search(r'CUDA_SRC\s*=\s*"""(.*?)"""', py_text, re.S)
    if m is None:
        raise RuntimeError("no CUDA_SRC string in the reference file")
    src = m.group(1)
    out = []
    for name in KERNELS:
        start = src.find("__global__ void " + name + "(")
        if start < 0:
            raise RuntimeError(name + " not found in CUDA_SRC")
        depth, i = 0, src.index("{", start)
        while True:
            if src[i] == "{":
                depth += 1
            elif src[i] == "}":
                depth -= 1
                if depth == 0:
                    break
            i += 1
        out.append(src[start:i + 1])
    return "\n\n".join(out) + "\n"


def available() -> bool:
    return os.path.exists(OUT)


def build(force: bool = False) -> str | None:
    src = reference_source()
    if src is None:
        return OUT if available() else None
    newest = max(os.path.getmtime(p) for p in (src, SHIM, DRIVER, os.path.abspath(__file__)))
    if not force and available() and os.path.getmtime(OUT) >= newest:
        return OUT
    with open(src, "r", encoding="utf-8") as f:
        kernels = extract_kernels(f.read())
    unit = open(SHIM).read() + "\n" + kernels + "\n" + open(DRIVER).read()
    os.makedirs(OUT_DIR, exist_ok=True)
    subprocess.run(["g++", "-x", "c++", "-std=c++17", "-O2", "-fno-fast-math", "-ffp-contract=off", "-shared", "-fPIC",
                    "-o", OUT, "-"], input=unit.encode(), check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
