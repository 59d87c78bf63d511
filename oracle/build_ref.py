"""Compiles the reference's own dequantise kernels for the host CPU: oracle/_ref/libfp8mm_ref.so.

Test infrastructure. The reference's dequantise-then-matmul script
(1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py) carries its device code as a Python string.
Two functions in it, `dqa_kernel` (lines 17-25) and `dqb_kernel` (lines 34-42), are plain strided
loops with no matrix-unit builtin. This recipe

1. reads that file where it lies in the reference checkout (never imports or executes it),
2. cuts the text of those two `__global__` functions out of the string, unmodified,
3. feeds gcc, through standard input, one translation unit made of
   ref_shim.h (stand-ins for the HIP names the two functions use) + the two functions +
   ref_driver.inc (an `extern "C"` host loop that plays the `<<<k, 64>>>` launch),
4. writes only the shared library to oracle/_ref/ (git-ignored; no reference text is stored).

What the shim decides: `__hip_fp8_e4m3_fnuz` converts to float as **e4m3fn** (the encoding this
repository's contract fixes for both operands), `blockIdx`/`threadIdx`/`blockDim` are plain
variables the driver sets. Everything else - the `[k][m]` / `[k][n]` storage, the
`k_idx / 128 * m + m_idx` and `k_idx / 128 * ((n + 127) / 128) + n_idx / 128` scale indexing,
the fp32 multiply - is the reference's own code as compiled.

The reference checkout is looked for in $FP8MM_REFERENCE_ROOT, else in the default location of
`reference_root()`. On a machine without it the recipe does nothing and the prebuilt library (if it travelled) is used."""
from __future__ import annotations

import os
import re
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libfp8mm_ref.so")
SHIM = os.path.join(HERE, "ref_shim.h")
DRIVER = os.path.join(HERE, "ref_driver.inc")
REL_SOURCE = os.path.join("1-amd-fp8-mm", "0-amd-fp8-mm-new-begins.py")
KERNELS = ("dqa_kernel", "dqb_kernel")


def reference_root() -> str:
    return os.environ.get("FP8MM_REFERENCE_ROOT", "/root/reference")


def reference_source() -> str | None:
    path = os.path.join(reference_root(), REL_SOURCE)
    return path if os.path.isfile(path) else None


def extract_kernels(py_text: str) -> str:
    """The text of the two __global__ functions inside the CUDA_SRC string, as written there."""
    m = re.search(r'CUDA_SRC\s*=\s*"""(.*?)"""', py_text, re.S)
    if m is None:
        raise RuntimeError("no CUDA_SRC string in the reference file")
    src = m.group(1)
    out = []
    for name in KERNELS:
        start = src.find("__global__ void " + name + "(")
        if start < 0:
            raise RuntimeError(name + " not found in CUDA_SRC")
        brace = src.index("{", start)
        depth, i = 0, brace
        while True:
            ch = src[i]
            if ch == "{":
                depth += 1
            elif ch == "}":
                depth -= 1
                if depth == 0:
                    break
            i += 1
        out.append(src[start:i + 1])
    return "\n\n".join(out) + "\n"


def available() -> bool:
    return os.path.exists(OUT)


def build(force: bool = False) -> str | None:
    """Returns the library path, or None when neither the reference checkout nor a prebuilt library exists."""
    src = reference_source()
    if src is None:
        return OUT if available() else None
    newest = max(os.path.getmtime(p) for p in (src, SHIM, DRIVER, os.path.abspath(__file__)))
    if not force and available() and os.path.getmtime(OUT) >= newest:
        return OUT
    with open(src, "r", encoding="utf-8") as f:
        kernels = extract_kernels(f.read())
    with open(SHIM, "r", encoding="utf-8") as f:
        shim = f.read()
    with open(DRIVER, "r", encoding="utf-8") as f:
        driver = f.read()
    unit = shim + "\n" + kernels + "\n" + driver
    os.makedirs(OUT_DIR, exist_ok=True)
    subprocess.run(
        ["g++", "-x", "c++", "-std=c++17", "-O2", "-fno-fast-math", "-ffp-contract=off", "-fopenmp", "-shared",
         "-fPIC", "-o", OUT, "-"],
        input=unit.encode(), check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
