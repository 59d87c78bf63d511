"""ctypes binding of lib/libb200fp8mm.so (declarations: include/b200_fp8_mm.h, include/b200_mla_consumers.h).

Loading fails loudly: there is no fallback implementation of the operator."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# B200_FP8_MM_LIB selects another build of the same library (e.g. one made with extra nvcc flags).
LIB_PATH = os.environ.get("B200_FP8_MM_LIB") or os.path.join(HERE, "lib", "libb200fp8mm.so")

ABI_VERSION = 7

# Every symbol the two headers declare.
EXPORTS = (
    "b200_fp8_mm",
    "b200_fp8_mm_planned",
    "b200_fp8_mm_strided",
    "b200_fp8_mm_grouped",
    "b200_fp8_mm_static_scratch",
    "b200_fp8_mm_static_scratch_limit",
    "b200_fp8_mm_selftest_wait_expiry",
    "b200_fp8_mm_workspace_bytes",
    "b200_fp8_mm_plan_workspace_bytes",
    "b200_fp8_mm_describe",
    "b200_fp8_mm_estimate_clocks",
    "b200_fp8_mm_strerror",
    "b200_fp8_mm_abi_version",
    # include/b200_mla_consumers.h
    "b200_mla_rope",
    "b200_mla_div_softmax",
)


class CPlan(ctypes.Structure):
    _fields_ = [
        ("block_m", ctypes.c_int),
        ("block_n", ctypes.c_int),
        ("cta_pair", ctypes.c_int),
        ("split_k", ctypes.c_int),
        ("stages", ctypes.c_int),
        ("grid", ctypes.c_int),
        ("tiles", ctypes.c_int),
        ("smem_bytes", ctypes.c_int),
        ("store_bufs", ctypes.c_int),
        ("full_tiles", ctypes.c_int),
    ]


_GEMM_ARGS = (
    [ctypes.c_void_p] * 5
    + [ctypes.c_int] * 3
    + [ctypes.c_longlong] * 7
    + [ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
)

_lib = None


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m amd_developer_challenge_2025_b200.build` "
            "(needs nvcc). There is no CPU fallback for this operator."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(lib, name):
            raise ImportError(f"{LIB_PATH} does not export {name}")
    lib.b200_fp8_mm.argtypes = _GEMM_ARGS
    lib.b200_fp8_mm.restype = ctypes.c_int
    lib.b200_fp8_mm_planned.argtypes = _GEMM_ARGS + [ctypes.POINTER(CPlan)]
    lib.b200_fp8_mm_planned.restype = ctypes.c_int
    # both strides of a and b (two more 64-bit integers) and the optional plan
    lib.b200_fp8_mm_strided.argtypes = (_GEMM_ARGS[:8] + [ctypes.c_longlong] * 9 + _GEMM_ARGS[15:]
                                        + [ctypes.POINTER(CPlan)])
    lib.b200_fp8_mm_strided.restype = ctypes.c_int
    lib.b200_fp8_mm_grouped.argtypes = ([ctypes.c_void_p] * 5 + [ctypes.c_int] * 4 + [ctypes.c_longlong] * 12
                                        + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(CPlan)])
    lib.b200_fp8_mm_grouped.restype = ctypes.c_int
    # the same argument list without the (workspace, workspace_bytes) pair
    lib.b200_fp8_mm_static_scratch.argtypes = _GEMM_ARGS[:16] + _GEMM_ARGS[18:]
    lib.b200_fp8_mm_static_scratch.restype = ctypes.c_int
    # a .. ldc as for b200_fp8_mm, then (wait_limit_ns, skip_kblock, device_status, stream)
    lib.b200_fp8_mm_selftest_wait_expiry.argtypes = (_GEMM_ARGS[:15] + [ctypes.c_ulonglong, ctypes.c_int,
                                                                      ctypes.c_void_p, ctypes.c_void_p])
    lib.b200_fp8_mm_selftest_wait_expiry.restype = ctypes.c_int
    lib.b200_fp8_mm_static_scratch_limit.argtypes = []
    lib.b200_fp8_mm_static_scratch_limit.restype = ctypes.c_size_t
    lib.b200_fp8_mm_workspace_bytes.argtypes = [ctypes.c_int] * 3
    lib.b200_fp8_mm_workspace_bytes.restype = ctypes.c_size_t
    lib.b200_fp8_mm_plan_workspace_bytes.argtypes = [ctypes.c_int] * 3 + [ctypes.POINTER(CPlan)]
    lib.b200_fp8_mm_plan_workspace_bytes.restype = ctypes.c_size_t
    lib.b200_fp8_mm_describe.argtypes = [ctypes.c_int] * 5 + [ctypes.POINTER(CPlan)]
    lib.b200_fp8_mm_describe.restype = ctypes.c_int
    lib.b200_fp8_mm_estimate_clocks.argtypes = [ctypes.c_int] * 4
    lib.b200_fp8_mm_estimate_clocks.restype = ctypes.c_double
    lib.b200_fp8_mm_strerror.argtypes = [ctypes.c_int]
    lib.b200_fp8_mm_strerror.restype = ctypes.c_char_p
    lib.b200_mla_rope.argtypes = ([ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 4 + [ctypes.c_longlong] * 4
                                  + [ctypes.c_void_p])
    lib.b200_mla_rope.restype = ctypes.c_int
    lib.b200_mla_div_softmax.argtypes = [ctypes.c_void_p] + [ctypes.c_int] * 5 + [ctypes.c_void_p]
    lib.b200_mla_div_softmax.restype = ctypes.c_int
    lib.b200_fp8_mm_abi_version.argtypes = []
    lib.b200_fp8_mm_abi_version.restype = ctypes.c_int
    if lib.b200_fp8_mm_abi_version() != ABI_VERSION:
        raise ImportError(f"{LIB_PATH}: ABI version {lib.b200_fp8_mm_abi_version()} != {ABI_VERSION}; rebuild")
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().b200_fp8_mm_strerror(code).decode()
