"""ctypes front end of the plain-C oracle (oracle/fp8_mm_oracle.c). Test infrastructure."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build())
        for name in ("fp8mm_oracle_dequant", "fp8mm_oracle_blocks"):
            fn = getattr(_lib, name)
            fn.restype = ctypes.c_int
            fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 4
        _lib.fp8mm_e4m3fn_table.argtypes = [ctypes.c_void_p]
        _lib.fp8mm_e4m3fn_table.restype = None
    return _lib


def e4m3fn_table() -> np.ndarray:
    out = np.zeros(256, dtype=np.float32)
    lib().fp8mm_e4m3fn_table(out.ctypes.data)
    return out


def _run(name, a, b, a_scale, b_scale, n_phase):
    a8 = a.cpu().contiguous().view(torch.uint8).numpy()
    b8 = b.cpu().contiguous().view(torch.uint8).numpy()
    as_ = a_scale.cpu().contiguous().float().numpy()
    bs_ = b_scale.cpu().contiguous().float().numpy()
    m, k = a8.shape
    n = b8.shape[0]
    c = np.zeros((m, n), dtype=np.float32)
    rc = getattr(lib(), name)(a8.ctypes.data, b8.ctypes.data, as_.ctypes.data, bs_.ctypes.data, c.ctypes.data,
                              m, n, k, n_phase)
    if rc != 0:
        raise RuntimeError(f"{name} failed with {rc}")
    return torch.from_numpy(c)


def dequant_matmul_fp32(a, b, a_scale, b_scale, n_phase=0):
    return _run("fp8mm_oracle_dequant", a, b, a_scale, b_scale, n_phase)


def block_order_fp32(a, b, a_scale, b_scale, n_phase=0):
    return _run("fp8mm_oracle_blocks", a, b, a_scale, b_scale, n_phase)
