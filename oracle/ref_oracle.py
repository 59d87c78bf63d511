"""The reference's own dequantise kernels, compiled for the host (oracle/_ref), behind ctypes.

Test infrastructure. `dqa_kernel` / `dqb_kernel` are the reference's text compiled unmodified
(see build_ref.py); this module lays the operands out the way the reference's launcher hands
them over (1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py:27-31, 44-48: a as [k][m], b as [k][n],
a_scale as [k/128][m], b_scale as [k/128][ceil(n/128)]) and finishes with the script's
`a_fp32.T @ b_fp32` (same file, 85-89) as a torch CPU fp32 matmul.

The reference has no notion of a column shard (`n_phase`): shards are checked by running the
whole problem here and cutting the columns out of the result."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import build_ref

_lib = None


def available() -> bool:
    """True when the compiled reference kernels can be used on this machine."""
    return build_ref.build() is not None


def lib():
    global _lib
    if _lib is None:
        path = build_ref.build()
        if path is None:
            raise RuntimeError("oracle/_ref is not built and the reference checkout is absent")
        _lib = ctypes.CDLL(path)
        for name in ("fp8mm_ref_dqa", "fp8mm_ref_dqb"):
            fn = getattr(_lib, name)
            fn.restype = None
            fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 2
        _lib.fp8mm_ref_decode_table.restype = None
        _lib.fp8mm_ref_decode_table.argtypes = [ctypes.c_void_p]
    return _lib


def decode_table() -> np.ndarray:
    out = np.zeros(256, dtype=np.float32)
    lib().fp8mm_ref_decode_table(out.ctypes.data)
    return out


def _bytes_km(t: torch.Tensor) -> np.ndarray:
    """[rows, K] fp8 tensor -> uint8 array stored [K][rows], the reference's operand storage."""
    return np.ascontiguousarray(t.cpu().view(torch.uint8).numpy().T)


def dequant_a_km(a: torch.Tensor, a_scale: torch.Tensor) -> torch.Tensor:
    """The reference's `a_fp32`: fp32 [K, M] = dqa_kernel over a [k][m] and a_scale [k/128][m]."""
    m, k = a.shape
    src = _bytes_km(a)
    sc = np.ascontiguousarray(a_scale.cpu().float().numpy().T)
    assert sc.shape == (k // 128, m)
    dst = np.empty((k, m), dtype=np.float32)
    lib().fp8mm_ref_dqa(dst.ctypes.data, src.ctypes.data, sc.ctypes.data, m, k)
    return torch.from_numpy(dst)


def dequant_b_kn(b: torch.Tensor, b_scale: torch.Tensor) -> torch.Tensor:
    """The reference's `b_fp32`: fp32 [K, N] = dqb_kernel over b [k][n] and b_scale [k/128][ceil(n/128)]."""
    n, k = b.shape
    src = _bytes_km(b)
    sc = np.ascontiguousarray(b_scale.cpu().float().numpy().T)
    assert sc.shape == (k // 128, (n + 127) // 128)
    dst = np.empty((k, n), dtype=np.float32)
    lib().fp8mm_ref_dqb(dst.ctypes.data, src.ctypes.data, sc.ctypes.data, n, k)
    return torch.from_numpy(dst)


class Prepared:
    """A problem laid out once the way the reference's launcher receives it, so that a timed call
    holds only the reference's own work (dqa_kernel, dqb_kernel, the fp32 matmul, the cast)."""

    def __init__(self, a, b, a_scale, b_scale):
        self.m, self.k = a.shape
        self.n = b.shape[0]
        self.a_km = _bytes_km(a)
        self.b_kn = _bytes_km(b)
        self.as_km = np.ascontiguousarray(a_scale.cpu().float().numpy().T)
        self.bs_kn = np.ascontiguousarray(b_scale.cpu().float().numpy().T)
        assert self.as_km.shape == (self.k // 128, self.m)
        assert self.bs_kn.shape == (self.k // 128, (self.n + 127) // 128)

    def run_fp32(self) -> torch.Tensor:
        a_fp32 = torch.empty(self.k, self.m, dtype=torch.float32)
        b_fp32 = torch.empty(self.k, self.n, dtype=torch.float32)
        L = lib()
        L.fp8mm_ref_dqa(a_fp32.data_ptr(), self.a_km.ctypes.data, self.as_km.ctypes.data, self.m, self.k)
        L.fp8mm_ref_dqb(b_fp32.data_ptr(), self.b_kn.ctypes.data, self.bs_kn.ctypes.data, self.n, self.k)
        return a_fp32.T @ b_fp32

    def run(self) -> torch.Tensor:
        return self.run_fp32().to(torch.bfloat16)


def dequant_matmul_fp32(a, b, a_scale, b_scale) -> torch.Tensor:
    """fp32 [M, N], the reference script's return value."""
    return Prepared(a, b, a_scale, b_scale).run_fp32()


def dequant_matmul(a, b, a_scale, b_scale) -> torch.Tensor:
    """bf16 [M, N]: the reference's result with the cast the contract adds."""
    return dequant_matmul_fp32(a, b, a_scale, b_scale).to(torch.bfloat16)
