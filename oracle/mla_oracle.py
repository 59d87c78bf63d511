"""CPU oracle for the two custom kernels around the KV down-projection in the reference's MLA-decode
submission (test infrastructure, not product code).

* ``rope_3d``      restates rope_3d_kernel (3-amd-mla-decode/amd-mla-submission.py:17-34; the three
                   specialised variants at 36-108 compute the same values in another thread layout). It is
                   pinned to the reference's own kernels compiled for the host (build_mla_ref.py /
                   ``rope_3d_ref``): bit for bit in tests/test_mla_oracle.py.
* ``div_softmax``  restates div_softmax_kernel (same file, 127-225) including its summation order and its
                   bf16 roundings. Pinning: the kernel cannot be compiled for the host (its reduction relies
                   on 64 threads in lockstep), so this function is checked against torch.softmax within the
                   error its bf16 intermediate allows; **parity unpinned by the reference's code** for this
                   function.

bf16 arithmetic: the reference computes the rotation angle with bf16 adds, multiplies and divides
(`__hadd`, `__hmul`, `__hdiv`), i.e. every operation rounds to bf16 (round to nearest even). torch's
bf16 CPU operators do the same (compute in fp32, round once), so they are used operation by operation."""
from __future__ import annotations

import ctypes
import math

import numpy as np
import torch

from . import build_mla_ref

BF16 = torch.bfloat16


def _b(x) -> torch.Tensor:
    return torch.as_tensor(x).to(BF16)


_libm = None


def _libm_f32(name: str, *cols) -> np.ndarray:
    """Elementwise fp32 libm call (powf, cosf, sinf): the scalar C library routines the reference's kernels
    resolve to when they are compiled for the host, so that the restatement can be compared bit for bit
    (vectorised numpy / torch versions of these functions differ from them in the last bit now and then)."""
    global _libm
    if _libm is None:
        _libm = ctypes.CDLL("libm.so.6")
        for fn, n in (("powf", 2), ("cosf", 1), ("sinf", 1)):
            getattr(_libm, fn).restype = ctypes.c_float
            getattr(_libm, fn).argtypes = [ctypes.c_float] * n
    fn = getattr(_libm, name)
    flat = [np.asarray(c, dtype=np.float32).ravel() for c in cols]
    out = np.fromiter((fn(*(float(c[i]) for c in flat)) for i in range(flat[0].size)), dtype=np.float32,
                      count=flat[0].size)
    return out.reshape(np.asarray(cols[0]).shape)


def rope_angles(d1: int, d2: int, pos: int):
    """(cos, sin) as bf16 [d1, d2/2], computed operation by operation as the reference's kernel does
    (same file, 21-31): idx = bf16(pos) + bf16(d1_idx); theta = bf16(d2_idx) * -2 / d2, all in bf16;
    theta = bf16(powf(bf16(10000), theta)); theta = theta * idx (bf16); cosf/sinf of float(theta), rounded to bf16."""
    idx = (_b(float(pos)) + _b(torch.arange(d1, dtype=torch.float32))).to(BF16)           # [d1]
    th = _b(torch.arange(d2 // 2, dtype=torch.float32))
    th = (th * _b(-2.0)).to(BF16)
    th = (th / _b(float(d2))).to(BF16)
    # the base is written `(__hip_bfloat16)10000.0f` in the reference: 9984 once rounded to bf16
    base = np.full(d2 // 2, float(_b(10000.0)), dtype=np.float32)
    th = torch.from_numpy(_libm_f32("powf", base, th.float().numpy())).to(BF16)            # [d2/2]
    th = (th[None, :] * idx[:, None]).to(BF16)                                             # [d1, d2/2]
    # the angle depends on (idx, d2_idx) only; idx repeats once bf16 can no longer tell positions apart
    thf = th.float().numpy()
    uniq, inv = np.unique(thf, return_inverse=True)
    cos = torch.from_numpy(_libm_f32("cosf", uniq)[inv].reshape(thf.shape)).to(BF16)
    sin = torch.from_numpy(_libm_f32("sinf", uniq)[inv].reshape(thf.shape)).to(BF16)
    return cos, sin


def rope_3d(x: torch.Tensor, pos: int) -> torch.Tensor:
    """x: bf16 [d0, d1, d2] (any strides) -> bf16 [d0, d1, d2], rotated:
    y[..., j] = x1*cos - x2*sin, y[..., j + d2/2] = x2*cos + x1*sin with x1 = x[..., j], x2 = x[..., j + d2/2];
    each product and each sum rounds to bf16 (same file, 32-33)."""
    d0, d1, d2 = x.shape
    cos, sin = rope_angles(d1, d2, pos)
    x = x.to(BF16)
    x1, x2 = x[..., : d2 // 2], x[..., d2 // 2:]
    y1 = ((x1 * cos).to(BF16) - (x2 * sin).to(BF16)).to(BF16)
    y2 = ((x2 * cos).to(BF16) + (x1 * sin).to(BF16)).to(BF16)
    return torch.cat([y1, y2], dim=-1)


def div_softmax(qk: torch.Tensor, dnope: int, drope: int, threads: int = 512) -> torch.Tensor:
    """qk: bf16 [bs, nh, sl] -> bf16, softmax over the last dimension of qk / sqrt(dnope + drope) as the
    reference's kernel computes it: e = expf(float(v) * scale) (no maximum is subtracted), e is rounded to
    bf16 and kept; the row sum adds the UNROUNDED e in fp32, per thread over its strided elements and then
    up the kernel's 512 -> 64 -> 8 -> 1 tree; the result is bf16(float(bf16(e)) / sum)."""
    bs, nh, sl = qk.shape
    scale = np.float32(1.0) / np.float32(math.sqrt(np.float32(dnope + drope)))
    v = qk.to(BF16).float().numpy().astype(np.float32)
    e = np.exp((v * scale).astype(np.float32)).astype(np.float32)                 # [bs, nh, sl]
    # per-thread partial sums: thread t takes elements [8t, 8t+8) + k * 8 * threads of the 8-aligned part in
    # order, then elements sl_aligned + t + k * threads of the rest
    sl_al = sl // 8 * 8
    sums = np.zeros((bs, nh, threads), dtype=np.float32)
    for start in range(0, sl_al, 8 * threads):
        chunk = e[..., start:min(sl_al, start + 8 * threads)]
        nthr = chunk.shape[-1] // 8
        part = chunk.reshape(bs, nh, nthr, 8)
        for j in range(8):
            sums[..., :nthr] = (sums[..., :nthr] + part[..., j]).astype(np.float32)
    for start in range(sl_al, sl, threads):
        chunk = e[..., start:min(sl, start + threads)]
        sums[..., : chunk.shape[-1]] = (sums[..., : chunk.shape[-1]] + chunk).astype(np.float32)

    def tree(vals, half):
        # thread t adds vals[4t..4t+3] then vals[4t+half..4t+half+3], left to right, starting from 0
        n_out = half // 4
        out = np.zeros(vals.shape[:-1] + (n_out,), dtype=np.float32)
        for i in range(4):
            out = (out + vals[..., i:4 * n_out:4]).astype(np.float32)
        for i in range(4):
            out = (out + vals[..., half + i:half + 4 * n_out:4]).astype(np.float32)
        return out

    s64 = tree(sums, 256)       # 64 values
    s8 = tree(s64, 32)          # 8 values
    total = np.zeros((bs, nh), dtype=np.float32)
    for i in range(8):
        total = (total + s8[..., i]).astype(np.float32)
    e16 = torch.from_numpy(e).to(BF16).float().numpy()
    out = (e16 / total[..., None]).astype(np.float32)
    return torch.from_numpy(out).to(BF16)


# ---------------------------------------------------------------------------------------------
# the reference's own RoPE kernels, compiled for the host
# ---------------------------------------------------------------------------------------------

_lib = None


def ref_available() -> bool:
    return build_mla_ref.build() is not None


def rope_3d_ref(x: torch.Tensor, pos: int, which: int = 0) -> torch.Tensor:
    """The reference's kernels (launcher's choice for which=0; 1/2/3 force one) on a contiguous bf16 [d0, d1, d2]."""
    global _lib
    if _lib is None:
        path = build_mla_ref.build()
        if path is None:
            raise RuntimeError("oracle/_ref/libmla_ref.so is not built and the reference checkout is absent")
        _lib = ctypes.CDLL(path)
        _lib.mla_ref_rope.restype = ctypes.c_int
        _lib.mla_ref_rope.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 9
    x = x.to(BF16).contiguous()
    d0, d1, d2 = x.shape
    y = torch.empty_like(x)
    rc = _lib.mla_ref_rope(x.data_ptr(), y.data_ptr(), pos, d0, d1, d2, d1 * d2, d2, d1 * d2, d2, which)
    if rc < 0:
        raise ValueError("that kernel does not take this shape")
    return y
