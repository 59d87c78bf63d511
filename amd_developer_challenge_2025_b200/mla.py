"""Host side of the two custom kernels around the KV down-projection of the reference's MLA-decode
submission, plus that projection itself as an FP8 block-scaled GEMM.

`mla_decode` and `div_softmax` keep the names, argument order and meaning of the reference's pybind module
(3-amd-mla-decode/amd-mla-submission.py:7-11, 110-125, 221-225); the work is done by sm_100a CUDA kernels in
lib/libb200fp8mm.so reached through the C ABI of include/b200_mla_consumers.h. There is no CPU path."""
from __future__ import annotations

import torch

from . import _lib
from .fp8_mm import Fp8MmError, _check, fp8_mm


def mla_decode(x, y, pos: int, xoff: int, yoff: int, d0: int, d1: int, d2: int, xs1: int, xs2: int, ys1: int,
               ys2: int):
    """Rotary position embedding, the reference's `module.mla_decode`: reads the bf16 elements
    x.data_ptr() + xoff + i0*xs1 + i1*xs2 + j and writes the rotated values to y at yoff + i0*ys1 + i1*ys2 + j
    (i0 < d0, i1 < d1, j < d2; row i1 has position pos + i1). y may be x. Runs on the current stream."""
    _check(x.is_cuda and y.is_cuda and x.device == y.device, "x and y must be CUDA tensors on one device")
    _check(x.dtype == torch.bfloat16 and y.dtype == torch.bfloat16, "x and y must be bfloat16")
    _check(d0 > 0 and d1 > 0 and d2 > 0 and d2 % 2 == 0, "d0, d1, d2 must be positive and d2 even")
    # the last element touched must lie inside each tensor's storage
    last_x = xoff + (d0 - 1) * xs1 + (d1 - 1) * xs2 + d2 - 1
    last_y = yoff + (d0 - 1) * ys1 + (d1 - 1) * ys2 + d2 - 1
    _check(0 <= xoff and last_x < x.untyped_storage().nbytes() // 2 - x.storage_offset(), "x: range outside the tensor")
    _check(0 <= yoff and last_y < y.untyped_storage().nbytes() // 2 - y.storage_offset(), "y: range outside the tensor")
    with torch.cuda.device(x.device):
        rc = _lib.load().b200_mla_rope(x.data_ptr() + 2 * xoff, y.data_ptr() + 2 * yoff, pos, d0, d1, d2, xs1, xs2, ys1,
                                       ys2, torch.cuda.current_stream(x.device).cuda_stream)
    if rc != 0:
        raise Fp8MmError(rc, "mla_decode (rope)")
    return y


def div_softmax(qk, bs: int, nh: int, sl: int, dnope: int, drope: int):
    """In-place softmax(qk / sqrt(dnope + drope)) over the last dimension of the contiguous bf16 tensor
    qk [bs, nh, sl], the reference's `module.div_softmax`. Runs on the current stream."""
    _check(qk.is_cuda and qk.dtype == torch.bfloat16 and qk.is_contiguous(), "qk must be a contiguous bfloat16 CUDA tensor")
    _check(qk.numel() == bs * nh * sl and bs > 0 and nh > 0 and sl > 0, "qk must hold bs * nh * sl elements")
    with torch.cuda.device(qk.device):
        rc = _lib.load().b200_mla_div_softmax(qk.data_ptr(), bs, nh, sl, dnope, drope,
                                              torch.cuda.current_stream(qk.device).cuda_stream)
    if rc != 0:
        raise Fp8MmError(rc, "div_softmax")
    return qk


def kv_down_projection_fp8(x, x_scale, w_dkv, w_scale, out=None):
    """The KV down-projection `x @ wDKV.T` (3-amd-mla-decode/amd-mla-submission.py:269; [bs, d] x [dkv + drope, d],
    i.e. N = 576, K = 7168 for the reference's model) as the FP8 block-scaled GEMM of this package: x and w_dkv
    in e4m3fn with fp32 scales per (row, 128 of K) and per (128 rows of w, 128 of K). Returns bf16 [bs, dkv + drope]
    (the row the reference writes into its KV cache)."""
    if out is None:
        out = torch.empty(x.shape[0], w_dkv.shape[0], dtype=torch.bfloat16, device=x.device)
    return fp8_mm(x, w_dkv, x_scale, w_scale, out)
