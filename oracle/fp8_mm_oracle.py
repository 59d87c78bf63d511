"""CPU oracle for the FP8 block-scaled GEMM (test infrastructure, not product code).

Pinning. The reference ships no golden vectors, tests or fixtures for this path, but the two
dequantise kernels of its dequantise-then-matmul script are plain loops, and oracle/build_ref.py
compiles them UNMODIFIED for the host (oracle/_ref, behind oracle/ref_oracle.py). Against them:

* ``dequant_a`` / ``dequant_b`` are bit-for-bit equal to the reference's ``dqa_kernel`` /
  ``dqb_kernel`` run on the reference's own [k][m] / [k][n] / [k/128][m] / [k/128][ceil(n/128)]
  storage (tests/test_oracle.py), and the committed fixtures under tests/golden/ are those
  kernels' outputs (tests/golden/make_golden.py).
* What stays unpinned: (1) the byte decode. The reference reads its bytes as e4m3fnuz; the
  contract this repository is built to fixes e4m3fn on both sides, so the shim that compiles the
  reference's kernels gives their ``(float)src_val`` an e4m3fn decode (checked against torch's for
  all 256 codes). (2) The order in which the final ``a_fp32.T @ b_fp32`` adds its K products: a
  BLAS property on either side, worth about 1e-6 relative in fp32, far below the bf16 output's
  resolution.

A second, independent pin: a plain-C restatement with its own e4m3fn decoder
(oracle/fp8_mm_oracle.c).

Functions and the reference lines they follow:

* ``dequant_a``            1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py:17-25  (dqa_kernel)
* ``dequant_b``            1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py:34-42  (dqb_kernel)
* ``dequant_matmul``       1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py:65-89  (custom_kernel),
                           followed by the cast to bf16 that the contract adds
* ``block_order_matmul``   1-amd-fp8-mm/amd-fp8-mm-submission.py:302-357 (the K loop of
                           fp8_mm_128x128_ft2: per-block partial from zero, then
                           ``acc += P * a_s * b_s`` left to right)

Format note: the reference decodes its bytes as e4m3fnuz (AMD); the contract this
repository is built to fixes e4m3fn on both sides, so both oracle and kernel decode
e4m3fn.
"""
from __future__ import annotations

import torch

SCALE_BLOCK = 128
RTOL = 2e-2
ATOL = 1e-3


def _expand_b_scale(b_scale: torch.Tensor, n: int, n_phase: int) -> torch.Tensor:
    """Row j of the result is the scale row of column j: b_scale[(j + n_phase) // 128]."""
    rows = (torch.arange(n) + n_phase) // SCALE_BLOCK
    return b_scale.float()[rows]


def dequant_a(a: torch.Tensor, a_scale: torch.Tensor) -> torch.Tensor:
    """fp32 [M,K]: float(a[i,kk]) * a_scale[i, kk // 128]."""
    return a.float() * a_scale.float().repeat_interleave(SCALE_BLOCK, dim=1)


def dequant_b(b: torch.Tensor, b_scale: torch.Tensor, n_phase: int = 0) -> torch.Tensor:
    """fp32 [N,K]: float(b[j,kk]) * b_scale[(j + n_phase) // 128, kk // 128]."""
    n = b.shape[0]
    return b.float() * _expand_b_scale(b_scale, n, n_phase).repeat_interleave(SCALE_BLOCK, dim=1)


def dequant_matmul_fp32(a, b, a_scale, b_scale, n_phase: int = 0) -> torch.Tensor:
    """The reference's fp32 result: dequantise both operands, one fp32 matmul."""
    a, b, a_scale, b_scale = (t.cpu() for t in (a, b, a_scale, b_scale))
    assert a.shape[1] == b.shape[1] and a.shape[1] % SCALE_BLOCK == 0
    return dequant_a(a, a_scale) @ dequant_b(b, b_scale, n_phase).T


def dequant_matmul(a, b, a_scale, b_scale, n_phase: int = 0) -> torch.Tensor:
    """bf16 [M,N] — the oracle every parity test compares against."""
    return dequant_matmul_fp32(a, b, a_scale, b_scale, n_phase).to(torch.bfloat16)


def block_order_matmul(a, b, a_scale, b_scale, n_phase: int = 0) -> torch.Tensor:
    """Second restatement, in the order the GPU kernels compute: one unscaled fp32
    product per 128-wide K block, scaled by a_scale then b_scale, accumulated in fp32."""
    a, b, a_scale, b_scale = (t.cpu() for t in (a, b, a_scale, b_scale))
    m, k = a.shape
    n = b.shape[0]
    bs = _expand_b_scale(b_scale, n, n_phase)  # [N, K/128]
    acc = torch.zeros(m, n, dtype=torch.float32)
    af, bf = a.float(), b.float()
    for kb in range(k // SCALE_BLOCK):
        sl = slice(kb * SCALE_BLOCK, (kb + 1) * SCALE_BLOCK)
        part = af[:, sl] @ bf[:, sl].T
        acc += (part * a_scale.float()[:, kb : kb + 1]) * bs[:, kb][None, :]
    return acc.to(torch.bfloat16)


def check(c: torch.Tensor, ref: torch.Tensor, rtol: float = RTOL, atol: float = ATOL):
    """(ok, worst_excess, max_abs_err): ok iff |c-ref| <= atol + rtol*|ref| everywhere."""
    c32, r32 = c.detach().cpu().float(), ref.detach().cpu().float()
    if c32.shape != r32.shape:
        return False, float("inf"), float("inf")
    if not torch.isfinite(c32).all():
        return False, float("inf"), float("inf")
    err = (c32 - r32).abs()
    excess = (err - (atol + rtol * r32.abs())).max().item() if err.numel() else 0.0
    return excess <= 0.0, excess, (err.max().item() if err.numel() else 0.0)
