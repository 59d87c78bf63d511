"""Seeded synthetic inputs for the FP8 block-scaled GEMM.

The competition's own generator lives in an external harness that is not part of the
reference project (the reference only lists `m;n;k;seed` lines, README.md:65-82), so
this generator follows the stated distributions instead: a, b ~ N(0,1) in bf16 cast
to e4m3fn; a_scale [M, K/128] and b_scale [ceil(N/128), K/128] ~ U(0.01, 1) in fp32;
c an empty bf16 [M, N] (tensor shapes as documented at
1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py:66-77)."""
from __future__ import annotations

import torch

SCALE_BLOCK = 128


def mn_major(t: torch.Tensor) -> torch.Tensor:
    """The same [rows, K] matrix stored with `rows` contiguous (stride (1, rows)): the storage the
    reference's kernels index as `a[k*m + i]` (1-amd-fp8-mm/amd-fp8-mm-submission.py:283-300)."""
    return t.t().contiguous().t()


def make_inputs(m: int, n: int, k: int, seed: int, device: str | torch.device = "cpu", layout: str = "k"):
    """Returns (a, b, a_scale, b_scale, c). Always generated on the CPU from `seed`, so the
    CPU oracle and the GPU see identical bits, then moved to `device`. `layout`: "k" (a and b with
    K contiguous) or "mn" (both stored MN-major); the values are the same either way."""
    if k % SCALE_BLOCK != 0:
        raise ValueError("K must be a multiple of 128")
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    a = torch.randn(m, k, dtype=torch.bfloat16, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn(n, k, dtype=torch.bfloat16, generator=g).to(torch.float8_e4m3fn)
    kb = k // SCALE_BLOCK
    nb = (n + SCALE_BLOCK - 1) // SCALE_BLOCK
    a_scale = 0.01 + 0.99 * torch.rand(m, kb, dtype=torch.float32, generator=g)
    b_scale = 0.01 + 0.99 * torch.rand(nb, kb, dtype=torch.float32, generator=g)
    c = torch.empty(m, n, dtype=torch.bfloat16)
    dev = torch.device(device)
    if dev.type != "cpu":
        a, b, a_scale, b_scale, c = (t.to(dev) for t in (a, b, a_scale, b_scale, c))
    if layout == "mn":
        a, b = mn_major(a), mn_major(b)
    elif layout != "k":
        raise ValueError("layout must be 'k' or 'mn'")
    return a, b, a_scale, b_scale, c
