"""Drop-in for the reference's submission module: `from submission import custom_kernel`
(README.md:94-95) resolves to this function when this directory is on sys.path, or import it
as `amd_developer_challenge_2025_b200.custom_kernel`."""
from __future__ import annotations

from typing import Tuple

import torch

try:  # imported as a package module
    from .fp8_mm import fp8_mm
except ImportError:  # imported as top-level `submission` by the external harness
    from amd_developer_challenge_2025_b200.fp8_mm import fp8_mm

# The reference takes these aliases from the harness's `task` module
# (1-amd-fp8-mm/amd-fp8-mm-submission.py:6), which is not part of the project.
input_t = Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]
output_t = torch.Tensor


def custom_kernel(data: input_t) -> output_t:
    """Block-scaled FP8 GEMM; same contract as the reference's `custom_kernel`
    (1-amd-fp8-mm/amd-fp8-mm-submission.py:594-604; argument doc at
    1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py:66-77).

    data = (a, b, a_scale, b_scale, c):
        a        float8_e4m3fn [M, K]
        b        float8_e4m3fn [N, K]
        a_scale  float32 [M, K // 128]
        b_scale  float32 [ceil(N / 128), K // 128]
        c        bfloat16 [M, N], pre-allocated by the caller
    Returns the same `c` object, filled. Inputs are never modified (the reference's
    pre-transpose path overwrites a and b in place)."""
    a, b, a_scale, b_scale, c = data
    return fp8_mm(a, b, a_scale, b_scale, c)
