"""Generates tests/golden/*.npz: small seeded problems with the outputs of the torch CPU
restatement of the reference's dequantise-then-matmul script
(1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py:17-49, 85-89) plus the e4m3fn decode table.

The reference itself cannot be imported or compiled on a CUDA machine (HIP for gfx942 and a
`task` module that is not part of the project), and it holds no golden vectors, so these
fixtures pin the oracle against regressions and against the independent C restatement; they
are not outputs of the reference's own code.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from amd_developer_challenge_2025_b200.inputs import make_inputs  # noqa: E402
from oracle import fp8_mm_oracle as oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, M, N, K, seed, n_phase)
CASES = [
    ("one_block", 32, 128, 128, 11, 0),
    ("ragged_n", 48, 160, 256, 12, 0),       # N not a multiple of 128: 2 scale rows
    ("n576_like", 40, 576, 384, 13, 0),      # 4.5 scale blocks -> 5 rows
    ("shard_phase64", 24, 192, 256, 14, 64), # a column shard that starts mid scale block
    ("odd_m", 129, 64, 512, 15, 0),
]


def main():
    torch.set_num_threads(1)
    for name, m, n, k, seed, phase in CASES:
        if phase:
            # build a wider problem and cut the shard out of it, as the multi-GPU path does
            a, b_full, a_s, bs_full, _ = make_inputs(m, n + phase, k, seed)
            b = b_full[phase:].contiguous()
            b_s = bs_full
        else:
            a, b, a_s, b_s, _ = make_inputs(m, n, k, seed)
        c32 = oracle.dequant_matmul_fp32(a, b, a_s, b_s, phase)
        c16 = c32.to(torch.bfloat16)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            a=a.view(torch.uint8).numpy(), b=b.view(torch.uint8).numpy(),
            a_scale=a_s.numpy(), b_scale=b_s.numpy(),
            c_fp32=c32.numpy(), c_bf16_bits=c16.view(torch.int16).numpy(),
            meta=np.array([m, n, k, seed, phase], dtype=np.int64),
        )
    table = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    np.save(os.path.join(HERE, "e4m3fn_table.npy"), table)


if __name__ == "__main__":
    main()
