"""Generates tests/golden/*.npz from the REFERENCE'S OWN dequantise kernels compiled for the host.

Each fixture is a small seeded problem plus what the reference's code made of it:
`dqa_kernel` / `dqb_kernel` (1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py:17-25, 34-42), compiled
unmodified by oracle/build_ref.py, give the dequantised operands (stored as SHA-256 digests of
their fp32 bytes, in the reference's [k][m] / [k][n] storage), and the script's
`a_fp32.T @ b_fp32` (same file, 85-89) as a torch CPU matmul gives `c_fp32`. A column shard
(`n_phase` > 0) is cut out of the whole problem's result, since the reference has no shards.

Needs the reference checkout (see oracle/build_ref.py); the fixtures it writes travel without it.
Run from the repository root:  python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from amd_developer_challenge_2025_b200.inputs import make_inputs  # noqa: E402
from oracle import ref_oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, M, N, K, seed, n_phase)
CASES = [
    ("one_block", 32, 128, 128, 11, 0),
    ("ragged_n", 48, 160, 256, 12, 0),       # N not a multiple of 128: 2 scale rows
    ("n576_like", 40, 576, 384, 13, 0),      # 4.5 scale blocks -> 5 rows
    ("shard_phase64", 24, 192, 256, 14, 64), # a column shard that starts mid scale block
    ("odd_m", 129, 64, 512, 15, 0),
]


def digest(t: torch.Tensor) -> np.ndarray:
    return np.frombuffer(hashlib.sha256(t.contiguous().numpy().tobytes()).digest(), dtype=np.uint8).copy()


def main():
    torch.set_num_threads(1)
    if ref_oracle.build_ref.reference_source() is None:
        raise SystemExit("the reference checkout is needed to regenerate the fixtures")
    for name, m, n, k, seed, phase in CASES:
        # a shard is generated as the wider problem it is cut from, as the multi-GPU path does
        a, b_full, a_s, bs_full, _ = make_inputs(m, n + phase, k, seed)
        a_km = ref_oracle.dequant_a_km(a, a_s)              # [K, M]
        b_kn = ref_oracle.dequant_b_kn(b_full, bs_full)     # [K, N + phase]
        c32 = (a_km.T @ b_kn)[:, phase:].contiguous()
        b = b_full[phase:].contiguous()
        c16 = c32.to(torch.bfloat16)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            a=a.view(torch.uint8).numpy(), b=b.view(torch.uint8).numpy(),
            a_scale=a_s.numpy(), b_scale=bs_full.numpy(),
            c_fp32=c32.numpy(), c_bf16_bits=c16.view(torch.int16).numpy(),
            dq_a_km_sha256=digest(a_km), dq_b_kn_sha256=digest(b_kn[:, phase:]),
            meta=np.array([m, n, k, seed, phase], dtype=np.int64),
        )
    # the decode table comes from torch's e4m3fn decoder (a third party to both the oracle and the shim)
    table = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    np.save(os.path.join(HERE, "e4m3fn_table.npy"), table)


if __name__ == "__main__":
    main()
