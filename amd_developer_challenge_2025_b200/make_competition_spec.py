"""Writes competition_spec.txt (beside this file) from the reference project's README.

The reference lists the benchmark cases its kernels were run on as `m: ..; n: ..; k: ..; seed: ..`
lines (README.md:65-82 of the reference project). This script copies exactly those lines out of a
checkout of the reference, so that `runner --competition-shapes` and the tests use the same shapes
and seeds. Usage:  python -m amd_developer_challenge_2025_b200.make_competition_spec [REFERENCE_ROOT]
"""
from __future__ import annotations

import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "competition_spec.txt")
LINE = re.compile(r"^\s*m:\s*\d+\s*;\s*n:\s*\d+\s*;\s*k:\s*\d+\s*;\s*seed:\s*\d+\s*$")


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    root = argv[0] if argv else os.environ.get("FP8MM_REFERENCE_ROOT", "/root/reference")
    with open(os.path.join(root, "README.md"), "r", encoding="utf-8") as f:
        lines = [ln.strip() for ln in f if LINE.match(ln)]
    if not lines:
        raise SystemExit("no spec lines found in the reference README")
    with open(OUT, "w", encoding="utf-8") as f:
        f.write("# benchmark cases listed in the reference project's README (m; n; k; seed)\n")
        f.write("\n".join(lines) + "\n")
    print(f"{len(lines)} cases -> {OUT}")


if __name__ == "__main__":
    main()
