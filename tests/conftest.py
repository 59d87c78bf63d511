import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); deselected on CPU-only machines")


@pytest.fixture(scope="session")
def built_library():
    """Path of the C-ABI library; built with nvcc when it is missing or stale."""
    from amd_developer_challenge_2025_b200 import build

    return build.build()
