import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")
    import torch
    torch.set_num_threads(2)


@pytest.fixture(scope="session", autouse=True)
def _native_planner():
    """Build the C++ planner once per session (seconds; no GPU needed)."""
    from dcp_b200.csrc import build
    build.build_planner()
