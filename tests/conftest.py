import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def gateup_lib():
    """Builds (if stale) and loads libgateup.so; CPU-only checks use it without computing."""
    from sol_execbench_b200_kernels_b200 import build

    build.build()
    from sol_execbench_b200_kernels_b200 import _cabi

    return _cabi
