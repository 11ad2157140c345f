import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


def _gpu_count() -> int:
    try:
        import torch
        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


@pytest.fixture(scope="session")
def gpu_count():
    return _gpu_count()


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """Every test session starts from a current build of the CUDA library and the C oracle."""
    from aristos_b200 import build as kbuild
    from oracle import c_oracle
    kbuild.build()
    c_oracle.build()
