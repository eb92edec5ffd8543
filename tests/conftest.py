"""Test configuration. GPU tests (`-m gpu`) call the CUDA path through the C
ABI and compare with the oracle; everything else runs on CPU."""
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "jax-mps_b200"))
sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def client():
    import b200
    c = b200.Client()
    yield c
    c.synchronize()
