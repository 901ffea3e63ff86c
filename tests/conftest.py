"""Shared fixtures.  GPU tests carry @pytest.mark.gpu; everything else runs on CPU."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import fp8_oracle
    fp8_oracle.lib()
    return fp8_oracle


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN
