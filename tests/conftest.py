import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import cpu_oracle
    cpu_oracle.load()
    return cpu_oracle


@pytest.fixture(scope="session")
def l2j():
    """The product library through its C ABI; built on demand, never replaced by a fallback."""
    from llama2j_b200 import lib
    lib.load(build_if_missing=True)
    return lib
