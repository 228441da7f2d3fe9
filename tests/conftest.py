import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def engine():
    """One context on cuda:0 for the whole session; fails loudly when the library or GPU is missing."""
    from gpu_bpe_b200 import BPEEngine
    e = BPEEngine(0).init()
    yield e
    e.destroy()
