import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture
def moe_option():
    """set(option, value): a process-wide mode of the CUDA library (moe_set_option) for the length of one test."""
    from tirx_harness_b200 import _lib
    saved = []

    def set_(option, value):
        saved.append((option, _lib.set_option(option, value)))
    yield set_
    for option, old in reversed(saved):
        _lib.set_option(option, old)
