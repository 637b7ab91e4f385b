import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def built_lib():
    """Path of the C-ABI library, built on demand when nvcc is available."""
    from uniql_b200 import _build
    if not os.path.exists(_build.LIB_PATH):
        _build.build()
    if not os.path.exists(_build.EXT_PATH):
        _build.build_torch_ext()
    return _build.LIB_PATH
