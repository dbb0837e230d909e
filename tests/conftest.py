import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built():
    """The native pieces are built in-tree before any test uses them."""
    from alsparse_b200 import build
    build.build_library()
    build.build_synth()
    build.build_oracle()
