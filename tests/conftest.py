import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built_libraries():
    """The CPU oracle is built on demand (gcc, seconds); libforge_b200.so must already exist or
    be buildable with nvcc - there is no fallback."""
    import oracle_lib
    oracle_lib.oracle()
    from forge_b200 import build as fb_build
    fb_build.build()
