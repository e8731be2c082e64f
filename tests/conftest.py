import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def built_lib():
    """The in-tree shared library, (re)built if stale. nvcc cross-compiles without a GPU."""
    from pega_omni_b200 import build, lib
    build.build()
    return lib.load()


@pytest.fixture(scope="session")
def oracle_lib():
    from oracle import build
    build.build()
    from oracle import cpu
    return cpu
