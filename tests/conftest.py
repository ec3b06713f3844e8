import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session", autouse=True)
def _built_library():
    """The shared library is a build artefact (git-ignored): compile it if it is not there."""
    from xopes_b200 import build
    if not os.path.exists(build.LIB):
        build.build()


@pytest.fixture(scope="session")
def lib():
    from xopes_b200 import _lib
    return _lib.load()
