import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    # The shared library is a build artefact (git-ignored): compile it before collection imports
    # the package, which refuses to import without it.
    sys.path.insert(0, ROOT)
    import importlib.util
    spec = importlib.util.spec_from_file_location("_xb_build", os.path.join(ROOT, "xopes_b200", "build.py"))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    if not os.path.exists(b.LIB):
        b.build()


@pytest.fixture(scope="session")
def lib():
    from xopes_b200 import _lib
    return _lib.load()
