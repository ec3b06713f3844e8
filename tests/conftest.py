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


@pytest.fixture(autouse=True)
def _device_status_stays_clear(request):
    """After every GPU test the watchdog word must read 0: a bounded wait that ran out inside a
    kernel leaves undefined outputs behind an LA_OK return code, which a parity assert might not
    notice.  Tests that make a wait run out on purpose clear the word themselves."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import ctypes

    import torch
    if not torch.cuda.is_available():
        return
    from xopes_b200 import _lib
    lib = _lib.load()
    word = ctypes.c_int(-1)
    assert lib.la_device_status(None, ctypes.byref(word)) == 0
    if word.value != 0:
        lib.la_device_status_clear(None)
        torch.cuda.synchronize()
        pytest.fail(f"device status word reads {word.value} after the test: a bounded wait gave up")
