"""xopes_b200: B200-native (sm_100a) lightning attention -- a drop-in for xopes/ops/lightning_attn.

The compute lives in libxopes_b200.so (hand-written CUDA behind a C ABI, include/xopes_b200.h);
this package is the host-side mirror of the reference's Python operator interface.  The shared
library is loaded by the first operator call (or by xopes_b200.load_library()), which fails loudly
if it has not been built: there is no CPU or PyTorch fallback.  Importing the package alone maps no
native code, so tools that only need the input generators (xopes_b200.workloads) stay pure Python.
"""
from . import _lib
from ._lib import load as load_library  # noqa: F401

from .lightning_attn import *  # noqa: E402,F401,F403
from .lightning_attn import __all__ as _la_all  # noqa: E402


def install_as_xopes():
    """Register this package's operators under the reference's module paths
    (xopes.ops.lightning_attn[.scalar_decay|.vector_decay|.constant_decay]) in sys.modules, so
    code written against the reference imports them unchanged.  Refuses to shadow a real xopes."""
    import sys
    import types

    from . import lightning_attn as la
    if "xopes" in sys.modules and not getattr(sys.modules["xopes"], "__xopes_b200_shim__", False):
        raise RuntimeError("a real `xopes` package is already imported")
    root = types.ModuleType("xopes")
    root.__xopes_b200_shim__ = True
    ops = types.ModuleType("xopes.ops")
    root.ops = ops
    ops.lightning_attn = la
    ops.lightning_attn_func = la.lightning_attn_func
    sys.modules.update({
        "xopes": root, "xopes.ops": ops, "xopes.ops.lightning_attn": la,
        "xopes.ops.lightning_attn.scalar_decay": la.scalar_decay,
        "xopes.ops.lightning_attn.vector_decay": la.vector_decay,
        "xopes.ops.lightning_attn.constant_decay": la.constant_decay,
    })


__all__ = list(_la_all) + ["install_as_xopes", "load_library"]
