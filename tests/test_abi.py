"""CPU: the C-ABI shared library loads, exports every symbol include/xopes_b200.h declares, and its
host-side logic (argument checks, path choice, workspace sizes) behaves -- no kernel is launched."""
import ctypes
import os
import re

import pytest

from xopes_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "xopes_b200.h")


def declared_symbols():
    src = open(HEADER).read()
    return sorted(set(re.findall(r"LA_API[^;(]*?\b(la_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for name in ("la_lasd_fwd", "la_lasd_bwd", "la_lavd_fwd", "la_lavd_bwd", "la_decode_scalar",
                 "la_decode_vector"):
        assert name in syms


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_binding_covers_every_declared_symbol():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_status_strings(lib):
    assert lib.la_abi_version() >= 1
    assert lib.la_status_string(0) == b"ok"
    for code in range(-7, 0):
        assert lib.la_status_string(code) not in (b"ok", b"unknown status")


def test_path_choice(lib):
    # tensor-core chunk kernels: 16-bit inputs, head dimensions up to 128 in multiples of 8, N >= 128
    assert lib.la_lasd_path(8192, 128, 128, _lib.LA_BF16, 0) == 1
    assert lib.la_lasd_path(8192, 128, 128, _lib.LA_F32, 0) == 0
    assert lib.la_lasd_path(8192, 64, 128, _lib.LA_BF16, 0) == 1
    assert lib.la_lasd_path(8192, 64, 64, _lib.LA_F16, 0) == 1
    assert lib.la_lasd_path(8192, 256, 128, _lib.LA_BF16, 0) == 0
    assert lib.la_lasd_path(8192, 60, 64, _lib.LA_BF16, 0) == 0
    assert lib.la_lasd_path(64, 128, 128, _lib.LA_BF16, 0) == 0
    assert lib.la_lasd_path(8192, 128, 128, _lib.LA_BF16, _lib.FLAG_FORCE_RECURRENCE) == 0
    assert lib.la_lasd_path(8192, 33, 63, _lib.LA_BF16, _lib.FLAG_REQUIRE_TENSOR) == -3
    assert lib.la_lasd_path(8192, 128, 128, 7, 0) == -3


def test_argument_checks_return_codes_without_a_gpu(lib):
    one = ctypes.c_void_p(16)  # never dereferenced: the checks fail first
    args = dict(B=1, N=4, H=2, D=8, E=8)
    # NULL q
    rc = lib.la_lasd_fwd(None, one, one, one, 0, 0, 1, None, None, one, None,
                         args["B"], args["N"], args["H"], args["D"], args["E"], 0, _lib.LA_F32, 0, None)
    assert rc == -1
    # bad shape
    rc = lib.la_lasd_fwd(one, one, one, one, 0, 0, 1, None, None, one, None,
                         1, 0, 2, 8, 8, 0, _lib.LA_F32, 0, None)
    assert rc == -2
    # cu_seqlens with B != 1
    rc = lib.la_lasd_fwd(one, one, one, one, 0, 0, 1, None, one, one, None,
                         2, 4, 2, 8, 8, 3, _lib.LA_F32, 0, None)
    assert rc == -2
    # a document count without cu_seqlens (scratch would be sized for M, kernels would run B)
    rc = lib.la_lasd_fwd(one, one, one, one, 0, 0, 1, None, None, one, None,
                         4, 4, 2, 8, 8, 1, _lib.LA_F32, 0, None)
    assert rc == -2
    rc = lib.la_lasd_bwd_noalloc(one, one, one, one, 0, 0, 1, None, one, None, None, one, one, one, one, None,
                                 4, 4, 32, 128, 128, 1, _lib.LA_BF16, 0, None)
    assert rc == -2
    rc = lib.la_lavd_bwd(one, one, one, one, None, None, one, None, None, one, one, one, one, None, None,
                         None, 0, 4, 4, 2, 8, 8, 1, _lib.LA_F32, 0, None)
    assert rc == -2
    # unknown dtype
    rc = lib.la_lasd_fwd(one, one, one, one, 0, 0, 1, None, None, one, None,
                         1, 4, 2, 8, 8, 0, 9, 0, None)
    assert rc == -3
    # lavd needs at least one decay
    rc = lib.la_lavd_fwd(one, one, one, None, None, None, None, one, None,
                         1, 4, 2, 8, 8, 0, _lib.LA_F32, 0, None)
    assert rc == -1
    # 16-bit decays: only with 16-bit q, k, v, and only for the vector decay
    rc = lib.la_lavd_fwd(one, one, one, one, None, None, None, one, None,
                         1, 4, 2, 8, 8, 0, _lib.LA_F32, _lib.FLAG_LD_16BIT, None)
    assert rc == -3
    rc = lib.la_lasd_fwd(one, one, one, one, 0, 0, 1, None, None, one, None,
                         1, 4, 2, 8, 8, 0, _lib.LA_BF16, _lib.FLAG_LD_16BIT, None)
    assert rc == -3
    # dld requested without workspace
    rc = lib.la_lasd_bwd(one, one, one, one, 0, 0, 1, None, one, None, None, one, one, one, one,
                         None, None, 0, 1, 4, 2, 8, 8, 0, _lib.LA_F32, 0, None)
    assert rc == -7


def test_importing_the_package_maps_no_native_code():
    """The input generators must be importable without loading the CUDA library (the CPU
    reference arm of the benchmark uses them)."""
    import subprocess
    import sys
    code = ("import xopes_b200.workloads, sys; "
            "maps = open('/proc/self/maps').read(); "
            "sys.exit(1 if 'libxopes_b200' in maps else 0)")
    assert subprocess.run([sys.executable, "-c", code], cwd=ROOT).returncode == 0


def test_workspace_sizes(lib):
    assert lib.la_lasd_bwd_workspace_bytes(2, 100, 4, 64, 64, 0, 0) == 0
    w = lib.la_lasd_bwd_workspace_bytes(2, 100, 4, 64, 64, 0, 1)
    assert w >= (2 * 2 * 100 * 4 + 2 * 4 * 64 * 64) * 4
    assert lib.la_lavd_bwd_workspace_bytes(2, 100, 4, 64, 32, 0) == 2 * 4 * 64 * 32 * 4
    assert lib.la_lavd_bwd_workspace_bytes(1, 100, 4, 64, 32, 5) == 5 * 4 * 64 * 32 * 4


def test_front_end_refuses_cpu_tensors_and_bad_decay_type():
    import torch
    import xopes_b200 as xb
    q = torch.randn(1, 4, 2, 8)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        xb.lasd_fn(q, q, q, torch.zeros(1, 4, 2))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        xb.lavd_fn(q, q, q, ldk=torch.zeros(1, 4, 2, 8))
    with pytest.raises(ValueError, match="Invalid decay type"):
        xb.lightning_attn_func(q, q, q, decay_type="nonsense")


def test_install_as_xopes_registers_reference_module_paths():
    import sys
    import xopes_b200 as xb
    saved = {k: v for k, v in sys.modules.items() if k == "xopes" or k.startswith("xopes.")}
    try:
        xb.install_as_xopes()
        from xopes.ops.lightning_attn import lightning_attn_func  # noqa: F401
        from xopes.ops.lightning_attn.scalar_decay import lasd_parallel_triton, lasd_fn  # noqa: F401
        from xopes.ops.lightning_attn.vector_decay import lavd_parallel_triton, lavd_fn  # noqa: F401
    finally:
        for k in [k for k in sys.modules if k == "xopes" or k.startswith("xopes.")]:
            del sys.modules[k]
        sys.modules.update(saved)
