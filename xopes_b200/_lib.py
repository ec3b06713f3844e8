"""ctypes binding of libxopes_b200.so (the C ABI declared in include/xopes_b200.h).

There is no fallback: if the shared library is missing the import of any operator raises, and
every operator refuses non-CUDA tensors.  Build the library with `python -m xopes_b200.build`.
"""
import ctypes
import os

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libxopes_b200.so")

LA_F32, LA_BF16, LA_F16 = 0, 1, 2
FLAG_FORCE_RECURRENCE = 1
FLAG_REQUIRE_TENSOR = 2
FLAG_LD_LOGSIGMOID = 4
FLAG_LD_16BIT = 8

_DTYPES = {torch.float32: LA_F32, torch.bfloat16: LA_BF16, torch.float16: LA_F16}

_vp, _i64, _i32, _u32, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_uint, ctypes.c_float

# name -> (restype, argtypes); mirrors include/xopes_b200.h one to one
SIGNATURES = {
    "la_abi_version": (_i32, []),
    "la_status_string": (ctypes.c_char_p, [_i32]),
    "la_lasd_path": (_i32, [_i64, _i64, _i64, _i32, _u32]),
    "la_device_status": (_i32, [_vp, ctypes.POINTER(_i32)]),
    "la_device_status_clear": (_i32, [_vp]),
    "la_debug_lavd_unsafe": (_i32, [_vp, ctypes.POINTER(_i32)]),
    "la_debug_wait_probe": (_i32, [_i64, _vp]),
    "la_debug_last_cuda_error": (ctypes.c_char_p, []),
    "la_debug_umma_probe": (_i32, [_i32, _vp, _vp, _vp, _i32, _vp]),
    "la_lasd_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp,
                           _i64, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _vp]),
    "la_lasd_bwd_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64, _i64, _i64, _i32]),
    "la_lasd_bwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                           _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _u32,
                           _vp]),
    "la_lasd_bwd_noalloc": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp,
                                   _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _vp]),
    "la_lavd_path": (_i32, [_i64, _i64, _i64, _i32, _i32, _i32, _u32]),
    "la_lavd_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                           _i64, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _vp]),
    "la_lavd_bwd_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64, _i64, _i64]),
    "la_lavd_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                           _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _u32, _vp]),
    "la_lasd_state_pass": (_i32, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp,
                                  _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _u32, _vp]),
    "la_lasd_fold_states": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "la_lavd_state_pass": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32,
                                  _i32, _u32, _vp]),
    "la_lavd_fold_states": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "la_seqpar_fold": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "la_seqpar_fold_segments": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "la_seqpar_correct_multi": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "la_seqpar_correct": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "la_normalize_gate_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _f32, _f32,
                                     _i32, _vp]),
    "la_normalize_gate_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32,
                                     _i32, _f32, _f32, _i32, _vp]),
    "la_decode_scalar": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp,
                                _i64, _i64, _i64, _i64, _i32, _vp]),
    "la_decode_vector": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp,
                                _i64, _i64, _i64, _i64, _i32, _vp]),
}

_lib = None


def load():
    """Load the shared library (once) and declare every entry point's signature."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. "
            "Run `python -m xopes_b200.build` (needs nvcc). There is no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float32, bfloat16 or float16")


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("xopes_b200 operators run on CUDA tensors only (no CPU fallback)")


def check(rc: int, what: str):
    if rc != 0:
        lib = load()
        msg = lib.la_status_string(rc).decode()
        if rc == -4:
            msg += " [" + lib.la_debug_last_cuda_error().decode() + "]"
        raise RuntimeError(f"{what} failed: {msg} (status {rc})")
