"""GPU: the tensor-core building blocks of the chunk kernels, one 128x128x128 product per operand
staging form, against a torch fp32 matmul of the same 16-bit inputs."""
import pytest
import torch

from util import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("variant", [0, 1, 2, 3, 4])
def test_umma_probe(variant, dtype, lib):
    from xopes_b200 import _lib
    g = torch.Generator().manual_seed(variant)
    a = torch.randn(128, 128, generator=g).to(dtype).cuda()
    b = torch.randn(128, 128, generator=g).to(dtype).cuda()
    d = torch.full((128, 128), float("nan"), device="cuda")
    rc = lib.la_debug_umma_probe(variant, a.data_ptr(), b.data_ptr(), d.data_ptr(),
                                 _lib.dtype_code(a), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    af, bf = a.float(), b.float()
    ref = {0: af @ bf.T, 1: af @ bf, 2: af @ bf, 3: af.T @ bf, 4: af @ bf}[variant]
    assert_close(f"variant {variant}", ref, d, 1e-5)


def test_device_status_word_is_clear(lib):
    import ctypes
    st = ctypes.c_int(-1)
    assert lib.la_device_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(st)) == 0
    assert st.value == 0, f"a bounded wait ran out on the device (code {st.value})"


def test_a_wait_that_runs_out_returns_a_status_and_leaves_the_gpu_usable(lib):
    """The give-up path of the kernels' bounded waits: one CTA waits 1 ms on an mbarrier nothing
    arrives on.  The launch must come back by itself, the status word must carry the probe's code,
    clearing it must work, and an ordinary call afterwards must be correct."""
    import ctypes
    import time

    import xopes_b200 as xb
    from oracle import lightning_attn_oracle as orc
    from xopes_b200 import workloads
    stream = torch.cuda.current_stream().cuda_stream
    st = ctypes.c_int(-1)
    assert lib.la_device_status(stream, ctypes.byref(st)) == 0 and st.value == 0
    t0 = time.perf_counter()
    assert lib.la_debug_wait_probe(1000, stream) == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0, "the bounded wait did not give up in time"
    assert lib.la_device_status(stream, ctypes.byref(st)) == 0
    assert st.value == 199, f"expected the probe's code, read {st.value}"
    assert lib.la_device_status_clear(stream) == 0
    assert lib.la_device_status(stream, ctypes.byref(st)) == 0 and st.value == 0
    # the context is intact: a tcgen05 forward right after
    w = workloads.lasd_inputs(1, 256, 2, 128, 128, torch.bfloat16, seed=3, use_do=False)
    o, sf = xb.lasd_fn(w["q"].cuda(), w["k"].cuda(), w["v"].cuda(), w["ld"].cuda(),
                       initial_state=w["initial_state"].cuda())
    ro, rsf = orc.lasd_forward(w["q"].float(), w["k"].float(), w["v"].float(), w["ld"], w["initial_state"])
    assert_close("o", ro, o.float(), 1e-2)
    assert_close("state", rsf, sf, 1e-2)
    assert lib.la_debug_wait_probe(0, stream) == -2
