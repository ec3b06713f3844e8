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
