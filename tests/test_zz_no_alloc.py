"""GPU: la_lasd_bwd_noalloc, the backward entry point for callers that must not allocate.

Some hosts of the library cannot give it scratch memory when they call it -- their device memory
was divided up once at start-up, or the hook they call from is barred from using the allocator.
For them the library keeps a fixed 8 MiB scratch array of its own.  This test drives the entry
point through the C ABI and checks that it returns what la_lasd_bwd returns with caller-provided
scratch: twice in a row with different inputs (the array is shared and keeps the first call's
contents), once on the fp32 scan kernels and once on the tcgen05 chunk kernels, and that a problem
too large for the array is refused without launching anything.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes

import pytest
import torch

from util import assert_close

pytestmark = pytest.mark.gpu


def _inputs(seed, b, n, h, d, e, dtype):
    g = torch.Generator().manual_seed(seed)
    dev = "cuda"
    t = dict(
        q=(torch.randn(b, n, h, d, generator=g) * d ** -0.5).to(dtype).to(dev),
        k=(torch.randn(b, n, h, d, generator=g) * d ** -0.5).to(dtype).to(dev),
        v=torch.randn(b, n, h, e, generator=g).to(dtype).to(dev),
        ld=torch.nn.functional.logsigmoid(torch.randn(b, n, h, generator=g) + 2).to(dev),
        s0=(0.1 * torch.randn(b, h, d, e, generator=g)).to(dev),
        do=torch.randn(b, n, h, e, generator=g).to(dtype).to(dev),
        dsf=torch.randn(b, h, d, e, generator=g).to(dev),
    )
    return t


def _outputs(t):
    b, n, h, d = t["q"].shape
    e = t["v"].shape[-1]
    dev = t["q"].device
    return dict(dq=torch.empty_like(t["q"]), dk=torch.empty_like(t["k"]), dv=torch.empty_like(t["v"]),
                dld=torch.empty(b, n, h, device=dev), ds0=torch.empty(b, h, d, e, device=dev))


def _call(lib, t, out, noalloc):
    from xopes_b200 import _lib
    b, n, h, d = t["q"].shape
    e = t["v"].shape[-1]
    stream = torch.cuda.current_stream().cuda_stream
    head = [t["q"].data_ptr(), t["k"].data_ptr(), t["v"].data_ptr(), t["ld"].data_ptr(), *t["ld"].stride(),
            t["s0"].data_ptr(), t["do"].data_ptr(), t["dsf"].data_ptr(), None,
            out["dq"].data_ptr(), out["dk"].data_ptr(), out["dv"].data_ptr(), out["dld"].data_ptr(),
            out["ds0"].data_ptr()]
    tail = [b, n, h, d, e, 0, _lib.dtype_code(t["q"]), 0, stream]
    if noalloc:
        return lib.la_lasd_bwd_noalloc(*head, *tail)
    nbytes = lib.la_lasd_bwd_workspace_bytes(b, n, h, d, e, 0, 1)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    rc = lib.la_lasd_bwd(*head, ws.data_ptr(), nbytes, *tail)
    torch.cuda.synchronize()  # keep ws alive until the kernels have run
    return rc


@pytest.mark.parametrize("shape,dtype", [((2, 150, 3, 32, 48), torch.float32),       # scan kernels
                                         ((1, 300, 2, 128, 128), torch.bfloat16),    # tcgen05 kernels
                                         ((1, 129, 3, 128, 128), torch.bfloat16)])   # odd B*N*H
def test_noalloc_matches_caller_scratch_twice_in_a_row(lib, shape, dtype):
    for seed in (1, 2):  # second call reuses the array with the first call's leftovers in it
        t = _inputs(seed, *shape, dtype)
        ref, got = _outputs(t), _outputs(t)
        assert _call(lib, t, ref, noalloc=False) == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        assert _call(lib, t, got, noalloc=True) == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "the no-allocation entry point took device memory"
        for name in ref:
            assert_close(f"{name} (call {seed})", ref[name].float(), got[name].float(), 1e-6)


def test_noalloc_refuses_sizes_beyond_its_array(lib):
    from xopes_b200 import _lib
    one = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    b, n, h, d, e = 8, 8192, 32, 128, 128
    assert lib.la_lasd_bwd_workspace_bytes(b, n, h, d, e, 0, 1) > (8 << 20)
    rc = lib.la_lasd_bwd_noalloc(one, one, one, one, 0, 0, 1, None, one, None, None, one, one, one, one, None,
                                 b, n, h, d, e, 0, _lib.LA_BF16, 0, None)
    assert rc == -5
    assert lib.la_status_string(rc) == b"size exceeds a fixed maximum"
