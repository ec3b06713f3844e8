"""GPU: the chunk-level intermediates of the reference's fixtures
(xopes/ops/lightning_attn/scalar_decay/torch_utils.py) from the CUDA path.  The kernels keep no
per-chunk state or intra/inter split in HBM, but every one of those intermediates is what a public
entry point returns when the 128-token chunks are handed to it as segments:

  local states (forward / reverse)   la_lasd_state_pass over the chunks
  scanned states                     la_lasd_fold_states over those
  intra outputs (forward)            la_lasd_fwd with the chunks as documents and no initial state
  intra outputs (reverse)            dv of la_lasd_bwd on the same documents with roles (k, q, do)
  inter outputs                      full forward minus the intra outputs

Each is compared with oracle/chunk_fixtures.py (pinned to the reference's outputs by
tests/golden/chunkfx_lasd.npz) on bf16 inputs with D = E = 128 and a ragged last chunk."""
import pytest
import torch

from oracle import chunk_fixtures as cfx
from util import TOL_BF16, assert_close

pytestmark = pytest.mark.gpu


def _inputs(n=600, h=2, d=128):
    g = torch.Generator().manual_seed(41)
    cast = lambda t: t.bfloat16().float()  # noqa: E731
    q = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    k = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    v = cast(torch.randn(1, n, h, d, generator=g))
    ld = torch.nn.functional.logsigmoid(torch.randn(1, n, h, generator=g) + 2)
    s0 = 0.1 * torch.randn(1, h, d, d, generator=g)
    return q, k, v, ld, s0


def test_local_and_scanned_states(lib):
    from xopes_b200 import _lib
    q, k, v, ld, s0 = _inputs()
    n, h, d, block = q.shape[1], q.shape[2], q.shape[3], 128
    bounds = list(range(0, n, block)) + [n]
    L = len(bounds) - 1
    dev = "cuda"
    kc, vc, ldc = k.bfloat16().to(dev), v.bfloat16().to(dev), ld.to(dev)
    cu = torch.tensor(bounds, dtype=torch.int64, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    tab = torch.tensor([[0, int(i == 0), int(i == L - 1), i] for i in range(L)], dtype=torch.int32, device=dev)
    first = torch.exp(ld[0, bounds[:-1]]).view(L, h, 1, 1)                 # e^{ld of each chunk's first token}
    for reverse in (0, 1):
        local = torch.empty(L, h, d, d, device=dev)
        gsum = torch.empty(L, h, device=dev)
        assert lib.la_lasd_state_pass(kc.data_ptr(), vc.data_ptr(), ldc.data_ptr(), 0, h, 1, cu.data_ptr(),
                                      local.data_ptr(), gsum.data_ptr(), 1, n, h, d, d, L, _lib.LA_BF16, reverse, 0,
                                      0, stream) == 0
        inc, ends = torch.empty_like(local), torch.empty(1, h, d, d, device=dev)   # one document
        assert lib.la_lasd_fold_states(local.data_ptr(), gsum.data_ptr(), tab.data_ptr(), None, s0.to(dev).data_ptr(),
                                       inc.data_ptr(), ends.data_ptr(), L, h, d, d, reverse, stream) == 0
        rloc, rglob = cfx.lasd_chunk_states(k, v, ld, s0, block, bool(reverse))
        rloc, rglob = rloc[0].transpose(0, 1), rglob[0].transpose(0, 1)     # (L, H, D, E), (L+1, H, D, E)
        if not reverse:
            assert_close("local states", rloc, local, TOL_BF16)
            assert_close("scanned states (entering each chunk)", rglob[:L], inc, TOL_BF16)
            assert_close("final state", rglob[L], ends[0], TOL_BF16)
        else:
            # the kernel's reverse state includes the decay of the chunk's first token, the
            # reference applies it one step later (oracle/chunk_fixtures.py)
            assert_close("local states (reverse)", rloc * first, local, TOL_BF16)
            nxt = torch.cat([first[1:], torch.ones(1, h, 1, 1)])            # nothing follows the last chunk
            assert_close("scanned states (reverse)", rglob[:L] * nxt, inc, TOL_BF16)
            assert_close("state after the whole sequence (reverse)", rglob[L], ends[0], TOL_BF16)


def test_intra_and_inter_outputs():
    import xopes_b200 as xb
    q, k, v, ld, s0 = _inputs()
    n, h, block = q.shape[1], q.shape[2], 128
    dev = "cuda"
    cu = torch.tensor(list(range(0, n, block)) + [n], dtype=torch.int64, device=dev)
    qc, kc, vc = (t.bfloat16().to(dev) for t in (q, k, v))
    o_intra, _ = xb.lasd_fn(qc, kc, vc, ld.to(dev), cu_seqlens=cu)
    assert_close("intra (forward)", cfx.lasd_chunk_intra(q, k, v, ld, block), o_intra.float(), TOL_BF16)
    o_full, _ = xb.lasd_fn(qc, kc, vc, ld.to(dev), initial_state=s0.to(dev))
    inter = o_full.float() - o_intra.float()
    ref_inter = cfx.lasd_chunk_inter(q, k, v, ld, s0, block)
    # a difference of two 16-bit tensors: bounded against the magnitude of the outputs themselves
    err = float((inter.cpu() - ref_inter).norm() / o_full.float().norm().cpu())
    assert err <= TOL_BF16, f"inter: error {err:.3e} relative to the output norm"
    # reverse intra: dv of the chunks-as-documents backward is lasd_intra_torch(reverse) with roles (k, q, do)
    g = torch.Generator().manual_seed(42)
    do = torch.randn(1, n, h, v.shape[-1], generator=g).bfloat16().float()
    ql, kl, vl = (t.clone().requires_grad_() for t in (qc, kc, vc))
    o2, _ = xb.lasd_fn(ql, kl, vl, ld.to(dev), cu_seqlens=cu)
    o2.backward(do.bfloat16().to(dev))
    assert_close("intra (reverse)", cfx.lasd_chunk_intra(k, q, do, ld, block, reverse=True), vl.grad.float(), TOL_BF16)
