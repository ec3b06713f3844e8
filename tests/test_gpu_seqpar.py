"""GPU: the sequence-parallel forward with the CUDA local forward and the CUDA correction kernel.
Several ranks are emulated one after another on one device (each phase for every rank, with the
published summaries stacked in place of the all-gather), and the stitched result is compared with
the oracle run on the whole stream."""
import pytest
import torch

from oracle import lightning_attn_oracle as orc
from util import TOL_BF16, TOL_FP32, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world,lens,h,d,e,dtype,tol,per_head", [
    (4, [100, 700, 400, 336], 2, 128, 128, torch.bfloat16, TOL_BF16, True),   # tcgen05 path, a document spans a rank
    (4, [100, 700, 400, 336], 2, 128, 128, torch.float16, TOL_BF16, False),
    (3, [10, 60, 26], 2, 16, 24, torch.float32, TOL_FP32, False),             # fp32 generic path
    (2, [64, 64], 2, 128, 128, torch.bfloat16, TOL_BF16, True),               # nothing crosses the cut
])
def test_emulated_ranks_match_whole_stream(world, lens, h, d, e, dtype, tol, per_head):
    from xopes_b200.lightning_attn import seq_parallel as sp
    n = sum(lens)
    g = torch.Generator().manual_seed(11)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    q = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    k = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    v = cast(torch.randn(1, n, h, e, generator=g))
    if per_head:
        ld = torch.log(1 - 2.0 ** (-5 - torch.arange(h, dtype=torch.float32) / 2))
        ld_full = ld.view(1, 1, h).expand(1, n, h)
    else:
        ld_full = torch.nn.functional.logsigmoid(torch.randn(1, n, h, generator=g) + 3)
    cu = [0] + [int(x) for x in torch.tensor(lens).cumsum(0)]
    dev = "cuda"
    ranks = []
    for r in range(world):
        a, b = sp.token_range(n, r, world)
        plan = sp.shard_documents(cu, a, b)
        ql, kl, vl = (t[:, a:b].to(dtype).to(dev).contiguous() for t in (q, k, v))
        ldl = ld.to(dev) if per_head else ld_full[:, a:b].to(dev).contiguous()
        o, states, summary = sp.local_phase(ql, kl, vl, ldl, plan)
        ranks.append((plan, ql, ldl, o, states, summary, a, b))
    gathered = torch.stack([x[5] for x in ranks])
    ro, rs = orc.lasd_forward(q, k, v, ld_full, None, torch.tensor(cu))
    for r, (plan, ql, ldl, o, states, _, a, b) in enumerate(ranks):
        s_in = sp.fold_incoming_state(gathered, r, h, d, e)
        sp.correct_phase(ql, o, states, ldl, s_in, plan)
        assert_close(f"o rank {r}", ro[:, a:b], o.float(), tol)
        for j, doc in enumerate(plan.doc_ids):
            if cu[doc + 1] <= b:
                assert_close(f"state doc {doc}", rs[doc], states[j], tol)


@pytest.mark.parametrize("per_head", [True, False])
@pytest.mark.parametrize("b,n,h", [(1, 8192, 2), (2, 3000, 1)])
def test_segmented_forward_inside_one_gpu(b, n, h, per_head):
    """Few long sequences: lasd_fn cuts them into segments that run concurrently and stitches them
    (xopes_b200/lightning_attn/segmented.py).  Output, final state and the gradients that follow
    must match the oracle on the whole sequences."""
    import xopes_b200 as xb
    from xopes_b200.lightning_attn import segmented as sg
    d = e = 128
    dtype = torch.bfloat16
    assert sg.worth_segmenting([(i * n, (i + 1) * n) for i in range(b)], h, sg.auto_cap(b * n, h, sg.num_sms()), sg.num_sms())
    g = torch.Generator().manual_seed(3)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    q = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    k = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    v = cast(torch.randn(b, n, h, e, generator=g))
    if per_head:
        ld = torch.log(1 - 2.0 ** (-6 - torch.arange(h, dtype=torch.float32)))
        ld_full = ld.view(1, 1, h).expand(b, n, h)
    else:
        ld = ld_full = torch.nn.functional.logsigmoid(torch.randn(b, n, h, generator=g) + 4)
    s0 = 0.1 * torch.randn(b, h, d, e, generator=g)
    do = cast(torch.randn(b, n, h, e, generator=g))
    qc, kc, vc = (t.to(dtype).cuda().requires_grad_() for t in (q, k, v))
    o, sf = xb.lasd_fn(qc, kc, vc, ld.cuda(), initial_state=s0.cuda())
    ro, rsf = orc.lasd_forward(q, k, v, ld_full, s0)
    assert_close("o", ro, o.float(), TOL_BF16)
    assert_close("final_state", rsf, sf, TOL_BF16)
    (o.float() * do.cuda()).sum().backward()
    rq, rk, rv, _, _ = orc.lasd_backward(q, k, v, ld_full, do, s0)
    assert_close("dq", rq, qc.grad.float(), TOL_BF16)
    assert_close("dk", rk, kc.grad.float(), TOL_BF16)
    assert_close("dv", rv, vc.grad.float(), TOL_BF16)
