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
