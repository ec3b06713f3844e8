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


@pytest.mark.parametrize("world,lens,h,per_head", [
    (4, [100, 700, 400, 336], 2, True),
    (4, [100, 700, 400, 336], 2, False),
    (4, [300, 3000, 796], 2, True),          # one document covers two whole ranks
    (2, [5000, 11000, 384], 2, False),       # long documents: the ranks cut them into segments
    (2, [64, 64, 128], 2, True),             # nothing crosses the cut
])
def test_emulated_ranks_exchange_before_the_chunk_pass(world, lens, h, per_head):
    """forward_exchange_first (what lasd_seqpar_forward runs on CUDA with the all-gather exchange):
    state-only pass -> exchange -> one chunk pass from true states, no correction.  Ranks are
    emulated in order, the gather handing each rank the summaries of the ranks before it."""
    from xopes_b200.lightning_attn import seq_parallel as sp
    d = e = 128
    n = sum(lens)
    g = torch.Generator().manual_seed(13)
    cast = lambda t: t.bfloat16().float()  # noqa: E731
    q = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    k = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    v = cast(torch.randn(1, n, h, e, generator=g))
    if per_head:
        ld = torch.log(1 - 2.0 ** (-5 - torch.arange(h, dtype=torch.float32) / 2))
        ld_full = ld.view(1, 1, h).expand(1, n, h)
    else:
        ld_full = torch.nn.functional.logsigmoid(torch.randn(1, n, h, generator=g) + 4)
    cu = [0] + [int(x) for x in torch.tensor(lens).cumsum(0)]
    dev = "cuda"
    ro, rs = orc.lasd_forward(q, k, v, ld_full, None, torch.tensor(cu))
    published = []
    for r in range(world):
        a, b = sp.token_range(n, r, world)
        plan = sp.shard_documents(cu, a, b)
        ql, kl, vl = (t[:, a:b].bfloat16().to(dev).contiguous() for t in (q, k, v))
        ldl = ld.to(dev) if per_head else ld_full[:, a:b].to(dev).contiguous()

        def gather(summary):
            published.append(summary)
            rows = published + [torch.zeros_like(summary)] * (world - len(published))
            return torch.stack(rows)

        o, states, plan = sp.forward_exchange_first(ql, kl, vl, ldl, plan, r, gather)
        assert (plan.s_in is not None) == plan.open_start
        assert_close(f"o rank {r}", ro[:, a:b], o.float(), TOL_BF16)
        for j, doc in enumerate(plan.doc_ids):
            if cu[doc + 1] <= b:
                assert_close(f"state doc {doc}", rs[doc], states[j], TOL_BF16)


@pytest.mark.parametrize("world,lens,per_head", [(4, [100, 700, 400, 336], True), (3, [900, 1400, 772], False),
                                                  (2, [2048, 2048], True)])
def test_emulated_ranks_backward_matches_whole_stream(world, lens, per_head):
    """Sequence-parallel backward with the CUDA local backward and the CUDA correction kernel, ranks
    emulated one after another on one device: dq, dk, dv of every rank against the oracle's gradients
    of the whole stream."""
    from xopes_b200.lightning_attn import seq_parallel as sp
    n, h, d, e, dtype = sum(lens), 2, 128, 128, torch.bfloat16
    g = torch.Generator().manual_seed(12)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    q = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    k = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    v = cast(torch.randn(1, n, h, e, generator=g))
    do = cast(torch.randn(1, n, h, e, generator=g))
    if per_head:
        ld = torch.log(1 - 2.0 ** (-5 - torch.arange(h, dtype=torch.float32) / 2))
        ld_full = ld.view(1, 1, h).expand(1, n, h)
    else:
        ld_full = torch.nn.functional.logsigmoid(torch.randn(1, n, h, generator=g) + 3)
    cu = [0] + [int(x) for x in torch.tensor(lens).cumsum(0)]
    dev = "cuda"
    fwd = []
    for r in range(world):
        a, b = sp.token_range(n, r, world)
        plan = sp.shard_documents(cu, a, b)
        loc = [t[:, a:b].to(dtype).to(dev).contiguous() for t in (q, k, v, do)]
        ldl = ld.to(dev) if per_head else ld_full[:, a:b].to(dev).contiguous()
        o, states, summary = sp.local_phase(loc[0], loc[1], loc[2], ldl, plan)
        fwd.append((plan, loc, ldl, summary, a, b))
    gathered = torch.stack([x[3] for x in fwd])
    bwd = []
    for r, (plan, loc, ldl, _, a, b) in enumerate(fwd):
        s_in = sp.fold_incoming_state(gathered, r, h, d, e) if plan.open_start else None
        dq, dk, dv, ds0, summ = sp.local_backward_phase(loc[0], loc[1], loc[2], ldl, loc[3], plan, s_in)
        bwd.append((dq, dk, dv, summ))
    gathered_b = torch.stack([x[3] for x in bwd])
    rq, rk, rv, _, _ = orc.lasd_backward(q, k, v, ld_full, do, None, None, torch.tensor(cu))
    for r, (plan, loc, ldl, _, a, b) in enumerate(fwd):
        dq, dk, dv, _ = bwd[r]
        ds_out = sp.fold_outgoing_gradient(gathered_b, r, h, d, e)
        sp.correct_backward_phase(loc[1], loc[2], dk, dv, ldl, ds_out, plan)
        assert_close(f"dq rank {r}", rq[:, a:b], dq.float(), TOL_BF16)
        assert_close(f"dk rank {r}", rk[:, a:b], dk.float(), TOL_BF16)
        assert_close(f"dv rank {r}", rv[:, a:b], dv.float(), TOL_BF16)


@pytest.mark.parametrize("per_head", [True, False])
@pytest.mark.parametrize("b,n,h", [(1, 8192, 2), (2, 3000, 1), (1, 4000, 3)])
def test_segmented_passes_inside_one_gpu(b, n, h, per_head):
    """Few long sequences: lasd_fn cuts them into segments that all run at once, each from its true
    incoming state (xopes_b200/lightning_attn/segmented.py: state-only pass, fold, varlen chunk
    pass), forward and backward.  Outputs, final state and every gradient -- including the
    log-decay gradient and the gradient of the initial state, with a final-state gradient coming
    in -- must match the oracle on the whole sequences."""
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
    dsf = 0.1 * torch.randn(b, h, d, e, generator=g)
    qc, kc, vc = (t.to(dtype).cuda().requires_grad_() for t in (q, k, v))
    ldc, s0c = ld.cuda().requires_grad_(), s0.cuda().requires_grad_()
    o, sf = xb.lasd_fn(qc, kc, vc, ldc, initial_state=s0c)
    ro, rsf = orc.lasd_forward(q, k, v, ld_full, s0)
    assert_close("o", ro, o.float(), TOL_BF16)
    assert_close("final_state", rsf, sf, TOL_BF16)
    ((o.float() * do.cuda()).sum() + (sf * dsf.cuda()).sum()).backward()
    rq, rk, rv, rld, rs0 = orc.lasd_backward(q, k, v, ld_full, do, s0, dsf)
    assert_close("dq", rq, qc.grad.float(), TOL_BF16)
    assert_close("dk", rk, kc.grad.float(), TOL_BF16)
    assert_close("dv", rv, vc.grad.float(), TOL_BF16)
    assert_close("dld", rld.sum((0, 1)) if per_head else rld, ldc.grad, TOL_BF16)
    assert_close("dinitial_state", rs0, s0c.grad, TOL_BF16)


def test_state_pass_and_fold_match_the_oracle(lib):
    """la_lasd_state_pass / la_lasd_fold_states through the C ABI: the state a segment's own tokens
    build (forward and reverse flow) and the states entering every segment of two documents, against
    the oracle's final states / initial-state gradients of the same token ranges."""
    from xopes_b200 import _lib
    n, h, d = 1000, 2, 128
    g = torch.Generator().manual_seed(8)
    cast = lambda t: t.bfloat16().float()  # noqa: E731
    q = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    k = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    v = cast(torch.randn(1, n, h, d, generator=g))
    do = cast(torch.randn(1, n, h, d, generator=g))
    ld = torch.nn.functional.logsigmoid(torch.randn(1, n, h, generator=g) + 3)
    segs = [(0, 256), (256, 300), (300, 684), (684, 1000)]          # documents: [0,300) and [300,1000)
    dev = "cuda"
    qc, kc, vc, doc_, ldc = (t.to(dev) for t in (q.bfloat16(), k.bfloat16(), v.bfloat16(), do.bfloat16(), ld))
    ranges = torch.tensor(segs, dtype=torch.int64, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for reverse, (y, z) in ((0, (kc, vc)), (1, (qc, doc_))):
        states = torch.empty(len(segs), h, d, d, device=dev)
        gsum = torch.empty(len(segs), h, device=dev)
        rc = lib.la_lasd_state_pass(y.data_ptr(), z.data_ptr(), ldc.data_ptr(), 0, h, 1, ranges.data_ptr(),
                                    states.data_ptr(), gsum.data_ptr(), 1, n, h, d, d, len(segs), _lib.LA_BF16,
                                    reverse, 1, 0, stream)
        assert rc == 0
        for j, (a, b) in enumerate(segs):
            sl = slice(a, b)
            if reverse == 0:
                _, ref = orc.lasd_forward(q[:, sl], k[:, sl], v[:, sl], ld[:, sl])
            else:  # gradient of a (zero-valued) initial state = the reverse-flow state at the segment start
                zero = torch.zeros(1, h, d, d)
                *_, ref = orc.lasd_backward(q[:, sl], k[:, sl], v[:, sl], ld[:, sl], do[:, sl], zero)
            assert_close(f"state seg {j} reverse={reverse}", ref[0], states[j], TOL_BF16)
            assert_close(f"gsum seg {j}", ld[0, sl].sum(0), gsum[j], 1e-5)
        # fold: documents {0: segs 0-1, 1: segs 2-3}
        tab = torch.tensor([[0, 1, 0, 0], [0, 0, 1, 1], [1, 1, 0, 2], [1, 0, 1, 3]], dtype=torch.int32, device=dev)
        ext = 0.1 * torch.randn(2, h, d, d, generator=g).to(dev)
        inc = torch.empty_like(states)
        rc = lib.la_lasd_fold_states(states.data_ptr(), gsum.data_ptr(), tab.data_ptr(), None, ext.data_ptr(),
                                     inc.data_ptr(), None, len(segs), h, d, d, reverse, stream)
        assert rc == 0
        dec = torch.exp(gsum).view(len(segs), h, 1, 1)
        if reverse == 0:
            want = [ext[0], states[0] + dec[0] * ext[0], ext[1], states[2] + dec[2] * ext[1]]
        else:
            want = [states[1] + dec[1] * ext[0], ext[0], states[3] + dec[3] * ext[1], ext[1]]
        for j in range(len(segs)):
            assert_close(f"incoming seg {j} reverse={reverse}", want[j], inc[j], 1e-6)


@pytest.mark.parametrize("regime", ["weak", "reference_benchmark"])
def test_vector_decay_state_pass_and_fold(lib, regime):
    """la_lavd_state_pass / la_lavd_fold_states through the C ABI against the oracle's final states
    (forward flow) and initial-state gradients (reverse flow) of the same token ranges; the strong
    decay of the reference's benchmark script must be as exact as the weak one (no range limit)."""
    from xopes_b200 import _lib
    n, h, d = 900, 2, 128
    g = torch.Generator().manual_seed(9)
    cast = lambda t: t.bfloat16().float()  # noqa: E731
    q = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    k = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
    v = cast(torch.randn(1, n, h, d, generator=g))
    do = cast(torch.randn(1, n, h, d, generator=g))
    x = torch.randn(1, n, h, d, generator=g)
    ldk = torch.nn.functional.logsigmoid(x) / (16 if regime == "weak" else 1)
    segs = [(0, 300), (300, 556), (556, 900)]
    dev = "cuda"
    qc, kc, vc, doc_, lc = (t.to(dev) for t in (q.bfloat16(), k.bfloat16(), v.bfloat16(), do.bfloat16(), ldk))
    ranges = torch.tensor(segs, dtype=torch.int64, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for reverse, (y, z) in ((0, (kc, vc)), (1, (qc, doc_))):
        states = torch.empty(len(segs), h, d, d, device=dev)
        gsum = torch.empty(len(segs), h, d, device=dev)
        assert lib.la_lavd_state_pass(y.data_ptr(), z.data_ptr(), lc.data_ptr(), ranges.data_ptr(), states.data_ptr(),
                                      gsum.data_ptr(), 1, n, h, d, d, len(segs), _lib.LA_BF16, reverse, 1, 0, stream) == 0
        for j, (a, b) in enumerate(segs):
            sl = slice(a, b)
            if reverse == 0:
                _, ref = orc.lavd_forward(q[:, sl], k[:, sl], v[:, sl], ldk[:, sl], None)
            else:
                zero = torch.zeros(1, h, d, d)
                *_, ref = orc.lavd_backward(q[:, sl], k[:, sl], v[:, sl], ldk[:, sl], None, do[:, sl], zero)
            assert_close(f"state seg {j} reverse={reverse}", ref[0], states[j], TOL_BF16)
            assert_close(f"gsum seg {j}", ldk[0, sl].sum(0), gsum[j], 1e-5)
        tab = torch.tensor([[0, 1, 0, 0], [0, 0, 0, 1], [0, 0, 1, 2]], dtype=torch.int32, device=dev)
        ext = 0.1 * torch.randn(1, h, d, d, generator=g).to(dev)
        inc = torch.empty_like(states)
        assert lib.la_lavd_fold_states(states.data_ptr(), gsum.data_ptr(), tab.data_ptr(), None, ext.data_ptr(),
                                       inc.data_ptr(), len(segs), h, d, d, reverse, stream) == 0
        dec = torch.exp(gsum).view(len(segs), h, d, 1)
        if reverse == 0:
            s1 = states[0] + dec[0] * ext[0]
            want = [ext[0], s1, states[1] + dec[1] * s1]
        else:
            s1 = states[2] + dec[2] * ext[0]
            want = [states[1] + dec[1] * s1, s1, ext[0]]
        for j in range(len(segs)):
            assert_close(f"incoming seg {j} reverse={reverse}", want[j], inc[j], 1e-6)


@pytest.mark.parametrize("regime", ["weak", "reference_benchmark"])
@pytest.mark.parametrize("b,n,h", [(1, 4096, 2), (2, 2500, 1)])
def test_vector_decay_segmented_passes(b, n, h, regime):
    """Few long sequences with vector decay: lavd_fn cuts them into segments (state-only pass, fold,
    varlen chunk passes) forward and backward; everything, the log-decay gradient and the gradient
    of the initial state included, must match the oracle on the whole sequences."""
    import xopes_b200 as xb
    from xopes_b200.lightning_attn import vector_decay as vd
    d = e = 128
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(5)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    x = torch.randn(b, n, h, d, generator=g)
    ldk = torch.nn.functional.logsigmoid(x) / (16 if regime == "weak" else 1)
    q = cast(torch.randn(b, n, h, d, generator=g))
    k = cast((1 - torch.exp(ldk)) * torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    v = cast(torch.randn(b, n, h, e, generator=g))
    s0 = 0.1 * torch.randn(b, h, d, e, generator=g)
    do = cast(torch.randn(b, n, h, e, generator=g))
    dsf = 0.1 * torch.randn(b, h, d, e, generator=g)
    qc, kc, vc = (t.to(dtype).cuda().requires_grad_() for t in (q, k, v))
    lc, s0c = ldk.cuda().requires_grad_(), s0.cuda().requires_grad_()
    assert vd._segmentation(xb.load_library(), qc, lc, None, None, b, n, h, d, e, 0) is not None
    o, sf = xb.lavd_fn(qc, kc, vc, ldk=lc, initial_state=s0c)
    ro, rsf = orc.lavd_forward(q, k, v, ldk, None, s0)
    assert_close("o", ro, o.float(), TOL_BF16)
    assert_close("final_state", rsf, sf, TOL_BF16)
    ((o.float() * do.cuda()).sum() + (sf * dsf.cuda()).sum()).backward()
    rq, rk, rv, rlk, _, rs0 = orc.lavd_backward(q, k, v, ldk, None, do, s0, dsf)
    assert_close("dq", rq, qc.grad.float(), TOL_BF16)
    assert_close("dk", rk, kc.grad.float(), TOL_BF16)
    assert_close("dv", rv, vc.grad.float(), TOL_BF16)
    assert_close("dldk", rlk, lc.grad, TOL_BF16)
    assert_close("dinitial_state", rs0, s0c.grad, TOL_BF16)
