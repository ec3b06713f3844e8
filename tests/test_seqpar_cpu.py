"""CPU: host-side logic of the sequence-parallel forward -- document sharding, the fold of the
published chunk-end states, and the whole protocol over gloo ranks (world_size 2 and 3), with the
oracle standing in for the local CUDA forward."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def test_shard_documents_intersects_ranges():
    from xopes_b200.lightning_attn.seq_parallel import shard_documents, token_range
    cu = [0, 10, 70, 96]
    assert token_range(96, 1, 3) == (32, 64)
    p0 = shard_documents(cu, 0, 32)
    assert (p0.local_cu, p0.doc_ids, p0.open_start, p0.open_end) == ([0, 10, 32], [0, 1], False, True)
    p1 = shard_documents(cu, 32, 64)
    assert (p1.local_cu, p1.doc_ids, p1.open_start, p1.open_end) == ([0, 32], [1], True, True)
    p2 = shard_documents(cu, 64, 96)
    assert (p2.local_cu, p2.doc_ids, p2.open_start, p2.open_end) == ([0, 6, 32], [1, 2], True, False)
    # a boundary that falls exactly on a rank boundary leaves nothing open
    p = shard_documents([0, 32, 64], 32, 64)
    assert (p.local_cu, p.open_start, p.open_end) == ([0, 32], False, False)


def test_fold_matches_chain_of_steps():
    from xopes_b200.lightning_attn.seq_parallel import fold_incoming_state, fold_incoming_state_step
    h, d, e = 2, 3, 4
    g = torch.Generator().manual_seed(0)
    rows = torch.randn(4, h * d * e + h + 2, generator=g)
    rows[:, -2:] = torch.tensor([[1., 0.], [1., 1.], [0., 0.], [1., 0.]])
    s = torch.zeros(h, d, e)
    for r in range(4):
        assert torch.allclose(fold_incoming_state(rows, r, h, d, e), s, atol=1e-6)
        s = fold_incoming_state_step(rows[r], s, h, d, e)


def _oracle_forward(q, k, v, ld, local_cu):
    from oracle import lightning_attn_oracle as orc
    cu = torch.tensor(local_cu, dtype=torch.int64)
    return orc.lasd_forward(q, k, v, ld, None, cu)


def _torch_correct(q, o, cum, s_in, t1):
    o[0, :t1] += torch.exp(cum).unsqueeze(-1) * torch.einsum("thd,hde->the", q[0, :t1].float(), s_in)


def _worker(rank, world, port, lens, per_head, exchange, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import lightning_attn_oracle as orc
        from xopes_b200.lightning_attn.seq_parallel import lasd_seqpar_forward, token_range
        n, h, d, e = sum(lens), 2, 8, 8
        g = torch.Generator().manual_seed(5)
        q = torch.randn(1, n, h, d, generator=g) * d ** -0.5
        k = torch.randn(1, n, h, d, generator=g) * d ** -0.5
        v = torch.randn(1, n, h, e, generator=g)
        if per_head:
            ld = torch.log(1 - 2.0 ** (-3 - torch.arange(h, dtype=torch.float32)))
            ld_full = ld.view(1, 1, h).expand(1, n, h)
        else:
            ld_full = torch.nn.functional.logsigmoid(torch.randn(1, n, h, generator=g) + 2)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
        a, b = token_range(n, rank, world)
        ld_arg = ld if per_head else ld_full[:, a:b]
        o, states, plan = lasd_seqpar_forward(q[:, a:b], k[:, a:b], v[:, a:b], ld_arg, cu,
                                              exchange=exchange, local_forward=_oracle_forward,
                                              correct=_torch_correct)
        ro, rs = orc.lasd_forward(q, k, v, ld_full, None, cu)
        err_o = float((o - ro[:, a:b]).abs().max())
        # documents that END on this rank must carry their complete final state
        err_s = 0.0
        for j, doc in enumerate(plan.doc_ids):
            if int(cu[doc + 1]) <= b:
                err_s = max(err_s, float((states[j] - rs[doc]).abs().max()))
        ret[rank] = (err_o, err_s)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["all_gather", "chain"])
@pytest.mark.parametrize("world,lens,per_head", [
    (2, [5, 20, 15], False),      # one document crosses the cut
    (3, [10, 60, 26], True),      # a document covers a whole rank (both ends open)
    (3, [32, 32, 32], False),     # boundaries coincide with the cuts: nothing to exchange
])
def test_protocol_over_gloo_ranks(world, lens, per_head, exchange):
    port = 29500 + (os.getpid() + world * 7 + len(exchange)) % 2000
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, lens, per_head, exchange, ret), nprocs=world, join=True)
        assert len(ret) == world
        for r in range(world):
            err_o, err_s = ret[r]
            assert err_o < 1e-5 and err_s < 1e-5, f"rank {r}: o {err_o:.2e} state {err_s:.2e}"


def _oracle_backward(q, k, v, ld, do, local_cu, s0):
    from oracle import lightning_attn_oracle as orc
    cu = torch.tensor(local_cu, dtype=torch.int64)
    t, h = q.shape[1], q.shape[2]
    ld_full = ld.view(1, 1, h).expand(1, t, h) if ld.dim() == 1 else ld
    dq, dk, dv, _, ds0 = orc.lasd_backward(q, k, v, ld_full, do, s0, None, cu)
    if s0 is None:  # the oracle returns no state gradient without an initial state
        zero = torch.zeros(len(local_cu) - 1, h, q.shape[3], v.shape[3])
        dq, dk, dv, _, ds0 = orc.lasd_backward(q, k, v, ld_full, do, zero, None, cu)
    return dq, dk, dv, ds0


def _torch_correct_bwd(x, out, cum, s_in, t1):
    out[0, :t1] += torch.exp(cum).unsqueeze(-1) * torch.einsum("thd,hde->the", x[0, :t1].float(), s_in)


def _worker_bwd(rank, world, port, lens, per_head, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import lightning_attn_oracle as orc
        from xopes_b200.lightning_attn.seq_parallel import (lasd_seqpar_backward, lasd_seqpar_forward,
                                                            token_range)
        n, h, d, e = sum(lens), 2, 8, 8
        g = torch.Generator().manual_seed(6)
        q = torch.randn(1, n, h, d, generator=g) * d ** -0.5
        k = torch.randn(1, n, h, d, generator=g) * d ** -0.5
        v = torch.randn(1, n, h, e, generator=g)
        do = torch.randn(1, n, h, e, generator=g)
        if per_head:
            ld = torch.log(1 - 2.0 ** (-3 - torch.arange(h, dtype=torch.float32)))
            ld_full = ld.view(1, 1, h).expand(1, n, h)
        else:
            ld_full = torch.nn.functional.logsigmoid(torch.randn(1, n, h, generator=g) + 2)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
        a, b = token_range(n, rank, world)
        ld_arg = ld if per_head else ld_full[:, a:b]
        _, _, plan = lasd_seqpar_forward(q[:, a:b], k[:, a:b], v[:, a:b], ld_arg, cu,
                                         local_forward=_oracle_forward, correct=_torch_correct)
        dq, dk, dv = lasd_seqpar_backward(q[:, a:b], k[:, a:b], v[:, a:b], ld_arg, do[:, a:b], cu, plan.s_in,
                                          local_backward=_oracle_backward, correct=_torch_correct_bwd)
        rq, rk, rv, _, _ = orc.lasd_backward(q, k, v, ld_full, do, None, None, cu)
        ret[rank] = tuple(float((x - r[:, a:b]).abs().max()) for x, r in ((dq, rq), (dk, rk), (dv, rv)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,lens,per_head", [
    (2, [5, 20, 15], False),      # one document crosses the cut
    (3, [10, 60, 26], True),      # a document covers a whole rank (both ends open)
    (3, [32, 32, 32], False),     # boundaries coincide with the cuts: nothing to exchange
])
def test_backward_protocol_over_gloo_ranks(world, lens, per_head):
    port = 31500 + (os.getpid() + world * 11) % 2000
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker_bwd, args=(world, port, lens, per_head, ret), nprocs=world, join=True)
        assert len(ret) == world
        for r in range(world):
            assert max(ret[r]) < 1e-5, f"rank {r}: dq, dk, dv max abs errors {ret[r]}"


def _worker_missing(rank, world, port, ret):
    """Rank 1 never joins the exchange (it leaves between steps, nothing in flight); rank 0 must get
    an error within the group's timeout instead of blocking."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from xopes_b200.lightning_attn.seq_parallel import SeqParExchangeError, lasd_seqpar_forward, token_range
    n, h, d = 40, 2, 8
    g = torch.Generator().manual_seed(1)
    q = torch.randn(1, n, h, d, generator=g)
    ld = torch.log(1 - 2.0 ** (-3 - torch.arange(h, dtype=torch.float32)))
    cu = torch.tensor([0, 30, 40], dtype=torch.int64)
    a, b = token_range(n, rank, world)
    if rank == 1:
        time.sleep(1.0)   # leaves without publishing its summary
        ret[rank] = "left"
        return
    t0 = time.perf_counter()
    try:
        lasd_seqpar_forward(q[:, a:b], q[:, a:b], q[:, a:b], ld, cu, local_forward=_oracle_forward,
                            correct=_torch_correct)
        ret[rank] = "no error"
    except SeqParExchangeError:
        ret[rank] = ("error", time.perf_counter() - t0)


def test_missing_rank_turns_into_an_error_not_a_hang():
    port = 33500 + os.getpid() % 2000
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker_missing, args=(2, port, ret), nprocs=2, join=True)
        assert ret[1] == "left"
        assert ret[0][0] == "error" and ret[0][1] < 30.0, ret[0]


def _worker_late(rank, world, port, ret):
    """A rank that publishes late (but inside the timeout) changes nothing in the result."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    try:
        from oracle import lightning_attn_oracle as orc
        from xopes_b200.lightning_attn.seq_parallel import lasd_seqpar_forward, token_range
        n, h, d = 40, 2, 8
        g = torch.Generator().manual_seed(1)
        q = torch.randn(1, n, h, d, generator=g) * 0.3
        ld = torch.log(1 - 2.0 ** (-3 - torch.arange(h, dtype=torch.float32)))
        cu = torch.tensor([0, 30, 40], dtype=torch.int64)
        a, b = token_range(n, rank, world)
        if rank == 0:
            time.sleep(1.5)
        o, _, _ = lasd_seqpar_forward(q[:, a:b], q[:, a:b], q[:, a:b], ld, cu, local_forward=_oracle_forward,
                                      correct=_torch_correct)
        ro, _ = orc.lasd_forward(q, q, q, ld.view(1, 1, h).expand(1, n, h), None, cu)
        ret[rank] = float((o - ro[:, a:b]).abs().max())
    finally:
        dist.destroy_process_group()


def test_late_rank_still_gives_the_right_result():
    port = 35500 + os.getpid() % 2000
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker_late, args=(2, port, ret), nprocs=2, join=True)
        assert len(ret) == 2 and max(ret.values()) < 1e-5, dict(ret)


def test_segment_planning():
    from xopes_b200.lightning_attn import segmented as sg
    assert sg.auto_cap(131072, 16, 148) % 128 == 0 and sg.auto_cap(100, 16, 148) == 1024
    seg_cu, first, last = sg.plan_segments([(0, 300), (300, 5000), (5000, 5100)], 1024)
    assert seg_cu[0] == 0 and seg_cu[-1] == 5100 and len(seg_cu) == len(first) + 1
    assert first == [1, 1, 0, 0, 0, 0, 1] and last == [0, 5, 6]
    # cuts inside a document fall on its 128-token chunk boundaries
    for i in range(2, 6):
        assert (seg_cu[i] - 300) % 128 == 0
    assert not sg.worth_segmenting([(0, 8192)] * 8, 32, sg.auto_cap(8 * 8192, 32, 148), 148)   # plenty of CTAs already
    assert sg.worth_segmenting([(0, 32768)], 16, sg.auto_cap(32768, 16, 148), 148)
