"""GPU, 2 devices: the sequence-parallel forward and backward over real NCCL ranks (skipped on a 1-GPU box).
Each rank is a child process on its own GPU; NVLS is switched off and no kernel of this library
touches a peer's memory, so a rank ends only between steps with nothing in flight."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, exchange, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import xopes_b200 as xb
        from oracle import lightning_attn_oracle as orc
        from xopes_b200.lightning_attn.seq_parallel import token_range
        lens = [100, 700, 400, 336]
        n, h, d = sum(lens), 2, 128
        g = torch.Generator().manual_seed(11)
        cast = lambda t: t.bfloat16().float()  # noqa: E731
        q = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
        k = cast(torch.randn(1, n, h, d, generator=g) * d ** -0.5)
        v = cast(torch.randn(1, n, h, d, generator=g))
        do = cast(torch.randn(1, n, h, d, generator=g))
        ld = torch.log(1 - 2.0 ** (-5 - torch.arange(h, dtype=torch.float32) / 2))
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
        a, b = token_range(n, rank, world)
        dev = torch.device("cuda", rank)
        o, states, plan = xb.lasd_seqpar_forward(q[:, a:b].bfloat16().to(dev), k[:, a:b].bfloat16().to(dev),
                                                 v[:, a:b].bfloat16().to(dev), ld.to(dev), cu, exchange=exchange)
        torch.cuda.synchronize()
        ld_full = ld.view(1, 1, h).expand(1, n, h)
        ro, _ = orc.lasd_forward(q, k, v, ld_full, None, cu)
        errs = [orc.rel_l2(ro[:, a:b], o.float().cpu())]
        if exchange == "all_gather":  # the backward over the same ranks
            dq, dk, dv = xb.lasd_seqpar_backward(q[:, a:b].bfloat16().to(dev), k[:, a:b].bfloat16().to(dev),
                                                 v[:, a:b].bfloat16().to(dev), ld.to(dev),
                                                 do[:, a:b].bfloat16().to(dev), cu, plan.s_in)
            torch.cuda.synchronize()
            rq, rk, rv, _, _ = orc.lasd_backward(q, k, v, ld_full, do, None, None, cu)
            errs += [orc.rel_l2(r[:, a:b], x.float().cpu()) for r, x in ((rq, dq), (rk, dk), (rv, dv))]
        ret[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["all_gather", "chain"])
def test_sequence_parallel_forward_over_nccl(exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    port = 29700 + (os.getpid() + len(exchange)) % 200
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(2, port, exchange, ret), nprocs=2, join=True)
        assert len(ret) == 2 and all(err <= 1e-2 for err in ret.values()), dict(ret)
