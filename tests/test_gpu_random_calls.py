"""GPU: a seeded sweep of random calls through the public API against the CPU oracle - both decay
types, fp32 / bf16 / fp16, head dimensions from 32 to 128, fixed-length and packed variable-length
input (empty and one-token documents included), N from 1 to 2100, with and without initial state and
final-state gradient, the fused logsigmoid producer, decays given in 16 bit.  Every output and every
gradient is compared.

Tolerances: relative L2 <= 1e-5 for fp32 inputs (5e-5 for the fp32 log-decay gradients, whose
cancellation amplifies fp32 rounding on both sides at the longer lengths drawn here), <= 1e-2 for
16-bit inputs.  A gradient that is zero mathematically (one token, no state) is compared absolutely."""
import random

import pytest
import torch
import torch.nn.functional as F

from oracle import lightning_attn_oracle as orc

pytestmark = pytest.mark.gpu

DEV = "cuda"
CASES_PER_SEED = 40


def _leaf(t, dtype=None):
    t = t.detach().clone()
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV).requires_grad_()


def _one_case(rng, case):
    import xopes_b200 as xb
    kind = rng.choice(["lasd", "lasd", "lavd_k", "lavd_v", "lavd_kv"])
    dtype = rng.choice([torch.bfloat16, torch.bfloat16, torch.float16, torch.float32])
    h = rng.choice([1, 2, 3, 5])
    d = rng.choice([128, 128, 64, 96, 32, 40])
    e = rng.choice([128, 128, 64, 32, 72])
    lens = None
    if rng.random() < 0.4:
        lens = [rng.choice([0, 1, 5, 127, 128, 129, 200, 256, 300, 511, 700]) for _ in range(rng.randint(1, 6))]
        if sum(lens) == 0:
            lens[0] = 130
        b, n, nb = 1, sum(lens), len(lens)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    else:
        b = rng.choice([1, 2, 3])
        n = rng.choice([1, 7, 128, 129, 255, 256, 257, 400, 1000, 2100])
        cu, nb = None, b
    act = rng.random() < 0.3
    use_s0, use_dsf = rng.random() < 0.6, rng.random() < 0.6
    scale = rng.choice([1.0, 1.0, 0.1])
    low = dtype != torch.float32 and rng.random() < 0.4   # vector decays given in the 16-bit type
    per_head = lens is None and rng.random() < 0.3        # scalar decay as a per-head vector
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    g = torch.Generator().manual_seed(case)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    q = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    k = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    v = cast(torch.randn(b, n, h, e, generator=g))
    do = cast(torch.randn(b, n, h, e, generator=g))
    s0 = 0.1 * torch.randn(nb, h, d, e, generator=g) if use_s0 else None
    dsf = 0.1 * torch.randn(nb, h, d, e, generator=g) if use_dsf else None
    desc = (f"{kind} {dtype} b{b} n{n} h{h} d{d} e{e} lens={lens} act={act} s0={use_s0} dsf={use_dsf} "
            f"scale={scale} low={low} per_head={per_head}")
    qc, kc, vc = _leaf(q, dtype), _leaf(k, dtype), _leaf(v, dtype)
    s0c = _leaf(s0) if use_s0 else None
    cuc = None if cu is None else cu.to(DEV)
    chain = lambda r, x: (r.double() * torch.sigmoid(-x.double())).float() if act else r  # noqa: E731
    activation = "logsigmoid" if act else None
    if kind == "lasd":
        x = torch.randn(h, generator=g) + 3 if per_head else torch.randn(b, n, h, generator=g) * 2 + 3
        ld = F.logsigmoid(x.double()).float() if act else F.logsigmoid(x) * scale
        lc = _leaf(x if act else ld)
        o, sf = xb.lasd_fn(qc, kc, vc, lc, initial_state=s0c, cu_seqlens=cuc, decay_activation=activation)
        full = (lambda t: t.view(1, 1, h).expand(b, n, h).contiguous()) if per_head else (lambda t: t)
        ro, rsf = orc.lasd_forward(q, k, v, full(ld), s0, cu)
        loss = (o.float() * do.to(DEV)).sum() + ((sf * dsf.to(DEV)).sum() if use_dsf else 0.0)
        loss.backward()
        rq, rk, rv, rld, rs0 = orc.lasd_backward(q, k, v, full(ld), do, s0, dsf, cu)
        rld = chain(rld, full(x))
        if per_head:
            rld = rld.sum(dim=(0, 1))
        pairs = [("o", ro, o), ("final_state", rsf, sf), ("dq", rq, qc.grad), ("dk", rk, kc.grad),
                 ("dv", rv, vc.grad), ("dld", rld, lc.grad)]
    else:
        xk = torch.randn(b, n, h, d, generator=g) + (3 if act else 0)
        xv = torch.randn(b, n, h, e, generator=g) + (3 if act else 0)
        if low and act:
            xk, xv = cast(xk), cast(xv)
        ldk = ldv = None
        if kind in ("lavd_k", "lavd_kv"):
            ldk = F.logsigmoid(xk.double()).float() if act else F.logsigmoid(xk) * scale
        if kind in ("lavd_v", "lavd_kv"):
            ldv = F.logsigmoid(xv.double()).float() if act else F.logsigmoid(xv) * scale
        if low and not act:
            ldk, ldv = (None if t is None else cast(t) for t in (ldk, ldv))
        ink = None if ldk is None else _leaf(xk if act else ldk, dtype if low else None)
        inv = None if ldv is None else _leaf(xv if act else ldv, dtype if low else None)
        o, sf = xb.lavd_fn(qc, kc, vc, ldk=ink, ldv=inv, initial_state=s0c, cu_seqlens=cuc,
                           decay_activation=activation)
        ro, rsf = orc.lavd_forward(q, k, v, ldk, ldv, s0, cu)
        loss = (o.float() * do.to(DEV)).sum() + ((sf * dsf.to(DEV)).sum() if use_dsf else 0.0)
        loss.backward()
        rq, rk, rv, rlk, rlv, rs0 = orc.lavd_backward(q, k, v, ldk, ldv, do, s0, dsf, cu)
        pairs = [("o", ro, o), ("final_state", rsf, sf), ("dq", rq, qc.grad), ("dk", rk, kc.grad),
                 ("dv", rv, vc.grad)]
        if ldk is not None:
            pairs.append(("dldk", chain(rlk, xk), ink.grad))
        if ldv is not None:
            pairs.append(("dldv", chain(rlv, xv), inv.grad))
    if use_s0:
        pairs.append(("dinitial_state", rs0, s0c.grad))
    bad = {}
    for name, ref, got in pairs:
        ref, got = ref.float(), got.float().cpu()
        if float(ref.norm()) < 1e-6 * max(1.0, ref.numel() ** 0.5):   # zero in exact arithmetic
            err, bound = float((got - ref).abs().max()), 1e-4
        else:
            err = orc.rel_l2(ref, got)
            bound = tol * (5.0 if dtype == torch.float32 and name.startswith("dld") else 1.0)
        if not err <= bound:
            bad[name] = err
    return desc, bad


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_calls_match_the_oracle(seed):
    rng = random.Random(seed)
    failures = []
    for i in range(CASES_PER_SEED):
        desc, bad = _one_case(rng, 1000 * seed + i)
        if bad:
            failures.append((desc, bad))
    assert not failures, failures
