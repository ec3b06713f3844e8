"""Seeded synthetic inputs of the five benchmark configurations (and scaled-down versions of
them for the parity tests).  Everything is drawn on the CPU from one torch.Generator in a fixed
order, in fp32, and cast afterwards, so the CUDA path and the CPU oracle see identical values.

The reference measures on random tensors only (benchmarks/lightning_attention/benchmark.py:299-324);
no dataset is involved.  "N(0, 0.01)" initial states are read as variance 0.01, i.e. std 0.1.
"""
import math

import torch
import torch.nn.functional as F


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def per_head_log_decay(h, step):
    """ld_h = log(1 - 2^(-5 - step*h)), h = 0..H-1."""
    idx = torch.arange(h, dtype=torch.float32)
    return torch.log(1 - torch.pow(2.0, -5 - step * idx))


def lasd_inputs(b, n, h, d, e, dtype=torch.bfloat16, seed=0, decay_step=None, use_state=True,
                use_do=True):
    """Configurations 1 and 2: q,k,v ~ N(0,1), q and k scaled by 1/sqrt(D); per-head decay
    ld_h = log(1 - 2^(-5 - step*h)) with step = 8/H unless given; optional initial state
    0.1*N(0,1) fp32 and upstream gradient do ~ N(0,1)."""
    g = _gen(seed)
    q = torch.randn(b, n, h, d, generator=g) * d ** -0.5
    k = torch.randn(b, n, h, d, generator=g) * d ** -0.5
    v = torch.randn(b, n, h, e, generator=g)
    step = 8.0 / h if decay_step is None else decay_step
    out = dict(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype), ld=per_head_log_decay(h, step))
    if use_state:
        out["initial_state"] = 0.1 * torch.randn(b, h, d, e, generator=g)
    if use_do:
        out["do"] = torch.randn(b, n, h, e, generator=g).to(dtype)
    return out


def lavd_inputs(b, n, h, d, e, dtype=torch.bfloat16, seed=0):
    """Configuration 3: ldk = logsigmoid(x)/16, k = (1-exp(ldk)) * k_raw, k_raw ~ N(0,1)/sqrt(D);
    q, v, do ~ N(0,1); no initial state."""
    g = _gen(seed)
    x = torch.randn(b, n, h, d, generator=g)
    ldk = F.logsigmoid(x) / 16
    k_raw = torch.randn(b, n, h, d, generator=g) * d ** -0.5
    k = (1 - torch.exp(ldk)) * k_raw
    q = torch.randn(b, n, h, d, generator=g)
    v = torch.randn(b, n, h, e, generator=g)
    do = torch.randn(b, n, h, e, generator=g)
    return dict(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype), ldk=ldk, do=do.to(dtype))


def decode_inputs(b, h, d, e, steps, vector, dtype=torch.bfloat16, seed=0):
    """Configuration 4: carried fp32 state 0.1*N(0,1); per step fresh q,k,v ~ N(0,1)/sqrt(D) and,
    for the vector variant, ldk = logsigmoid(N(0,1))/16."""
    g = _gen(seed)
    state = 0.1 * torch.randn(b, h, d, e, generator=g)
    toks = []
    for _ in range(steps):
        q = (torch.randn(b, 1, h, d, generator=g) * d ** -0.5).to(dtype)
        k = (torch.randn(b, 1, h, d, generator=g) * d ** -0.5).to(dtype)
        v = (torch.randn(b, 1, h, e, generator=g) * d ** -0.5).to(dtype)
        t = dict(q=q, k=k, v=v)
        if vector:
            t["ldk"] = F.logsigmoid(torch.randn(b, 1, h, d, generator=g)) / 16
        toks.append(t)
    return dict(state=state, ld=per_head_log_decay(h, 8.0 / h), steps=toks)


def varlen_doc_lengths(n_total, n_docs, seed=0):
    """Configuration 5: lengths uniform-random from the seed, normalised to the total; the remainder
    goes to the last document and every document has at least one token."""
    g = _gen(seed)
    w = torch.rand(n_docs, generator=g)
    lens = torch.floor(w / w.sum() * n_total).to(torch.int64).clamp_(min=1)
    lens[-1] += n_total - int(lens.sum())
    assert int(lens.min()) >= 1 and int(lens.sum()) == n_total
    return lens


def varlen_inputs(n_total, n_docs, h, d, e, dtype=torch.bfloat16, seed=0, block=65536,
                  token_range=None, device="cpu"):
    """Configuration 5: one packed stream, q,k,v ~ N(0,1), q and k scaled by 1/sqrt(D);
    ld_h = log(1 - 2^(-5 - h/2)).  The stream is generated in blocks of `block` tokens, each from
    its own generator seeded by (seed, block index), so a rank can generate just its own token
    range [a, b) and still see exactly the values of the whole stream.  With a CUDA `device` the
    blocks are drawn by that device's generator (the same values on every GPU of one model, not
    the CPU generator's values): the 1M-token stream is 6 G normal variates, minutes on the host."""
    lens = varlen_doc_lengths(n_total, n_docs, seed)
    cu = torch.zeros(n_docs + 1, dtype=torch.int64)
    cu[1:] = torch.cumsum(lens, 0)
    a, b = token_range if token_range is not None else (0, n_total)
    device = torch.device(device)
    q = torch.empty(1, b - a, h, d, dtype=dtype, device=device)
    k = torch.empty(1, b - a, h, d, dtype=dtype, device=device)
    v = torch.empty(1, b - a, h, e, dtype=dtype, device=device)
    for j in range(a // block, (b + block - 1) // block):
        s0, s1 = j * block, min((j + 1) * block, n_total)
        t = s1 - s0
        g = torch.Generator(device=device).manual_seed((seed + 1) * 100003 + j)
        qb = (torch.randn(t, h, d, generator=g, device=device) * d ** -0.5).to(dtype)
        kb = (torch.randn(t, h, d, generator=g, device=device) * d ** -0.5).to(dtype)
        vb = torch.randn(t, h, e, generator=g, device=device).to(dtype)
        lo, hi = max(s0, a), min(s1, b)
        q[0, lo - a:hi - a] = qb[lo - s0:hi - s0]
        k[0, lo - a:hi - a] = kb[lo - s0:hi - s0]
        v[0, lo - a:hi - a] = vb[lo - s0:hi - s0]
    return dict(q=q, k=k, v=v, ld=per_head_log_decay(h, 0.5), cu_seqlens=cu)


# the five configurations at full size
CONFIGS = {
    "C1": dict(kind="lasd_fwd", B=2, N=512, H=8, D=64, E=64, dtype="float32", decay_step=1.0),
    "C2": dict(kind="lasd_fwd_bwd", B=8, N=8192, H=32, D=128, E=128, dtype="bfloat16"),
    "C3": dict(kind="lavd_fwd_bwd", B=4, N=16384, H=16, D=128, E=128, dtype="bfloat16"),
    "C4": dict(kind="decode", B=256, H=32, D=128, E=128, steps=64, dtype="bfloat16"),
    "C5": dict(kind="lasd_varlen_fwd", N=1048576, docs=64, H=16, D=128, E=128, dtype="bfloat16"),
}

# algorithmic work per token per head at D = E = 128, chunk 128, causal tiles counted at half
FLOP_FWD = 98304
FLOP_BWD = 212992
BYTES_LASD_FWD = 1024
BYTES_LASD_BWD = 1792
BYTES_LAVD_FWD = 1536
BYTES_LAVD_BWD = 2816


def decode_bytes_per_step(b, h, d, e, vector):
    """state read + written (fp32), q,k,v,o (16-bit), and the decay: 4 B scalar or D*4 B vector."""
    per_bh = 2 * d * e * 4 + (2 * d + 2 * e) * 2 + (d * 4 if vector else 4)
    return b * h * per_bh
