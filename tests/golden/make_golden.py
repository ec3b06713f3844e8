"""Generate the golden vectors under tests/golden/ from the reference itself.

Run where a checkout of the reference project (Doraemonzzz/xopes) is available and pass its path
(or set XOPES_REFERENCE_ROOT):

    python tests/golden/make_golden.py <reference_root>

The reference's torch operators are loaded BY FILE PATH (importing the `xopes` package needs a
GPU because it queries the Triton driver at import time).  For every case this script

  1. draws seeded inputs on the CPU,
  2. runs the reference forward (lasd_torch / lavd_torch) and autograd through it, or the
     reference's chunk-level fixtures (scalar_decay/torch_utils.py),
  3. checks that oracle/lightning_attn_oracle.py (oracle/chunk_fixtures.py) reproduces all of it
     (rel-L2 <= 1e-5),
  4. stores inputs and the reference's outputs in one .npz per case.

The .npz files are what the CPU tests pin the oracle against and what the GPU tests compare the
CUDA path with; the reference checkout is not needed to run the tests.
"""
import importlib.util
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import chunk_fixtures as cfx  # noqa: E402
from oracle import lightning_attn_oracle as orc  # noqa: E402


def load(ref_root, rel, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ref_root, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def g(shape, gen, scale=1.0):
    return torch.randn(*shape, generator=gen) * scale


def save(name, **arrs):
    out = {}
    for k, v in arrs.items():
        if v is None:
            continue
        out[k] = v.detach().numpy() if isinstance(v, torch.Tensor) else np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: tuple(v.shape) for k, v in out.items()})


def check(tag, ref, got, tol=1e-5):
    err = orc.rel_l2(ref, got)
    assert err <= tol, f"{tag}: oracle differs from the reference, rel-L2 {err:.3e}"
    return err


def lasd_case(ref, name, seed, b, n, h, d, e, use_init, use_dfinal, lens=None, decay="sigmoid"):
    gen = torch.Generator().manual_seed(seed)
    q = g((b, n, h, d), gen, d ** -0.5).requires_grad_()
    k = g((b, n, h, d), gen, d ** -0.5).requires_grad_()
    v = g((b, n, h, e), gen).requires_grad_()
    if decay == "sigmoid":
        ld = F.logsigmoid(g((b, n, h), gen) + 1.0).requires_grad_()
    else:  # per-head constant, the benchmark configurations' form
        ld_h = torch.log(1 - 2.0 ** (-5 - torch.arange(h, dtype=torch.float32)))
        ld = ld_h.view(1, 1, h).expand(b, n, h).contiguous().requires_grad_()
    cu = None
    nb = b
    if lens is not None:
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.long)
        assert cu[-1] == n and b == 1
        nb = len(lens)
    s0 = (0.1 * g((nb, h, d, e), gen)).requires_grad_() if use_init else None
    do = g((b, n, h, e), gen)
    dsf = g((nb, h, d, e), gen) if use_dfinal else None

    o, sf = ref.lasd_torch(q, k, v, ld, initial_state=s0, cu_seqlens=cu)
    loss = (o * do).sum() + ((sf * dsf).sum() if use_dfinal else 0.0)
    inputs = [q, k, v, ld] + ([s0] if use_init else [])
    grads = torch.autograd.grad(loss, inputs)
    dq, dk, dv, dld = grads[:4]
    ds0 = grads[4] if use_init else None

    oo, osf = orc.lasd_forward(q, k, v, ld, s0, cu)
    check(name + ".o", o, oo)
    check(name + ".state", sf, osf)
    gq, gk, gv, gld, gs0 = orc.lasd_backward(q, k, v, ld, do, s0, dsf, cu)
    for t, r, x in (("dq", dq, gq), ("dk", dk, gk), ("dv", dv, gv), ("dld", dld, gld)):
        check(f"{name}.{t}", r, x)
    if use_init:
        check(name + ".dinitial", ds0, gs0)
    save(name, q=q, k=k, v=v, ld=ld, initial_state=s0, do=do, dfinal_state=dsf, cu_seqlens=cu,
         o=o, final_state=sf, dq=dq, dk=dk, dv=dv, dld=dld, dinitial_state=ds0)


def lavd_case(ref, name, seed, b, n, h, d, e, use_ldv, use_init, use_dfinal, share_k=False,
              lens=None):
    gen = torch.Generator().manual_seed(seed)
    q = g((b, n, h, d), gen, d ** -0.5).requires_grad_()
    ldk = F.logsigmoid(g((b, n, h, d), gen) + 1.0).requires_grad_()
    ldv = F.logsigmoid(g((b, n, h, e), gen) + 1.0).requires_grad_() if use_ldv else None
    k = None if share_k else g((b, n, h, d), gen, d ** -0.5).requires_grad_()
    v = g((b, n, h, e), gen).requires_grad_()
    cu = None
    nb = b
    if lens is not None:
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.long)
        nb = len(lens)
    s0 = (0.1 * g((nb, h, d, e), gen)).requires_grad_() if use_init else None
    do = g((b, n, h, e), gen)
    dsf = g((nb, h, d, e), gen) if use_dfinal else None

    if cu is None:
        o, sf = ref.lavd_torch(q, k, v, ldk, ldv, initial_state=s0)
    else:
        # lavd_torch never reads cu_seqlens (lavd_torch.py:16): run it once per document,
        # which is what lasd_torch's varlen branch does for scalar decay.
        outs, sts = [], []
        for i in range(nb):
            a0, a1 = int(cu[i]), int(cu[i + 1])
            oi, si = ref.lavd_torch(
                q[:, a0:a1], None if k is None else k[:, a0:a1], v[:, a0:a1], ldk[:, a0:a1],
                None if ldv is None else ldv[:, a0:a1],
                initial_state=None if s0 is None else s0[i:i + 1])
            outs.append(oi)
            sts.append(si)
        o, sf = torch.cat(outs, 1), torch.cat(sts, 0)
    loss = (o * do).sum() + ((sf * dsf).sum() if use_dfinal else 0.0)
    names = ["q", "ldk", "v"] + (["ldv"] if use_ldv else []) + ([] if share_k else ["k"]) + \
        (["s0"] if use_init else [])
    tens = dict(q=q, ldk=ldk, v=v, ldv=ldv, k=k, s0=s0)
    grads = dict(zip(names, torch.autograd.grad(loss, [tens[x] for x in names])))

    oo, osf = orc.lavd_forward(q, k, v, ldk, ldv, s0, cu)
    check(name + ".o", o, oo)
    check(name + ".state", sf, osf)
    gq, gk, gv, gldk, gldv, gs0 = orc.lavd_backward(q, k, v, ldk, ldv, do, s0, dsf, cu)
    check(name + ".dq", grads["q"], gq)
    check(name + ".dv", grads["v"], gv)
    check(name + ".dldk", grads["ldk"], gldk)
    if not share_k:
        check(name + ".dk", grads["k"], gk)
    if use_ldv:
        check(name + ".dldv", grads["ldv"], gldv)
    if use_init:
        check(name + ".dinitial", grads["s0"], gs0)
    save(name, q=q, k=k, v=v, ldk=ldk, ldv=ldv, initial_state=s0, do=do, dfinal_state=dsf,
         cu_seqlens=cu, o=o, final_state=sf, dq=grads["q"], dk=grads.get("k"), dv=grads["v"],
         dldk=grads["ldk"], dldv=grads.get("ldv"), dinitial_state=grads.get("s0"))


def chunk_fixture_case(ref_root, name, seed, b, n, h, d, e, block):
    """Outputs of the reference's chunk-level torch fixtures (scalar_decay/torch_utils.py): per-chunk
    intra outputs, each chunk's own state, the scanned states (forward and reverse) and the inter
    outputs.  The file imports `contiguous` from the xopes package, which cannot be imported without
    a GPU; a pass-through stand-in of that decorator (it only calls .contiguous() on tensor
    arguments, xopes/utils/utils.py:15-26) is registered for the by-path import."""
    import types
    stub = types.ModuleType("xopes.utils")
    stub.contiguous = lambda fn: fn
    saved = {m: sys.modules.get(m) for m in ("xopes", "xopes.utils")}
    sys.modules["xopes"], sys.modules["xopes.utils"] = types.ModuleType("xopes"), stub
    try:
        tu = load(ref_root, "xopes/ops/lightning_attn/scalar_decay/torch_utils.py", "ref_lasd_torch_utils")
    finally:
        for m, old in saved.items():
            if old is None:
                sys.modules.pop(m, None)
            else:
                sys.modules[m] = old
    gen = torch.Generator().manual_seed(seed)
    q = g((b, n, h, d), gen, d ** -0.5)
    k = g((b, n, h, d), gen, d ** -0.5)
    v = g((b, n, h, e), gen)
    ld = F.logsigmoid(g((b, n, h), gen) + 1.0)
    s0 = 0.1 * g((b, h, d, e), gen)
    out = dict(q=q, k=k, v=v, ld=ld, initial_state=s0, block=torch.tensor(block))
    for rev, tag in ((False, "fwd"), (True, "rev")):
        out["intra_" + tag] = tu.lasd_intra_torch(q, k, v, ld, reverse=rev, BLOCK_N=block)
        loc, glob = tu.compute_states(k, v, ld, s0, BLOCK_N=block, reverse=rev)
        out["local_" + tag], out["global_" + tag] = loc, glob
        check(f"{name}.intra_{tag}", out["intra_" + tag], cfx.lasd_chunk_intra(q, k, v, ld, block, rev))
        oloc, oglob = cfx.lasd_chunk_states(k, v, ld, s0, block, rev)
        check(f"{name}.local_{tag}", loc, oloc)
        check(f"{name}.global_{tag}", glob, oglob)
    out["inter"] = tu.lasd_inter_torch(q, k, v, ld, s0, BLOCK_N=block)
    check(name + ".inter", out["inter"], cfx.lasd_chunk_inter(q, k, v, ld, s0, block))
    save(name, **out)


def normgate_case(ref_root, name, seed):
    """Outputs and autograd gradients of the reference's normalize_torch with a gate
    (xopes/ops/normalize/normalize/normalize_torch.py) for every activation, both gate positions,
    with and without mean subtraction.  The file imports act_torch from the xopes package (not
    importable without a GPU); the activation table it needs is loaded by path from
    xopes/ops/act/_act_torch/act_torch.py and offered under that module name."""
    import types
    from oracle import normalize_oracle as norc
    acts = load(ref_root, "xopes/ops/act/_act_torch/act_torch.py", "ref_act_table")
    stub = types.ModuleType("xopes.ops.act")
    stub.act_torch = lambda x, act, dim=None: acts.ACT_TORCH_DICT[act](x)
    names = ("xopes", "xopes.ops", "xopes.ops.act")
    saved = {m: sys.modules.get(m) for m in names}
    sys.modules["xopes"], sys.modules["xopes.ops"] = types.ModuleType("xopes"), types.ModuleType("xopes.ops")
    sys.modules["xopes.ops.act"] = stub
    try:
        nt = load(ref_root, "xopes/ops/normalize/normalize/normalize_torch.py", "ref_normalize_torch")
    finally:
        for m, old in saved.items():
            if old is None:
                sys.modules.pop(m, None)
            else:
                sys.modules[m] = old
    gen = torch.Generator().manual_seed(seed)
    rows, groups, e = 7, 3, 40
    out = {}
    x = g((2, rows, groups * e), gen)
    gate = g((2, rows, groups * e), gen)
    w = 1 + 0.1 * g((groups * e,), gen)
    b = 0.1 * g((groups * e,), gen)
    do = g((2, rows, groups * e), gen)
    out.update(x=x, gate=gate, weight=w, bias=b, do=do, num_groups=torch.tensor(groups))
    idx = 0
    for act in ("none", "relu", "sigmoid", "silu"):
        for pos in ("pre", "post"):
            for use_mean in (False, True):
                xs, gs, ws, bs = (t.clone().requires_grad_() for t in (x, gate, w, b))
                o = nt.normalize_torch(xs, ws, bs, gate=gs, gate_act=act, gate_pos=pos, c=e ** 0.5, eps=1e-5,
                                       use_mean=use_mean, num_groups=groups)
                grads = torch.autograd.grad((o * do).sum(), [xs, gs, ws, bs])
                xo, go, wo, bo = (t.clone().requires_grad_() for t in (x, gate, w, b))
                oo = norc.normalize_gate(xo, wo, bo, go, act, pos, e ** 0.5, 1e-5, use_mean, groups)
                og = torch.autograd.grad((oo * do.double()).sum(), [xo, go, wo, bo])
                tag = f"{act}_{pos}_{int(use_mean)}"
                check(f"{name}.{tag}.o", o, oo.float())
                for nme, r, got in zip(("dx", "dgate", "dweight", "dbias"), grads, og):
                    check(f"{name}.{tag}.{nme}", r, got.float())
                    out[f"{tag}.{nme}"] = r
                out[f"{tag}.o"] = o
                idx += 1
    save(name, **out)


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("XOPES_REFERENCE_ROOT")
    if not ref_root:
        raise SystemExit("usage: make_golden.py <path to a checkout of Doraemonzzz/xopes>")
    lasd = load(ref_root, "xopes/ops/lightning_attn/scalar_decay/lasd_torch.py", "ref_lasd_torch")
    lavd = load(ref_root, "xopes/ops/lightning_attn/vector_decay/lavd_torch.py", "ref_lavd_torch")
    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # scalar decay: ragged lengths around the 128-token chunk, with and without states
    lasd_case(lasd, "lasd_ragged_init", 11, 2, 37, 3, 16, 24, True, True)
    lasd_case(lasd, "lasd_ragged_noinit", 12, 2, 65, 2, 33, 17, False, False)
    lasd_case(lasd, "lasd_chunky_d64", 13, 1, 300, 2, 64, 64, True, True)
    lasd_case(lasd, "lasd_d128_perhead", 14, 1, 257, 2, 128, 128, True, False, decay="perhead")
    lasd_case(lasd, "lasd_varlen", 15, 1, 90, 2, 32, 32, True, True, lens=[1, 40, 17, 32])
    lasd_case(lasd, "lasd_decode", 16, 3, 1, 4, 64, 48, True, True)
    # chunk-level intermediates (ragged last chunk)
    chunk_fixture_case(ref_root, "chunkfx_lasd", 17, 1, 300, 2, 16, 24, 128)
    normgate_case(ref_root, "normgate", 18)
    # vector decay
    lavd_case(lavd, "lavd_k_only", 21, 2, 41, 2, 16, 24, False, True, True)
    lavd_case(lavd, "lavd_kv", 22, 2, 35, 2, 24, 16, True, True, True)
    lavd_case(lavd, "lavd_k_noinit_d64", 23, 1, 200, 2, 64, 64, False, False, False)
    lavd_case(lavd, "lavd_share_k", 24, 1, 33, 2, 16, 16, True, False, True, share_k=True)
    lavd_case(lavd, "lavd_varlen", 25, 1, 70, 2, 32, 16, False, True, True, lens=[30, 1, 39])
    lavd_case(lavd, "lavd_decode", 26, 3, 1, 4, 64, 48, False, True, True)


if __name__ == "__main__":
    main()
