"""CPU oracle for the lightning-attention hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the sequential recurrences that
define the reference operators:

* scalar decay (lasd):   s_t = exp(ld_t) * s_{t-1} + k_t v_t^T ,  o_t = q_t^T s_t
  (reference: xopes/ops/lightning_attn/scalar_decay/lasd_torch.py:9-105)
* vector decay (lavd):   s_t = (exp(ldk_t) exp(ldv_t)^T) * s_{t-1} + k_t v_t^T , o_t = q_t^T s_t
  (reference: xopes/ops/lightning_attn/vector_decay/lavd_torch.py:7-97)

and their gradients written out as two explicit scans, the same scans the reference's
recurrence kernels perform (xopes/ops/lightning_attn/scalar_decay/lasd_recurrence_triton.py:176-494,
xopes/ops/lightning_attn/vector_decay/lavd_recurrence_triton.py:230-700).  The explicit scans need
O(B*H*D*E) memory, where autograd through the reference loop needs N times that.

Nothing in the product imports this file: only tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py may.  It is the checker, never the thing that is
shipped or measured as the product.

Parity pinning: every function here is checked against the reference's own lasd_torch /
lavd_torch (forward) and autograd through them (backward) by tests/golden/make_golden.py, which
imports the reference by file path and commits input/output vectors under tests/golden/.  The
reference's tests hold no golden vectors of their own (they compare against the same torch
functions on seeded random inputs), so the committed vectors are outputs of the reference run
in the build container.
"""
from typing import Optional, Tuple

import torch


def _f(x, acc):
    return None if x is None else x.detach().to("cpu").to(acc)


def _expand_ld(ld, b, n, h, acc):
    """Accept ld of shape (B,N,H) or a per-head (H,) vector (lightning_attn/__init__.py:35)."""
    ld = _f(ld, acc)
    if ld.dim() == 1:
        ld = ld.view(1, 1, h).expand(b, n, h)
    return ld


def _doc_ranges(b, n, cu_seqlens):
    if cu_seqlens is None:
        return None
    cu = [int(x) for x in cu_seqlens.detach().cpu().tolist()]
    return [(cu[i], cu[i + 1]) for i in range(len(cu) - 1)]


def _init_state(initial_state, nb, h, d, e, acc):
    """initial_state may be (B,H,D,E), (1,H,D,E) or (H,D,E)
    (scalar_decay/lasd_parallel_triton.py:855-859, lasd_torch.py:45-48,69-75)."""
    if initial_state is None:
        return torch.zeros(nb, h, d, e, dtype=acc)
    s = _f(initial_state, acc)
    if s.dim() == 4 and s.shape[0] == 1 and nb != 1:
        s = s.squeeze(0)
    if s.dim() == 3:
        s = s.unsqueeze(0).expand(nb, h, d, e)
    return s.clone()


# --------------------------------------------------------------------------------------
# scalar decay
# --------------------------------------------------------------------------------------
def lasd_forward(q, k, v, ld, initial_state=None, cu_seqlens=None, acc=torch.float32):
    """Forward recurrence (lasd_torch.py:50-59; varlen branch :61-103).

    Returns (o, final_state) with o in `acc` precision (cast it to q.dtype to obtain what the
    reference returns) and final_state (B,H,D,E) -- (M,H,D,E) with cu_seqlens -- in `acc`.
    """
    b, n, h, d = q.shape
    e = v.shape[-1]
    qf, kf, vf = _f(q, acc), _f(k, acc), _f(v, acc)
    ldf = _expand_ld(ld, b, n, h, acc)
    docs = _doc_ranges(b, n, cu_seqlens)
    o = torch.zeros(b, n, h, e, dtype=acc)
    if docs is None:
        state = _init_state(initial_state, b, h, d, e, acc)
        for t in range(n):
            lam = torch.exp(ldf[:, t]).unsqueeze(-1).unsqueeze(-1)
            state = lam * state + kf[:, t].unsqueeze(-1) * vf[:, t].unsqueeze(-2)
            o[:, t] = torch.einsum("bhd,bhde->bhe", qf[:, t], state)
        return o, state
    assert b == 1, "cu_seqlens is only supported for batch size 1"
    m = len(docs)
    state0 = _init_state(initial_state, m, h, d, e, acc)
    finals = []
    for i, (s0, s1) in enumerate(docs):
        st = state0[i]
        for t in range(s0, s1):
            lam = torch.exp(ldf[0, t]).unsqueeze(-1).unsqueeze(-1)
            st = lam * st + kf[0, t].unsqueeze(-1) * vf[0, t].unsqueeze(-2)
            o[0, t] = torch.einsum("hd,hde->he", qf[0, t], st)
        finals.append(st)
    return o, torch.stack(finals, 0)


def lasd_backward(q, k, v, ld, do, initial_state=None, dfinal_state=None, cu_seqlens=None,
                  acc=torch.float32):
    """Gradients of lasd by two explicit scans.

    Forward-direction scan  : dq_t = s_t do_t                        (lasd_recurrence_triton.py:176-276)
    Reverse-direction scan  : ds_t = q_t do_t^T + exp(ld_{t+1}) ds_{t+1}, ds_N += dfinal;
                              dk_t = ds_t v_t, dv_t = ds_t^T k_t; dinitial = exp(ld_1) ds_1
                                                                     (lasd_recurrence_triton.py:279-400)
    dld_t = sum_{s>=t} (q_s.dq_s - k_s.dk_s) + <s_N, dfinal>          (lasd_recurrence_triton.py:473-494)

    Returns dq, dk, dv, dld (B,N,H), dinitial_state, all in `acc`.
    """
    b, n, h, d = q.shape
    e = v.shape[-1]
    qf, kf, vf, dof = _f(q, acc), _f(k, acc), _f(v, acc), _f(do, acc)
    ldf = _expand_ld(ld, b, n, h, acc)
    docs = _doc_ranges(b, n, cu_seqlens)
    dq = torch.zeros_like(qf)
    dk = torch.zeros_like(kf)
    dv = torch.zeros_like(vf)
    dld = torch.zeros(b, n, h, dtype=acc)

    def run(bsl, t0, t1, s_init, ds_fin):
        # bsl: batch slice (slice object); tokens [t0,t1); s_init (nb,h,d,e); ds_fin or None
        st = s_init.clone()
        for t in range(t0, t1):
            lam = torch.exp(ldf[bsl, t]).unsqueeze(-1).unsqueeze(-1)
            st = lam * st + kf[bsl, t].unsqueeze(-1) * vf[bsl, t].unsqueeze(-2)
            dq[bsl, t] = torch.einsum("bhde,bhe->bhd", st, dof[bsl, t])
        s_fin = st
        ds = torch.zeros_like(s_init) if ds_fin is None else ds_fin.clone()
        run_sum = torch.zeros(ds.shape[0], h, dtype=acc)
        if ds_fin is not None:
            run_sum = run_sum + (s_fin * ds_fin).sum(-1).sum(-1)
        for t in range(t1 - 1, t0 - 1, -1):
            ds = ds + qf[bsl, t].unsqueeze(-1) * dof[bsl, t].unsqueeze(-2)
            dk[bsl, t] = torch.einsum("bhde,bhe->bhd", ds, vf[bsl, t])
            dv[bsl, t] = torch.einsum("bhde,bhd->bhe", ds, kf[bsl, t])
            run_sum = run_sum + (qf[bsl, t] * dq[bsl, t]).sum(-1) - (kf[bsl, t] * dk[bsl, t]).sum(-1)
            dld[bsl, t] = run_sum
            lam = torch.exp(ldf[bsl, t]).unsqueeze(-1).unsqueeze(-1)
            ds = lam * ds
        return ds

    if docs is None:
        s0 = _init_state(initial_state, b, h, d, e, acc)
        dsf = _f(dfinal_state, acc)
        dinit = run(slice(0, b), 0, n, s0, dsf)
        return dq, dk, dv, dld, dinit
    m = len(docs)
    s0 = _init_state(initial_state, m, h, d, e, acc)
    dsf = _f(dfinal_state, acc)
    dinits = []
    for i, (a0, a1) in enumerate(docs):
        di = run(slice(0, 1), a0, a1, s0[i:i + 1], None if dsf is None else dsf[i:i + 1])
        dinits.append(di[0])
    return dq, dk, dv, dld, torch.stack(dinits, 0)


# --------------------------------------------------------------------------------------
# vector decay
# --------------------------------------------------------------------------------------
def lavd_forward(q, k=None, v=None, ldk=None, ldv=None, initial_state=None, cu_seqlens=None,
                 acc=torch.float32):
    """Forward recurrence (lavd_torch.py:55-97).  k=None => k = 1-exp(ldk) (:55-57),
    v=None => v = 1-exp(ldv) (:61-63).  The reference's lavd_torch ignores cu_seqlens
    (:16, never read); here documents are independent with the state reset at each boundary,
    the semantics lasd_torch gives the same argument (lasd_torch.py:61-103).

    Returns (o, final_state) in `acc` (the reference casts both to q.dtype, :97).
    """
    assert ldk is not None or ldv is not None, "At least one of ldk or ldv must be used"
    b, n, h, d = q.shape
    qf = _f(q, acc)
    ldkf, ldvf = _f(ldk, acc), _f(ldv, acc)
    kf = (1 - torch.exp(ldkf)) if k is None else _f(k, acc)
    vf = (1 - torch.exp(ldvf)) if v is None else _f(v, acc)
    e = vf.shape[-1]
    docs = _doc_ranges(b, n, cu_seqlens)
    o = torch.zeros(b, n, h, e, dtype=acc)

    def run(bsl, t0, t1, st):
        for t in range(t0, t1):
            if ldkf is not None:
                st = torch.exp(ldkf[bsl, t]).unsqueeze(-1) * st
            if ldvf is not None:
                st = st * torch.exp(ldvf[bsl, t]).unsqueeze(-2)
            st = st + kf[bsl, t].unsqueeze(-1) * vf[bsl, t].unsqueeze(-2)
            o[bsl, t] = torch.einsum("bhd,bhde->bhe", qf[bsl, t], st)
        return st

    if docs is None:
        return o, run(slice(0, b), 0, n, _init_state(initial_state, b, h, d, e, acc))
    assert b == 1
    s0 = _init_state(initial_state, len(docs), h, d, e, acc)
    finals = [run(slice(0, 1), a0, a1, s0[i:i + 1])[0] for i, (a0, a1) in enumerate(docs)]
    return o, torch.stack(finals, 0)


def lavd_backward(q, k, v, ldk, ldv, do, initial_state=None, dfinal_state=None, cu_seqlens=None,
                  acc=torch.float32):
    """Gradients of lavd by two explicit scans (lavd_recurrence_triton.py:230-366 for dq,
    :369-520 for dk, dv, dinitial_state), then
      dldk_t = sum_{s>=t} (q_s*dq_s - k_s*dk_s) + sum_e s_N*dfinal      (:651-675)
      dldv_t = sum_{s>=t} (o_s*do_s - v_s*dv_s) + sum_d s_N*dfinal      (:677-699)
    and, when k (v) is shared with the decay, dldk += dk * (-exp(ldk))  (:701-709).

    Returns dq, dk, dv, dldk, dldv, dinitial_state in `acc`; dk/dv are still returned in share
    mode (the caller drops them as the reference does).
    """
    b, n, h, d = q.shape
    qf, dof = _f(q, acc), _f(do, acc)
    ldkf, ldvf = _f(ldk, acc), _f(ldv, acc)
    share_k, share_v = k is None, v is None
    kf = (1 - torch.exp(ldkf)) if share_k else _f(k, acc)
    vf = (1 - torch.exp(ldvf)) if share_v else _f(v, acc)
    e = vf.shape[-1]
    docs = _doc_ranges(b, n, cu_seqlens)
    dq = torch.zeros_like(qf)
    dk = torch.zeros_like(kf)
    dv = torch.zeros_like(vf)
    dldk = None if ldkf is None else torch.zeros_like(ldkf)
    dldv = None if ldvf is None else torch.zeros_like(ldvf)

    def decay(st, bsl, t):
        if ldkf is not None:
            st = torch.exp(ldkf[bsl, t]).unsqueeze(-1) * st
        if ldvf is not None:
            st = st * torch.exp(ldvf[bsl, t]).unsqueeze(-2)
        return st

    def run(bsl, t0, t1, s_init, ds_fin):
        st = s_init.clone()
        o_loc = {}
        for t in range(t0, t1):
            st = decay(st, bsl, t) + kf[bsl, t].unsqueeze(-1) * vf[bsl, t].unsqueeze(-2)
            dq[bsl, t] = torch.einsum("bhde,bhe->bhd", st, dof[bsl, t])
            if ldvf is not None:
                o_loc[t] = torch.einsum("bhd,bhde->bhe", qf[bsl, t], st)
        s_fin = st
        ds = torch.zeros_like(s_init) if ds_fin is None else ds_fin.clone()
        nb = ds.shape[0]
        sum_k = torch.zeros(nb, h, d, dtype=acc)
        sum_v = torch.zeros(nb, h, e, dtype=acc)
        if ds_fin is not None:
            sum_k = sum_k + (s_fin * ds_fin).sum(-1)
            sum_v = sum_v + (s_fin * ds_fin).sum(-2)
        for t in range(t1 - 1, t0 - 1, -1):
            ds = ds + qf[bsl, t].unsqueeze(-1) * dof[bsl, t].unsqueeze(-2)
            dk[bsl, t] = torch.einsum("bhde,bhe->bhd", ds, vf[bsl, t])
            dv[bsl, t] = torch.einsum("bhde,bhd->bhe", ds, kf[bsl, t])
            if ldkf is not None:
                sum_k = sum_k + qf[bsl, t] * dq[bsl, t] - kf[bsl, t] * dk[bsl, t]
                dldk[bsl, t] = sum_k
            if ldvf is not None:
                sum_v = sum_v + o_loc[t] * dof[bsl, t] - vf[bsl, t] * dv[bsl, t]
                dldv[bsl, t] = sum_v
            ds = decay(ds, bsl, t)
        return ds

    if docs is None:
        dinit = run(slice(0, b), 0, n, _init_state(initial_state, b, h, d, e, acc),
                    _f(dfinal_state, acc))
    else:
        s0 = _init_state(initial_state, len(docs), h, d, e, acc)
        dsf = _f(dfinal_state, acc)
        dinit = torch.stack([
            run(slice(0, 1), a0, a1, s0[i:i + 1], None if dsf is None else dsf[i:i + 1])[0]
            for i, (a0, a1) in enumerate(docs)], 0)
    if share_k:
        dldk = dldk + dk * (-torch.exp(ldkf))
    if share_v:
        dldv = dldv + dv * (-torch.exp(ldvf))
    return dq, dk, dv, dldk, dldv, dinit


# --------------------------------------------------------------------------------------
# single-token decode (the recurrences above with N == 1, state carried by the caller)
# --------------------------------------------------------------------------------------
def decode_step_scalar(q, k, v, ld, state, acc=torch.float32):
    """One token per sequence, scalar decay: lasd_recurrence_triton.py:28-113 with N=1.
    q,k (B,1,H,D), v (B,1,H,E), ld (B,1,H) or (H,), state (B,H,D,E) -> (o (B,1,H,E), new state)."""
    return lasd_forward(q, k, v, ld, initial_state=state, acc=acc)


def decode_step_vector(q, k, v, ldk, state, ldv=None, acc=torch.float32):
    """One token per sequence, vector decay: lavd_recurrence_triton.py:28-154 with N=1."""
    return lavd_forward(q, k, v, ldk, ldv, initial_state=state, acc=acc)


def rel_l2(ref: torch.Tensor, x: torch.Tensor) -> float:
    """Relative L2 error, the acceptance metric (xopes/utils/test_utils.py:8-11)."""
    ref = ref.detach().double().cpu()
    x = x.detach().double().cpu()
    return float((ref - x).norm() / (ref.norm() + 1e-8))
