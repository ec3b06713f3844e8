"""Sequence-parallel scalar-decay forward for one long packed (varlen) stream.

The reference has no distributed code; what is fixed by it is the single-device math of
lasd_torch's varlen branch (xopes/ops/lightning_attn/scalar_decay/lasd_torch.py:61-103): documents
are independent recurrences, the state restarts at every boundary.  Here the token stream is cut
into contiguous ranges, one per rank, and a document that crosses a cut is stitched together:

  phase 1 (local)    every rank runs the ordinary varlen forward on its tokens with a zero
                     incoming state -> local o, per-document end states;
  phase 2 (exchange) every rank publishes (S_loc, G, open_end, spans): the end state of its last
                     local document, the summed log decay over that document's local part, and
                     whether the document continues on the next rank / covers the whole rank.
                     One all-gather (NCCL) moves them; each rank folds the ranks before it:
                         S_in(r+1) = open_end(r) * ( S_loc(r) + spans(r) * exp(G(r)) * S_in(r) )
  phase 3 (local)    a rank whose first document began earlier adds the missing term
                         o_t += exp(cum_t) q_t^T S_in        (la_seqpar_correct)
                     to that document's local tokens and exp(G_first) S_in to its end state.

On CUDA with the all-gather exchange the forward runs in another order (forward_exchange_first):
a state-only pass over k and v yields S_loc first, the exchange follows at once, and the chunk
pass then starts from true states, so phase 3 disappears.

The backward mirrors it in the other direction (lasd_seqpar_backward): every rank runs the local
backward with the forward state S_in it received and a zero incoming state gradient, publishes the
state gradient leaving its FIRST document towards the previous rank (d initial_state of that
document, R_loc), the ranks fold from the right,
                         dS_out(r-1) = open_start(r) * ( R_loc(r) + spans(r) * exp(G(r)) * dS_out(r) )
and a rank whose last document continues adds to that document's local tokens
                         dk_t += exp(rs_t) v_t dS_out^T ,  dv_t += exp(rs_t) k_t dS_out
(rs_t = log decay from token t, exclusive, to the rank's end) with the same correction kernel.
dq needs no correction.  The single-device math is the reference's reverse recurrence
(scalar_decay/lasd_recurrence_triton.py:279-400).

The three phases are separate functions so that tests can run them with any transport (gloo ranks
on CPU, or several emulated ranks in one process); lasd_seqpar_forward composes them over
torch.distributed.
"""
from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch

from .. import _lib


@dataclass
class ShardPlan:
    start: int                 # first global token of this rank
    end: int                   # one past the last
    local_cu: List[int]        # document boundaries relative to `start` (first 0, last end-start)
    doc_ids: List[int]         # global index of every local document
    open_start: bool           # first local document began on an earlier rank
    open_end: bool             # last local document continues on the next rank
    s_in: Optional[torch.Tensor] = None   # set by the forward: true state entering the rank (H,D,E)


def token_range(n_total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, near-equal split of n_total tokens."""
    per = (n_total + world - 1) // world
    return min(rank * per, n_total), min((rank + 1) * per, n_total)


def shard_documents(cu_seqlens: List[int], start: int, end: int) -> ShardPlan:
    """Intersect the documents [cu[i], cu[i+1]) with the rank's range [start, end)."""
    local_cu, doc_ids = [0], []
    open_start = open_end = False
    for i in range(len(cu_seqlens) - 1):
        a, b = cu_seqlens[i], cu_seqlens[i + 1]
        lo, hi = max(a, start), min(b, end)
        if lo >= hi:
            continue
        if not doc_ids and a < start:
            open_start = True
        doc_ids.append(i)
        local_cu.append(hi - start)
        open_end = b > end
    return ShardPlan(start, end, local_cu, doc_ids, open_start, open_end)


def _ld_local(ld: torch.Tensor, t: int, h: int) -> torch.Tensor:
    """Per-token log decay of the local range as a (T, H) fp32 view (expanded, not copied)."""
    if ld.dim() == 1:
        return ld.float().view(1, h).expand(t, h)
    return ld.float().reshape(t, h)


def _cuda_local_forward(q, k, v, ld, local_cu):
    from . import segmented as sg
    from .scalar_decay import _prep_ld, lasd_fn
    _, t, h, d = q.shape
    e = v.shape[-1]
    bounds = [(local_cu[i], local_cu[i + 1]) for i in range(len(local_cu) - 1)]
    sms = sg.num_sms(q.device) if q.is_cuda else 148
    cap = sg.auto_cap(t, h, sms)
    lib = _lib.load()
    if (q.is_cuda and d == 128 and e == 128 and lib.la_lasd_path(t, d, e, _lib.dtype_code(q), 0) == 1
            and sg.worth_segmenting(bounds, h, cap, sms)):
        # few long documents on this rank: cut them further so that every SM has a segment
        ld32, strides = _prep_ld(ld, 1, t, h)
        with torch.no_grad():
            return sg.lasd_forward_segmented(q.contiguous(), k.contiguous(), v.contiguous(), ld32, strides,
                                             None, bounds, cap)[:2]
    cu = torch.tensor(local_cu, dtype=torch.int64, device=q.device)
    with torch.no_grad():
        return lasd_fn(q, k, v, ld, cu_seqlens=cu)


def _cuda_correct(q, o, cum, s_in, t1):
    lib = _lib.load()
    _lib.require_cuda(q, o, cum, s_in)
    _, n, h, d = q.shape
    e = o.shape[-1]
    cum = cum.contiguous()
    s_in = s_in.contiguous()
    with torch.cuda.device(q.device):
        rc = lib.la_seqpar_correct(_lib.ptr(q), _lib.ptr(o), _lib.ptr(cum), _lib.ptr(s_in), t1, n, h, d, e,
                                   _lib.dtype_code(q), _lib.stream_of(q))
    _lib.check(rc, "la_seqpar_correct")


def local_phase(q, k, v, ld, plan: ShardPlan, local_forward: Optional[Callable] = None):
    """Phase 1.  Returns (o, states, summary) where summary is the flat fp32 tensor a rank
    publishes: [S_loc (H*D*E), G (H), open_end, spans]."""
    fwd = local_forward or _cuda_local_forward
    _, t, h, d = q.shape
    o, states = fwd(q, k, v, ld, plan.local_cu)
    e = o.shape[-1]
    dev = q.device
    if not plan.open_end:
        return o, states, torch.zeros(h * d * e + h + 2, dtype=torch.float32, device=dev)
    last0 = plan.local_cu[-2]
    if ld.dim() == 1:
        g = ld.float() * float(t - last0)
    else:
        g = _ld_local(ld, t, h)[last0:].sum(0)
    spans = 1.0 if (plan.open_start and len(plan.doc_ids) == 1) else 0.0
    flags = torch.tensor([1.0, spans], dtype=torch.float32).to(dev, non_blocking=True)
    summary = torch.cat([states[-1].reshape(-1), g, flags])
    return o, states, summary


def fold_incoming_state(gathered: torch.Tensor, rank: int, h: int, d: int, e: int) -> torch.Tensor:
    """Phase 2, after the all-gather: the true state entering `rank`, from the summaries of the
    ranks before it (gathered is (world, H*D*E + H + 2)).  No host synchronisation."""
    if gathered.is_cuda:  # one kernel instead of half a dozen small ones per preceding rank
        lib = _lib.load()
        g = gathered.contiguous()
        s_in = torch.empty(h, d, e, dtype=torch.float32, device=g.device)
        with torch.cuda.device(g.device):
            rc = lib.la_seqpar_fold(_lib.ptr(g), _lib.ptr(s_in), rank, h, d, e, _lib.stream_of(g))
        _lib.check(rc, "la_seqpar_fold")
        return s_in
    s_in = torch.zeros(h, d, e, dtype=torch.float32, device=gathered.device)
    for r in range(rank):
        row = gathered[r]
        s_loc = row[: h * d * e].view(h, d, e)
        g = row[h * d * e: h * d * e + h]
        open_end, spans = row[-2], row[-1]
        s_in = open_end * (s_loc + spans * torch.exp(g).view(h, 1, 1) * s_in)
    return s_in


def correct_phase(q, o, states, ld, s_in, plan: ShardPlan, correct: Optional[Callable] = None):
    """Phase 3, in place on o and states."""
    if not plan.open_start:
        return
    fix = correct or _cuda_correct
    _, t, h, _ = q.shape
    t1 = plan.local_cu[1]
    if ld.dim() == 1:
        # constant per-head decay: closed form, no scan
        steps = torch.arange(1, t1 + 1, dtype=torch.float32, device=q.device)
        cum = steps.view(t1, 1) * ld.float().view(1, h)
    else:
        # scan along the contiguous axis of a (H, T1) copy: torch's outer-dimension scan walks one
        # column per thread and takes milliseconds for a few thousand tokens
        cum = torch.cumsum(_ld_local(ld, t, h)[:t1].t().contiguous(), dim=1).t().contiguous()
    fix(q, o, cum, s_in, t1)
    states[0] += torch.exp(cum[t1 - 1]).view(h, 1, 1) * s_in


def lasd_seqpar_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ld: torch.Tensor,
                        cu_seqlens: torch.Tensor, group=None, exchange: str = "all_gather",
                        local_forward: Optional[Callable] = None, correct: Optional[Callable] = None):
    """Forward of lasd over a packed stream sharded by tokens across the ranks of `group`.

    q, k (1, T_r, H, D) and v (1, T_r, H, E) are THIS rank's contiguous token range
    (token_range(N, rank, world)); ld is (H,) or the local (1, T_r, H) slice; cu_seqlens holds the
    GLOBAL document boundaries.  Returns (o_local, states, plan): o for the local tokens, and the
    end state of every local document (for a document that continues on the next rank this is its
    state at the end of this rank).

    exchange = "all_gather": one collective, every rank folds its own prefix (default);
               "chain": rank r receives S_in from r-1 and sends its outgoing state to r+1
               (send/recv, world-1 serial hops).
    """
    import torch.distributed as dist
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    cu = [int(x) for x in cu_seqlens.tolist()]
    n_total = cu[-1]
    start, end = token_range(n_total, rank, world)
    if q.shape[1] != end - start:
        raise ValueError(f"rank {rank} holds {q.shape[1]} tokens, expected {end - start}")
    plan = shard_documents(cu, start, end)
    _, _, h, d = q.shape
    e = v.shape[-1]
    if exchange == "all_gather" and local_forward is None and correct is None and _tensor_path(q, v):
        def gather(summary):
            gathered = torch.empty(world * summary.numel(), dtype=torch.float32, device=summary.device)
            exchange_summaries(gathered, summary, group)
            return gathered.view(world, -1)
        return forward_exchange_first(q, k, v, ld, plan, rank, gather)
    o, states, summary = local_phase(q, k, v, ld, plan, local_forward)
    if exchange == "all_gather":
        gathered = torch.empty(world * summary.numel(), dtype=torch.float32, device=summary.device)
        exchange_summaries(gathered, summary, group)
        s_in = fold_incoming_state(gathered.view(world, -1), rank, h, d, e)
    elif exchange == "chain":
        s_in = torch.zeros(h, d, e, dtype=torch.float32, device=summary.device)
        if rank > 0:
            dist.recv(s_in, src=dist.get_global_rank(group, rank - 1) if group else rank - 1, group=group)
        if rank < world - 1:
            s_out = fold_incoming_state_step(summary, s_in, h, d, e)
            dist.send(s_out, dst=dist.get_global_rank(group, rank + 1) if group else rank + 1, group=group)
    else:
        raise ValueError(f"unknown exchange {exchange!r}")
    correct_phase(q, o, states, ld, s_in, plan, correct)
    plan.s_in = s_in if plan.open_start else None
    return o, states, plan


def _tensor_path(q, v) -> bool:
    """The local tokens can run on the tensor-core chunk kernels with 128-wide heads (what the
    state-only pass supports)."""
    _, t, _, d = q.shape
    e = v.shape[-1]
    return (q.is_cuda and d == 128 and e == 128 and t >= 128
            and _lib.load().la_lasd_path(t, d, e, _lib.dtype_code(q), 0) == 1)


def forward_exchange_first(q, k, v, ld, plan: ShardPlan, rank: int, gather: Callable):
    """The forward with the ranks meeting BEFORE the chunk pass (CUDA, tensor path): a state-only
    pass gives the end state of the rank's last document under a zero incoming state, the summaries
    are exchanged (gather(summary) -> (world, len) tensor of all ranks' summaries), the prefix
    fold gives the true state entering the rank, and the one chunk pass starts every local document
    and segment from true states.  Against the three phases above this drops the correction pass,
    and the ranks wait for each other after ~0.1 ms of local work instead of after the whole local
    forward, so that they differ less when they meet.  Returns what lasd_seqpar_forward returns."""
    from . import segmented as sg
    from .scalar_decay import _prep_ld
    _, t, h, d = q.shape
    e = v.shape[-1]
    dev = q.device
    local_cu = plan.local_cu
    bounds = [(local_cu[i], local_cu[i + 1]) for i in range(len(local_cu) - 1)]
    sms = sg.num_sms(dev)
    cap = sg.auto_cap(t, h, sms)
    if not sg.worth_segmenting(bounds, h, cap, sms):
        cap = 1 << 40  # documents as they are; only the open last one gets a state-only pass
    ld32, strides = _prep_ld(ld, 1, t, h)
    s_in_box = []

    def exchange(s_end):
        if plan.open_end:
            last0 = local_cu[-2]
            g = ld.float() * float(t - last0) if ld.dim() == 1 else _ld_local(ld, t, h)[last0:].sum(0)
            spans = 1.0 if (plan.open_start and len(plan.doc_ids) == 1) else 0.0
            flags = torch.tensor([1.0, spans], dtype=torch.float32).to(dev, non_blocking=True)
            summary = torch.cat([s_end.reshape(-1), g, flags])
        else:
            summary = torch.zeros(h * d * e + h + 2, dtype=torch.float32, device=dev)
        s_in = fold_incoming_state(gather(summary), rank, h, d, e)
        s_in_box.append(s_in)
        return s_in if plan.open_start else None

    with torch.no_grad():
        o, states, _ = sg.lasd_forward_exchange_first(q.contiguous(), k.contiguous(), v.contiguous(), ld32, strides,
                                                      bounds, cap, plan.open_start, plan.open_end, exchange)
    plan.s_in = s_in_box[0] if plan.open_start else None
    return o, states, plan


def fold_incoming_state_step(row: torch.Tensor, s_in: torch.Tensor, h: int, d: int, e: int) -> torch.Tensor:
    """One hop of the fold: the state leaving a rank, given its summary row and its own S_in."""
    s_loc = row[: h * d * e].view(h, d, e)
    g = row[h * d * e: h * d * e + h]
    return (row[-2] * (s_loc + row[-1] * torch.exp(g).view(h, 1, 1) * s_in)).contiguous()


# --------------------------------------------------------------------------------------------
# backward
# --------------------------------------------------------------------------------------------
def _cuda_local_backward(q, k, v, ld, do, local_cu, s0):
    """Local backward over the rank's documents (cut further into segments when they are few and
    long): returns dq, dk, dv and d initial_state per local document."""
    from . import segmented as sg
    from .scalar_decay import _prep_ld
    _, t, h, d = q.shape
    bounds = [(local_cu[i], local_cu[i + 1]) for i in range(len(local_cu) - 1)]
    sms = sg.num_sms(q.device)
    cap = sg.auto_cap(t, h, sms)
    e = v.shape[-1]
    tensor = d == 128 and e == 128 and _lib.load().la_lasd_path(t, d, e, _lib.dtype_code(q), 0) == 1
    if not (tensor and sg.worth_segmenting(bounds, h, cap, sms)):
        cap = 1 << 40  # documents as they are
    ld32, strides = _prep_ld(ld, 1, t, h)
    with torch.no_grad():
        dq, dk, dv, _, ds0 = sg.lasd_backward_segmented(q.contiguous(), k.contiguous(), v.contiguous(), ld32,
                                                        strides, s0, do.contiguous(), None, bounds, cap,
                                                        want_dld=False, want_ds0=True)
    return dq, dk, dv, ds0


def local_backward_phase(q, k, v, ld, do, plan: ShardPlan, s_in, local_backward: Optional[Callable] = None):
    """Phase 1 of the backward.  Returns (dq, dk, dv, ds0, summary); summary is the flat fp32 tensor
    a rank publishes towards the ranks before it: [R_loc (H*D*E), G (H), open_start, spans]."""
    bwd = local_backward or _cuda_local_backward
    _, t, h, d = q.shape
    e = v.shape[-1]
    dev = q.device
    ndocs = len(plan.doc_ids)
    s0 = None
    if plan.open_start and s_in is not None:
        s0 = torch.zeros(ndocs, h, d, e, dtype=torch.float32, device=dev)
        s0[0] = s_in
    dq, dk, dv, ds0 = bwd(q, k, v, ld, do, plan.local_cu, s0)
    if not plan.open_start:
        return dq, dk, dv, ds0, torch.zeros(h * d * e + h + 2, dtype=torch.float32, device=dev)
    t1 = plan.local_cu[1]
    g = ld.float() * float(t1) if ld.dim() == 1 else _ld_local(ld, t, h)[:t1].sum(0)
    spans = 1.0 if (plan.open_end and ndocs == 1) else 0.0
    flags = torch.tensor([1.0, spans], dtype=torch.float32).to(dev, non_blocking=True)
    return dq, dk, dv, ds0, torch.cat([ds0[0].reshape(-1), g, flags])


def fold_outgoing_gradient(gathered: torch.Tensor, rank: int, h: int, d: int, e: int) -> torch.Tensor:
    """The state gradient entering `rank` from the right (for its last, continuing document), from
    the summaries of the ranks after it: gathered is (world, H*D*E + H + 2)."""
    world = gathered.shape[0]
    s = torch.zeros(h, d, e, dtype=torch.float32, device=gathered.device)
    for r in range(world - 1, rank, -1):
        row = gathered[r]
        r_loc = row[: h * d * e].view(h, d, e)
        g = row[h * d * e: h * d * e + h]
        s = row[-2] * (r_loc + row[-1] * torch.exp(g).view(h, 1, 1) * s)
    return s


def correct_backward_phase(k, v, dk, dv, ld, ds_out, plan: ShardPlan, correct: Optional[Callable] = None):
    """Phase 3 of the backward, in place on dk and dv: the terms of the last local document that
    come from the state gradient entering at the rank's end."""
    if not plan.open_end:
        return
    fix = correct or _cuda_correct
    _, t, h, _ = k.shape
    last0 = plan.local_cu[-2]
    n = t - last0
    if ld.dim() == 1:
        steps = torch.arange(n - 1, -1, -1, dtype=torch.float32, device=k.device)   # tokens after t
        rs = steps.view(n, 1) * ld.float().view(1, h)
    else:
        lt = _ld_local(ld, t, h)[last0:]
        rs = (torch.flip(torch.cumsum(torch.flip(lt, [0]).t().contiguous(), dim=1), [1]).t() - lt).contiguous()
    fix(v[:, last0:], dk[:, last0:], rs, ds_out.transpose(1, 2).contiguous(), n)
    fix(k[:, last0:], dv[:, last0:], rs, ds_out.contiguous(), n)


def lasd_seqpar_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ld: torch.Tensor, do: torch.Tensor,
                         cu_seqlens: torch.Tensor, s_in: Optional[torch.Tensor], group=None,
                         local_backward: Optional[Callable] = None, correct: Optional[Callable] = None):
    """Backward of lasd_seqpar_forward for q, k, v: this rank's token range of each tensor and of
    the upstream gradient do; s_in is the state that entered the rank in the forward
    (plan.s_in of lasd_seqpar_forward; None if the rank starts on a document boundary).  One
    all-gather of the ranks' outgoing state gradients, folded from the right.  Returns
    (dq, dk, dv) for the local tokens.  Gradients of ld and of per-document initial states are not
    produced here."""
    import torch.distributed as dist
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    cu = [int(x) for x in cu_seqlens.tolist()]
    start, end = token_range(cu[-1], rank, world)
    if q.shape[1] != end - start:
        raise ValueError(f"rank {rank} holds {q.shape[1]} tokens, expected {end - start}")
    plan = shard_documents(cu, start, end)
    _, _, h, d = q.shape
    e = v.shape[-1]
    dq, dk, dv, _, summary = local_backward_phase(q, k, v, ld, do, plan, s_in, local_backward)
    gathered = torch.empty(world * summary.numel(), dtype=torch.float32, device=summary.device)
    exchange_summaries(gathered, summary, group)
    ds_out = fold_outgoing_gradient(gathered.view(world, -1), rank, h, d, e)
    correct_backward_phase(k, v, dk, dv, ld, ds_out, plan, correct)
    return dq, dk, dv


class SeqParExchangeError(RuntimeError):
    """The exchange of chunk-end states between ranks failed or timed out (a rank is missing or
    late beyond the process group's timeout).  Nothing on the device waits for another rank, so the
    caller may drop the step or rebuild the group."""


def exchange_summaries(gathered: torch.Tensor, summary: torch.Tensor, group=None):
    """One all-gather of the ranks' summaries.  The collective is ordered on the host (NCCL stream
    order / gloo), so a missing rank shows up here as the process group's timeout or a broken
    connection, which is turned into SeqParExchangeError instead of propagating a backend error."""
    import torch.distributed as dist
    try:
        dist.all_gather_into_tensor(gathered, summary, group=group)
    except (RuntimeError, ValueError) as exc:  # DistBackendError derives from RuntimeError
        raise SeqParExchangeError(f"state exchange failed: {exc}") from exc
