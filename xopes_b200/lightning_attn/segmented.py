"""Segmented scalar-decay forward: sequence parallelism inside one GPU.

The chunk kernel gives one CTA to every (sequence, head) and walks the sequence chunk by chunk, so
a call with few, long sequences (B*H well below the 148 SMs) is bound by that serial walk.  Here
long sequences are cut into segments that run as independent "documents" with a zero incoming
state, all at once; the segments of a sequence are then stitched exactly as ranks are in the
sequence-parallel forward: the segments' end states are folded front to back
(la_seqpar_fold_segments) and every segment that continues a sequence receives the missing term
o_t += exp(cum_t) q_t^T S_in (la_seqpar_correct_multi).  The price is one more pass over the
corrected tokens (768 B per token and head instead of 1,024), so segments are made no shorter than
needed to occupy the GPU.  Forward only; 16-bit inputs with D = E = 128.
"""
from typing import List, Optional, Tuple

import torch

from .. import _lib

_SMS = {}


def num_sms(device=None) -> int:
    """SM count of the device (the same number the library's launch logic queries)."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _SMS:
        _SMS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SMS[idx]


def auto_cap(total_tokens: int, h: int, sms: int) -> int:
    """Segment length (a multiple of the 128-token chunk) that yields about one CTA per SM."""
    segs = max(1, sms // max(1, h))
    cap = -(-total_tokens // segs)
    return max(1024, -(-cap // 128) * 128)


def plan_segments(doc_bounds: List[Tuple[int, int]], cap: int):
    """Cut every document [a, b) into ceil(len / cap) nearly equal segments whose boundaries fall on
    128-token chunk boundaries of the document.  Returns (seg_cu, first, last_of_doc)."""
    seg_cu, first, last_of_doc = [doc_bounds[0][0]], [], []
    for a, b in doc_bounds:
        n = b - a
        parts = max(1, -(-n // cap))
        per = -(-(-(-n // parts)) // 128) * 128
        t = a
        k = 0
        while t < b:
            e = min(b, t + per)
            seg_cu.append(e)
            first.append(1 if k == 0 else 0)
            t = e
            k += 1
        last_of_doc.append(len(first) - 1)
    return seg_cu, first, last_of_doc


def worth_segmenting(doc_bounds, h: int, cap: int, sms: int) -> bool:
    """Segmenting pays an extra pass over the continued segments (768 B per token and head, about
    half of all tokens when every long sequence is cut once) plus a few small launches, so it is
    used only when the plain launch would leave most SMs idle or one sequence would run at least
    three times longer than a balanced share.  Measured on 131072-token shards of 8-10 documents
    and 16 heads: the segment kernel alone 0.39 ms against 0.65-0.70 ms unsegmented, but 0.68-0.76
    ms with the stitching, i.e. no gain at 1.5-2.3 balanced shares."""
    ctas = len(doc_bounds) * h
    longest = max(b - a for a, b in doc_bounds)
    if ctas <= sms // 4:
        return longest > cap + cap // 2
    return ctas < sms and longest >= 3 * cap


class _Plan:
    """Host lists and device tables of one segmentation; built once per (documents, cap, device)."""

    def __init__(self, doc_bounds, cap, dev):
        seg_cu, first, last_of_doc = plan_segments(doc_bounds, cap)
        nseg = len(first)
        lens = [seg_cu[i + 1] - seg_cu[i] for i in range(nseg)]
        cont = [i for i in range(nseg) if not first[i]]
        tiles, tile0 = 0, []
        for i in cont:
            tile0.append(tiles)
            tiles += -(-lens[i] // 128)
        table_all = [[seg_cu[i], lens[i], 0, first[i]] for i in range(nseg)]
        table_cont = [[seg_cu[i], lens[i], tile0[j], 0] for j, i in enumerate(cont)]
        self.nseg, self.ncont, self.tiles = nseg, len(cont), tiles
        self.cu_dev = torch.tensor(seg_cu, dtype=torch.int64).to(dev)
        tab = torch.tensor(table_all + table_cont, dtype=torch.int32).to(dev)
        self.tab_all, self.tab_cont = tab[:nseg], tab[nseg:]
        self.first_idx = torch.tensor([i for i in range(nseg) if first[i]], dtype=torch.int64).to(dev)
        self.cont_idx = torch.tensor(cont, dtype=torch.int64).to(dev)
        self.last_idx = torch.tensor(last_of_doc, dtype=torch.int64).to(dev)
        self.lens_f = torch.tensor(lens, dtype=torch.float32).to(dev).view(nseg, 1)
        self.steps = None  # 1..T as fp32, made on first use by a constant-decay call


_PLANS = {}


def _plan(doc_bounds, cap, dev) -> _Plan:
    key = (tuple(doc_bounds), cap, dev.type, dev.index)
    p = _PLANS.get(key)
    if p is None:
        if len(_PLANS) >= 64:
            _PLANS.clear()
        p = _PLANS[key] = _Plan(doc_bounds, cap, dev)
    return p


def lasd_forward_segmented(q, k, v, ld32, ld_strides, initial_state, doc_bounds, cap):
    """q, k, v: (1, T, H, 128) contiguous 16-bit CUDA tensors (a batch flattened to one stream);
    ld32 fp32 with element strides over (stream token, head) = ld_strides[1:]; doc_bounds the
    sequences [(a, b), ...] in stream order; initial_state (ndocs, H, 128, 128) fp32 or None.
    Returns (o (1,T,H,128), final states (ndocs,H,128,128) fp32)."""
    lib = _lib.load()
    _, t, h, d = q.shape
    e = v.shape[-1]
    dev = q.device
    pl = _plan(doc_bounds, cap, dev)
    nseg = pl.nseg

    s0 = None
    if initial_state is not None:
        s0 = torch.zeros(nseg, h, d, e, dtype=torch.float32, device=dev)
        s0.index_copy_(0, pl.first_idx, initial_state)
    o = torch.empty(1, t, h, e, dtype=q.dtype, device=dev)
    st = torch.empty(nseg, h, d, e, dtype=torch.float32, device=dev)
    _, sn, sh = ld_strides
    stream = _lib.stream_of(q)
    with torch.cuda.device(dev):
        rc = lib.la_lasd_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ld32), 0, sn, sh, _lib.ptr(s0),
                             _lib.ptr(pl.cu_dev), _lib.ptr(o), _lib.ptr(st), 1, t, h, d, e, nseg,
                             _lib.dtype_code(q), _lib.FLAG_REQUIRE_TENSOR, stream)
        _lib.check(rc, "la_lasd_fwd (segmented)")
        # inclusive cumulative log decay of the stream, (T, H), and each segment's total
        if sn == 0:  # constant per head
            if pl.steps is None or pl.steps.numel() != t:
                pl.steps = torch.arange(1, t + 1, dtype=torch.float32, device=dev).view(t, 1)
            ldh = torch.as_strided(ld32, (1, h), (0, sh))
            cum = pl.steps * ldh
            seg_decay = pl.lens_f * ldh
        else:
            ldt = torch.as_strided(ld32, (h, t), (sh, sn))
            cum = torch.cumsum(ldt.contiguous(), dim=1).t().contiguous()
            total = cum.index_select(0, pl.cu_dev[1:] - 1)
            # a segment's decay = cum at its end minus cum just before its start
            starts = pl.cu_dev[:-1]
            before = torch.where((starts > 0).view(-1, 1), cum.index_select(0, (starts - 1).clamp(min=0)),
                                 torch.zeros(1, h, device=dev))
            seg_decay = total - before
        s_in = torch.empty(nseg, h, d, e, dtype=torch.float32, device=dev)
        rc = lib.la_seqpar_fold_segments(_lib.ptr(st), _lib.ptr(seg_decay.contiguous()), _lib.ptr(pl.tab_all),
                                         _lib.ptr(s_in), nseg, h, d, e, stream)
        _lib.check(rc, "la_seqpar_fold_segments")
        if pl.ncont:
            s_in_cont = s_in.index_select(0, pl.cont_idx)
            rc = lib.la_seqpar_correct_multi(_lib.ptr(q), _lib.ptr(o), _lib.ptr(cum), _lib.ptr(s_in_cont),
                                             _lib.ptr(pl.tab_cont), pl.ncont, pl.tiles, t, h, d, e,
                                             _lib.dtype_code(q), stream)
            _lib.check(rc, "la_seqpar_correct_multi")
    final = st.index_select(0, pl.last_idx)
    return o, final
