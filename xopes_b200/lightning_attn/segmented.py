"""Segmented scalar-decay passes: sequence parallelism inside one GPU.

The chunk kernel gives one CTA to every (sequence, head) and walks the sequence chunk by chunk, so
a call with few, long sequences (B*H well below the SM count) is bound by that serial walk, and so
is a rank of the sequence-parallel forward whose documents are much longer than a balanced share.
Here long sequences are cut into segments that all run at once, each from its TRUE incoming state:

  1. a state-only pass (la_lasd_state_pass: reads k and v, 512 B per token and head, no output rows)
     gives every segment that something follows its own end state and total log decay;
  2. a fold over the few segments of each sequence (la_lasd_fold_states) turns those into the state
     entering every segment;
  3. the ordinary varlen chunk pass runs with the segments as its "documents" and those states as
     their initial states.

The backward pass does the same in both directions: forward states (k, v) for the dq pass and
reverse states (q, do) for the dk and dv passes; a segment then is to la_lasd_bwd exactly what a
document with an initial state and a final-state gradient is, log-decay gradient included.

This is the associativity the reference's chunk kernels use at chunk granularity with states
materialised in HBM (scalar_decay/lasd_parallel_triton.py:22-253); at segment granularity the
extra traffic is 64 KB per segment and head plus the state-only pass over all but each sequence's
last segment.  16-bit inputs with D = E = 128.
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
        if n == 0:  # an empty document is one empty segment
            seg_cu.append(b)
            first.append(1)
        last_of_doc.append(len(first) - 1)
    return seg_cu, first, last_of_doc


def worth_segmenting(doc_bounds, h: int, cap: int, sms: int) -> bool:
    """Segmenting pays a state-only pass over all but the last segment of every cut sequence
    (512 B per token and head on top of 1,024) and two small launches; only sequences longer than
    `cap` (one balanced share of the launch) are cut.

    * More (sequence, head) pairs than SMs: the plain launch splits the chunk space evenly over the
      CTAs, and a sequence longer than one share then spans three of them - the middle one cannot
      start before the first has finished its part - so any such sequence is cut.
    * Few pairs (a quarter of the SMs or fewer): cut once a sequence is longer than 1.5 shares
      (B = 1, H = 16, N = 32768 forward + backward: 0.56 ms against 1.48 ms).
    * In between the plain launch gives one CTA to each pair and lasts as long as its longest
      sequence.  A CTA needs about 3 us per chunk at any occupancy, but with few pairs the
      backward's launches run side by side on two streams, so idle SMs cost a forward + backward
      step less than their count suggests; the effective cost per chunk and pass below is fitted to
      measured steps on B200 (1.6 us with 32 pairs, 2.2 with 64, 3.3 with 128, 3.7 with every SM
      busy).  Equal-length batches are left alone (48, 96, 128 pairs of N = 8192: cutting loses
      7-27 %); the cut is taken only when the longest sequence makes the plain launch clearly longer
      than the balanced one, as for the ragged documents of a sequence-parallel rank."""
    chunks = [-(-(b - a) // 128) for a, b in doc_bounds]
    longest = max(chunks)
    if longest * 128 <= cap:
        return False
    ctas = len(doc_bounds) * h
    if ctas > sms:
        return True
    if ctas <= sms // 4:
        return longest * 128 > cap + cap // 2
    per_chunk = lambda a: min(3.7, 1.1 + 2.2 * a / 128.0)  # noqa: E731
    plain = longest * per_chunk(ctas)
    cut = 0       # chunks the state-only pass walks: all but the last segment of every cut sequence
    for n in chunks:
        parts = -(-n * 128 // cap)
        cut += n - -(-n // parts)
    total = sum(chunks)
    seg = total * h / sms * per_chunk(sms) * (1.0 + 0.5 * cut / max(total, 1)) + 30.0
    return plain > 1.15 * seg


class _Plan:
    """Host lists and device tables of one segmentation; built once per (documents, cap, device)."""

    def __init__(self, doc_bounds, cap, dev, piece_target, tail=False):
        seg_cu, first, last_of_doc = plan_segments(doc_bounds, cap)
        nseg = len(first)
        last = [0] * nseg
        for i in last_of_doc:
            last[i] = 1
        doc_of, d = [], -1
        for i in range(nseg):
            if first[i]:
                d += 1
            doc_of.append(d)
        # forward flow: every segment that another one follows needs its own end state;
        # reverse flow: every segment that another one precedes needs its own start state.  The
        # state-only pass runs on finer pieces than the segments (there are few segments that need
        # it, and a piece per CTA walks its tokens serially), and the fold runs over the pieces.
        # tail: the forward flow also covers the last segment of the last document, whose end
        # state a sequence-parallel rank publishes before its chunk pass has run.
        self.nseg, self.ndocs = nseg, len(doc_bounds)
        self.cut = nseg > len(doc_bounds)
        i64 = lambda x: torch.tensor(x, dtype=torch.int64).to(dev)  # noqa: E731
        i32 = lambda x: torch.tensor(x, dtype=torch.int32).to(dev)  # noqa: E731
        self.cu_dev = i64(seg_cu)
        self.first_idx = i64([i for i in range(nseg) if first[i]])
        self.last_idx = i64(last_of_doc)
        self.flow = {}
        for reverse in (False, True):
            need = [(not first[s]) if reverse else (not last[s] or (tail and s == nseg - 1)) for s in range(nseg)]
            need_tokens = sum(seg_cu[s + 1] - seg_cu[s] for s in range(nseg) if need[s])
            piece = max(512, -(-need_tokens // max(1, piece_target)) // 128 * 128 + 128) if need_tokens else 512
            ranges, table, emit = [], [], []
            for s in range(nseg):
                a, b = seg_cu[s], seg_cu[s + 1]
                cuts = list(range(a, b, piece)) if (need[s] and b > a) else [a]
                for j, c0 in enumerate(cuts):
                    c1 = min(b, c0 + piece) if need[s] else b
                    is_first = first[s] and j == 0
                    is_last = last[s] and j == len(cuts) - 1
                    row = -1
                    if need[s]:
                        row = len(ranges)
                        ranges.append([c0, c1])
                    table.append([doc_of[s], 1 if is_first else 0, 1 if is_last else 0, row])
                    # the state entering segment s: before its first piece (forward flow), after
                    # its last piece (reverse flow)
                    emit.append(s if (j == (len(cuts) - 1 if reverse else 0)) else -1)
            self.flow[reverse] = dict(n_loc=len(ranges), ranges=i64(ranges or [[0, 0]]), table=i32(table),
                                      emit=i32(emit), nunits=len(table))
            if tail and not reverse:
                # the units of the last document alone, as document 0 of a table of their own
                rows = [[0] + r[1:] for r in table if r[0] == doc_of[nseg - 1]]
                self.tail_table, self.tail_units = i32(rows), len(rows)


_PLANS = {}


def _plan(doc_bounds, cap, dev, h, tail=False) -> _Plan:
    key = (tuple(doc_bounds), cap, dev.type, dev.index, h, tail)
    p = _PLANS.get(key)
    if p is None:
        if len(_PLANS) >= 64:
            _PLANS.clear()
        # about one state-pass piece per SM: one wave fills the GPU, and every piece costs a CTA
        # ramp-up, 64 KB of state and one step of the fold
        p = _PLANS[key] = _Plan(doc_bounds, cap, dev, max(1, num_sms(dev) // max(1, h)), tail)
    return p


def _incoming_states(lib, y, z, ld32, ld_strides, pl: _Plan, ext, reverse: bool, act: int = 0):
    """State entering every segment (forward flow: at its first token from ext = the documents'
    initial states; reverse flow: after its last token from ext = their final-state gradients),
    (nseg, H, 128, 128) fp32."""
    _, t, h, d = y.shape
    e = z.shape[-1]
    dev = y.device
    fl = pl.flow[reverse]
    n_loc = fl["n_loc"]
    _, sn, sh = ld_strides
    stream = _lib.stream_of(y)
    incoming = torch.empty(pl.nseg, h, d, e, dtype=torch.float32, device=dev)
    local = torch.empty(max(n_loc, 1), h, d, e, dtype=torch.float32, device=dev)
    gsum = torch.empty(max(n_loc, 1), h, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        if n_loc:
            rc = lib.la_lasd_state_pass(_lib.ptr(y), _lib.ptr(z), _lib.ptr(ld32), 0, sn, sh, _lib.ptr(fl["ranges"]),
                                        _lib.ptr(local), _lib.ptr(gsum), 1, t, h, d, e, n_loc,
                                        _lib.dtype_code(y), 1 if reverse else 0, 1, act, stream)
            _lib.check(rc, "la_lasd_state_pass")
        rc = lib.la_lasd_fold_states(_lib.ptr(local), _lib.ptr(gsum), _lib.ptr(fl["table"]), _lib.ptr(fl["emit"]),
                                     _lib.ptr(ext), _lib.ptr(incoming), None, fl["nunits"], h, d, e,
                                     1 if reverse else 0, stream)
        _lib.check(rc, "la_lasd_fold_states")
    return incoming


def lasd_forward_segmented(q, k, v, ld32, ld_strides, initial_state, doc_bounds, cap, act: int = 0):
    """q, k, v: (1, T, H, 128) contiguous 16-bit CUDA tensors (a batch flattened to one stream);
    ld32 fp32 with element strides over (stream token, head) = ld_strides[1:]; doc_bounds the
    sequences [(a, b), ...] in stream order; initial_state (ndocs, H, 128, 128) fp32 or None;
    act = FLAG_LD_LOGSIGMOID when ld32 holds pre-activations of a logsigmoid, else 0.
    Returns (o (1,T,H,128), final states (ndocs,H,128,128) fp32, the states entering the segments:
    the backward takes them back as s_in instead of running the state-only pass again)."""
    lib = _lib.load()
    _, t, h, d = q.shape
    e = v.shape[-1]
    dev = q.device
    pl = _plan(doc_bounds, cap, dev, h)
    s_in = _incoming_states(lib, k, v, ld32, ld_strides, pl, initial_state, reverse=False, act=act)
    o = torch.empty(1, t, h, e, dtype=q.dtype, device=dev)
    st = torch.empty(pl.nseg, h, d, e, dtype=torch.float32, device=dev)
    _, sn, sh = ld_strides
    with torch.cuda.device(dev):
        rc = lib.la_lasd_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ld32), 0, sn, sh, _lib.ptr(s_in),
                             _lib.ptr(pl.cu_dev), _lib.ptr(o), _lib.ptr(st), 1, t, h, d, e, pl.nseg,
                             _lib.dtype_code(q), (_lib.FLAG_REQUIRE_TENSOR if pl.cut else 0) | act, _lib.stream_of(q))
        _lib.check(rc, "la_lasd_fwd (segmented)")
    return o, st.index_select(0, pl.last_idx), s_in


def lasd_forward_exchange_first(q, k, v, ld32, ld_strides, doc_bounds, cap, open_start: bool, open_end: bool,
                                exchange):
    """The local forward of a sequence-parallel rank with the exchange BEFORE the chunk pass.

    The state-only pass also covers the end of the last document (when it continues on the next
    rank), a fold over that document's pieces gives its end state under a zero incoming state,
    `exchange(that state or None)` returns the true state entering the rank's first document (or
    None), a second fold seeds every segment from true states, and the one chunk pass then writes
    final outputs: no correction pass afterwards, and the ranks meet after the short state-only
    pass instead of after the long chunk pass.  Arguments as lasd_forward_segmented.
    Returns (o, end states per document, state that entered the rank or None)."""
    lib = _lib.load()
    _, t, h, d = q.shape
    e = v.shape[-1]
    dev = q.device
    pl = _plan(doc_bounds, cap, dev, h, tail=open_end)
    fl = pl.flow[False]
    n_loc = fl["n_loc"]
    _, sn, sh = ld_strides
    stream = _lib.stream_of(q)
    local = torch.empty(max(n_loc, 1), h, d, e, dtype=torch.float32, device=dev)
    gsum = torch.empty(max(n_loc, 1), h, dtype=torch.float32, device=dev)
    s_end = None
    with torch.cuda.device(dev):
        if n_loc:
            rc = lib.la_lasd_state_pass(_lib.ptr(k), _lib.ptr(v), _lib.ptr(ld32), 0, sn, sh, _lib.ptr(fl["ranges"]),
                                        _lib.ptr(local), _lib.ptr(gsum), 1, t, h, d, e, n_loc,
                                        _lib.dtype_code(k), 0, 1, 0, stream)
            _lib.check(rc, "la_lasd_state_pass")
        if open_end:
            s_end = torch.empty(1, h, d, e, dtype=torch.float32, device=dev)
            rc = lib.la_lasd_fold_states(_lib.ptr(local), _lib.ptr(gsum), _lib.ptr(pl.tail_table), None, None, None,
                                         _lib.ptr(s_end), pl.tail_units, h, d, e, 0, stream)
            _lib.check(rc, "la_lasd_fold_states (tail)")
    s_first = exchange(None if s_end is None else s_end[0])
    ext = None
    if open_start and s_first is not None:
        ext = torch.zeros(pl.ndocs, h, d, e, dtype=torch.float32, device=dev)
        ext[0].copy_(s_first)
    incoming = torch.empty(pl.nseg, h, d, e, dtype=torch.float32, device=dev)
    o = torch.empty(1, t, h, e, dtype=q.dtype, device=dev)
    st = torch.empty(pl.nseg, h, d, e, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.la_lasd_fold_states(_lib.ptr(local), _lib.ptr(gsum), _lib.ptr(fl["table"]), _lib.ptr(fl["emit"]),
                                     _lib.ptr(ext), _lib.ptr(incoming), None, fl["nunits"], h, d, e, 0, stream)
        _lib.check(rc, "la_lasd_fold_states")
        rc = lib.la_lasd_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ld32), 0, sn, sh, _lib.ptr(incoming),
                             _lib.ptr(pl.cu_dev), _lib.ptr(o), _lib.ptr(st), 1, t, h, d, e, pl.nseg,
                             _lib.dtype_code(q), _lib.FLAG_REQUIRE_TENSOR, _lib.stream_of(q))
        _lib.check(rc, "la_lasd_fwd (segmented)")
    return o, st.index_select(0, pl.last_idx), (s_first if open_start else None)


def lasd_backward_segmented(q, k, v, ld32, ld_strides, initial_state, do, dfinal_state, doc_bounds, cap,
                            want_dld: bool, want_ds0: bool, act: int = 0, s_in=None):
    """Backward twin: q, k, v, do (1, T, H, 128); initial_state / dfinal_state (ndocs, H, 128, 128)
    fp32 or None; s_in: the forward's segment-entering states if it kept them.
    Returns (dq, dk, dv, dld (1,T,H) fp32 or None, dinitial_state (ndocs,...) or None)."""
    lib = _lib.load()
    _, t, h, d = q.shape
    e = v.shape[-1]
    dev = q.device
    pl = _plan(doc_bounds, cap, dev, h)
    if s_in is None:
        s_in = _incoming_states(lib, k, v, ld32, ld_strides, pl, initial_state, reverse=False, act=act)
    ds_out = _incoming_states(lib, q, do, ld32, ld_strides, pl, dfinal_state, reverse=True, act=act)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dld = torch.empty(1, t, h, dtype=torch.float32, device=dev) if want_dld else None
    ds0 = torch.empty(pl.nseg, h, d, e, dtype=torch.float32, device=dev) if want_ds0 else None
    ws, ws_bytes = None, 0
    if want_dld:
        ws_bytes = lib.la_lasd_bwd_workspace_bytes(1, t, h, d, e, pl.nseg, 1)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    _, sn, sh = ld_strides
    with torch.cuda.device(dev):
        rc = lib.la_lasd_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ld32), 0, sn, sh, _lib.ptr(s_in),
                             _lib.ptr(do), _lib.ptr(ds_out), _lib.ptr(pl.cu_dev), _lib.ptr(dq), _lib.ptr(dk),
                             _lib.ptr(dv), _lib.ptr(dld), _lib.ptr(ds0), _lib.ptr(ws), ws_bytes, 1, t, h, d, e,
                             pl.nseg, _lib.dtype_code(q), (_lib.FLAG_REQUIRE_TENSOR if pl.cut else 0) | act,
                             _lib.stream_of(q))
        _lib.check(rc, "la_lasd_bwd (segmented)")
    if want_ds0:
        ds0 = ds0.index_select(0, pl.first_idx)
    return dq, dk, dv, dld, ds0


# --------------------------------------------------------------------------------------------
# vector decay (ldk): the same scheme with a per-feature decay on the state's rows
# --------------------------------------------------------------------------------------------
def _incoming_states_vec(lib, y, z, ldk, pl: _Plan, ext, reverse: bool, act: int = 0):
    _, t, h, d = y.shape
    e = z.shape[-1]
    dev = y.device
    fl = pl.flow[reverse]
    n_loc = fl["n_loc"]
    stream = _lib.stream_of(y)
    incoming = torch.empty(pl.nseg, h, d, e, dtype=torch.float32, device=dev)
    local = torch.empty(max(n_loc, 1), h, d, e, dtype=torch.float32, device=dev)
    gsum = torch.empty(max(n_loc, 1), h, d, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        if n_loc:
            rc = lib.la_lavd_state_pass(_lib.ptr(y), _lib.ptr(z), _lib.ptr(ldk), _lib.ptr(fl["ranges"]),
                                        _lib.ptr(local), _lib.ptr(gsum), 1, t, h, d, e, n_loc,
                                        _lib.dtype_code(y), 1 if reverse else 0, 1, act, stream)
            _lib.check(rc, "la_lavd_state_pass")
        rc = lib.la_lavd_fold_states(_lib.ptr(local), _lib.ptr(gsum), _lib.ptr(fl["table"]), _lib.ptr(fl["emit"]),
                                     _lib.ptr(ext), _lib.ptr(incoming), fl["nunits"], h, d, e,
                                     1 if reverse else 0, stream)
        _lib.check(rc, "la_lavd_fold_states")
    return incoming


def _tr(x):
    """(.., D, E) -> contiguous (.., E, D), None passes through."""
    return None if x is None else x.transpose(-1, -2).contiguous()


def _seg_states_vec(lib, q, k, v, do, ld, pl, ext, reverse, act, value_decay):
    """States entering the segments for the vector decay `ld`.  Key decay: the state-only pass runs on
    (k, v) (forward flow) or (q, do) (reverse flow) and decays the features of its first operand.
    Value decay: the decayed features are those of v / do, so the operands are exchanged, the pass
    yields transposed states, and the (small) state tensors are transposed on the way in and out."""
    if not value_decay:
        y, z = (q, do) if reverse else (k, v)
        return _incoming_states_vec(lib, y, z, ld, pl, ext, reverse, act)
    y, z = (do, q) if reverse else (v, k)
    return _tr(_incoming_states_vec(lib, y, z, ld, pl, _tr(ext), reverse, act))


def lavd_forward_segmented(q, k, v, ld, initial_state, doc_bounds, cap, flags, value_decay=False):
    """q, k, v (1, T, H, 128) 16-bit, ld (1, T, H, 128) the one vector decay - ldk, or ldv with
    value_decay=True - fp32 (or 16-bit with FLAG_LD_16BIT), all contiguous; flags as for la_lavd_fwd
    (the decay flags reach the state-only pass too).  Returns (o, final states per document, states
    entering the segments)."""
    lib = _lib.load()
    _, t, h, d = q.shape
    e = v.shape[-1]
    dev = q.device
    pl = _plan(doc_bounds, cap, dev, h)
    act = flags & (_lib.FLAG_LD_LOGSIGMOID | _lib.FLAG_LD_16BIT)
    s_in = _seg_states_vec(lib, q, k, v, None, ld, pl, initial_state, False, act, value_decay)
    o = torch.empty(1, t, h, e, dtype=q.dtype, device=dev)
    st = torch.empty(pl.nseg, h, d, e, dtype=torch.float32, device=dev)
    lk, lv = (None, ld) if value_decay else (ld, None)
    with torch.cuda.device(dev):
        rc = lib.la_lavd_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(lk), _lib.ptr(lv), _lib.ptr(s_in),
                             _lib.ptr(pl.cu_dev), _lib.ptr(o), _lib.ptr(st), 1, t, h, d, e, pl.nseg,
                             _lib.dtype_code(q), flags, _lib.stream_of(q))
        _lib.check(rc, "la_lavd_fwd (segmented)")
    return o, st.index_select(0, pl.last_idx), s_in


def lavd_backward_segmented(q, k, v, ld, initial_state, do, dfinal_state, doc_bounds, cap, want_ds0, flags,
                            s_in=None, value_decay=False):
    """Backward twin (s_in: the forward's segment-entering states if it kept them).
    Returns (dq, dk, dv, gradient of the decay (1,T,H,128) fp32, dinitial_state (ndocs,...) or None)."""
    lib = _lib.load()
    _, t, h, d = q.shape
    e = v.shape[-1]
    dev = q.device
    pl = _plan(doc_bounds, cap, dev, h)
    act = flags & (_lib.FLAG_LD_LOGSIGMOID | _lib.FLAG_LD_16BIT)
    if s_in is None:
        s_in = _seg_states_vec(lib, q, k, v, do, ld, pl, initial_state, False, act, value_decay)
    ds_out = _seg_states_vec(lib, q, k, v, do, ld, pl, dfinal_state, True, act, value_decay)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dld = torch.empty(1, t, h, ld.shape[-1], dtype=torch.float32, device=dev)
    ds0 = torch.empty(pl.nseg, h, d, e, dtype=torch.float32, device=dev) if want_ds0 else None
    ws_bytes = lib.la_lavd_bwd_workspace_bytes(1, t, h, d, e, pl.nseg)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    lk, lv = (None, ld) if value_decay else (ld, None)
    dlk, dlv = (None, dld) if value_decay else (dld, None)
    with torch.cuda.device(dev):
        rc = lib.la_lavd_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(lk), _lib.ptr(lv), _lib.ptr(s_in),
                             _lib.ptr(do), _lib.ptr(ds_out), _lib.ptr(pl.cu_dev), _lib.ptr(dq), _lib.ptr(dk),
                             _lib.ptr(dv), _lib.ptr(dlk), _lib.ptr(dlv), _lib.ptr(ds0), _lib.ptr(ws), ws_bytes,
                             1, t, h, d, e, pl.nseg, _lib.dtype_code(q), flags, _lib.stream_of(q))
        _lib.check(rc, "la_lavd_bwd (segmented)")
    if want_ds0:
        ds0 = ds0.index_select(0, pl.first_idx)
    return dq, dk, dv, dld, ds0
