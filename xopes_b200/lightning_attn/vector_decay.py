"""Lightning attention with per-token, per-dimension vector decay (lavd) on the CUDA library.

Mirror of xopes/ops/lightning_attn/vector_decay/__init__.py:10-64 and of LavdParallelFunction
(vector_decay/lavd_parallel_triton.py:1293-1486) / LavdRecurrenceFunction
(vector_decay/lavd_recurrence_triton.py:716-849): same names, keyword arguments, layout, return
and gradient order.

Differences, all deliberate:
  * final_state is returned in fp32 (the reference casts it to q.dtype,
    vector_decay/lavd_torch.py:97); rounding it to q.dtype reproduces the reference value;
  * cu_seqlens is honoured (documents independent, state reset at each boundary), where
    lavd_torch ignores the argument (vector_decay/lavd_torch.py:16);
  * k=None / v=None ("share" mode: k = 1-exp(ldk), v = 1-exp(ldv), lavd_torch.py:55-63) is
    expanded here with torch elementwise ops, so autograd adds the chain-rule term
    dldk += dk * (-exp(ldk)) of lavd_recurrence_triton.py:701-709 by itself;
  * decay_activation="logsigmoid" (an addition): ldk / ldv then hold the pre-activations x of
    ld = logsigmoid(x), applied inside the kernels, and their gradients come back as d/dx
    (not with k=None / v=None, which need the log decay itself).
"""
from typing import Optional, Tuple

import torch

from .. import _lib
from .scalar_decay import _act_flag, _cu, _prep_state


def _ld32(x):
    if x is None:
        return None
    x = x.detach()
    return (x if x.dtype == torch.float32 else x.float()).contiguous()


def _prep_decays(q, ldk, ldv):
    """The decays as the library reads them, and the flag that says how: contiguous fp32, or - when
    every decay given already has q's 16-bit dtype (as in the reference's benchmark,
    benchmarks/lightning_attention/benchmark.py:315-316) - as they are, read as 16-bit by the
    kernels (no conversion pass, half the decay traffic)."""
    given = [x for x in (ldk, ldv) if x is not None]
    if q.dtype in (torch.bfloat16, torch.float16) and all(x.dtype == q.dtype for x in given):
        lk, lv = (None if x is None else x.detach().contiguous() for x in (ldk, ldv))
        return lk, lv, _lib.FLAG_LD_16BIT
    return _ld32(ldk), _ld32(ldv), 0


def _segmentation(lib, q, lk, lv, cu, b, n, h, d, e, flags):
    """Few long sequences on the tensor path (one decay, D = E = 128): cut every sequence into as many
    segments as keep one CTA per (segment, head) within the SM count, so that the chunk passes fill
    the GPU (xopes_b200/lightning_attn/segmented.py).  Returns (bounds, cap) or None."""
    from . import segmented as sg
    if cu is not None or (lk is None) == (lv is None) or d != 128 or e != 128:
        return None
    if lib.la_lavd_path(n, d, e, _lib.dtype_code(q), int(lk is not None), int(lv is not None), flags) != 1:
        return None
    parts = sg.num_sms(q.device) // max(1, b * h)
    if parts < 2 or n < 2 * 1024:
        return None
    parts = min(parts, n // 1024)
    cap = -(-(-(-n // parts)) // 128) * 128
    return [(i * n, (i + 1) * n) for i in range(b)], cap


class LavdFunction(torch.autograd.Function):
    """forward(q, k, v, ldk, ldv, initial_state, cu_seqlens, flags) -> (o, final_state)."""

    @staticmethod
    def forward(ctx, q, k, v, ldk, ldv, initial_state, cu_seqlens, flags):
        lib = _lib.load()
        _lib.require_cuda(q, k, v, ldk, ldv, initial_state, cu_seqlens)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        b, n, h, d = q.shape
        e = v.shape[-1]
        cu, m = _cu(cu_seqlens, q.device)
        if cu is not None and b != 1:
            raise AssertionError("cu_seqlens is only supported for batch size 1")
        nb = m if cu is not None else b
        lk, lv, f16 = _prep_decays(q, ldk, ldv)
        flags = flags | f16
        s0 = None if initial_state is None else initial_state.detach().to(torch.float32).contiguous()
        seg = _segmentation(lib, q, lk, lv, cu, b, n, h, d, e, flags)
        if seg is not None:
            from .segmented import lavd_forward_segmented
            bounds, cap = seg
            ld1 = lk if lk is not None else lv   # the one decay given (D = E here)
            o, sf, s_seg = lavd_forward_segmented(q.view(1, b * n, h, d), k.view(1, b * n, h, d),
                                                  v.view(1, b * n, h, e), ld1.view(1, b * n, h, d), s0, bounds, cap,
                                                  flags, value_decay=lk is None)
            # the states entering the segments (64 KB per segment and head) are kept for the backward
            ctx.save_for_backward(q, k, v, ldk, ldv, s0, cu, s_seg)
            ctx.flags = flags
            ctx.seg = seg
            ctx.state_dtype = None if initial_state is None else initial_state.dtype
            ctx.set_materialize_grads(False)
            return o.view(b, n, h, e), sf
        ctx.seg = None
        o = torch.empty(b, n, h, e, dtype=q.dtype, device=q.device)
        sf = torch.empty(nb, h, d, e, dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            rc = lib.la_lavd_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(lk), _lib.ptr(lv),
                                 _lib.ptr(s0), _lib.ptr(cu), _lib.ptr(o), _lib.ptr(sf),
                                 b, n, h, d, e, m, _lib.dtype_code(q), flags, _lib.stream_of(q))
        _lib.check(rc, "la_lavd_fwd")
        ctx.save_for_backward(q, k, v, ldk, ldv, s0, cu, None)
        ctx.flags = flags
        ctx.state_dtype = None if initial_state is None else initial_state.dtype
        ctx.set_materialize_grads(False)
        return o, sf

    @staticmethod
    def backward(ctx, do, dfinal_state):
        lib = _lib.load()
        q, k, v, ldk, ldv, s0, cu, s_seg = ctx.saved_tensors
        b, n, h, d = q.shape
        e = v.shape[-1]
        m = 0 if cu is None else cu.numel() - 1
        nb = m if cu is not None else b
        if do is None:
            do = torch.zeros(b, n, h, e, dtype=q.dtype, device=q.device)
        do = do.contiguous().to(q.dtype)
        dsf = None if dfinal_state is None else dfinal_state.to(torch.float32).contiguous()
        lk, lv, _ = _prep_decays(q, ldk, ldv)
        want_ds0 = s0 is not None and ctx.needs_input_grad[5]
        if ctx.seg is not None:
            from .segmented import lavd_backward_segmented
            bounds, cap = ctx.seg
            ld1 = lk if lk is not None else lv
            dq, dk, dv, dld1, ds0 = lavd_backward_segmented(
                q.view(1, b * n, h, d), k.view(1, b * n, h, d), v.view(1, b * n, h, e), ld1.view(1, b * n, h, d), s0,
                do.view(1, b * n, h, e), dsf, bounds, cap, want_ds0, ctx.flags, s_in=s_seg, value_decay=lk is None)
            if want_ds0:
                ds0 = ds0.to(ctx.state_dtype)
            dld1 = dld1.view(b, n, h, d)
            dldk, dldv = (dld1.to(ldk.dtype), None) if lk is not None else (None, dld1.to(ldv.dtype))
            return (dq.view(b, n, h, d), dk.view(b, n, h, d), dv.view(b, n, h, e), dldk, dldv, ds0, None, None)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dldk = None if ldk is None else torch.empty(b, n, h, d, dtype=torch.float32, device=q.device)
        dldv = None if ldv is None else torch.empty(b, n, h, e, dtype=torch.float32, device=q.device)
        ds0 = torch.empty(nb, h, d, e, dtype=torch.float32, device=q.device) if want_ds0 else None
        ws, ws_bytes = None, 0
        if dsf is not None:
            ws_bytes = lib.la_lavd_bwd_workspace_bytes(b, n, h, d, e, m)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        with torch.cuda.device(q.device):
            rc = lib.la_lavd_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(lk), _lib.ptr(lv),
                                 _lib.ptr(s0), _lib.ptr(do), _lib.ptr(dsf), _lib.ptr(cu),
                                 _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(dldk),
                                 _lib.ptr(dldv), _lib.ptr(ds0), _lib.ptr(ws), ws_bytes,
                                 b, n, h, d, e, m, _lib.dtype_code(q), ctx.flags, _lib.stream_of(q))
        _lib.check(rc, "la_lavd_bwd")
        if dldk is not None:
            dldk = dldk.to(ldk.dtype)
        if dldv is not None:
            dldv = dldv.to(ldv.dtype)
        if want_ds0:
            ds0 = ds0.to(ctx.state_dtype)
        return dq, dk, dv, dldk, dldv, ds0, None, None


def _lavd(q, k, v, ldk, ldv, initial_state, cu_seqlens, flags):
    if ldk is None and ldv is None:
        raise AssertionError("At least one of ldk or ldv must be used")
    if (flags & _lib.FLAG_LD_LOGSIGMOID) and (k is None or v is None):
        raise ValueError("decay_activation needs explicit k and v (the share mode derives them from the log decay)")
    if k is None:
        if ldk is None:
            raise AssertionError("ldk must be provided when k is None")
        k = (1 - torch.exp(ldk.float())).to(q.dtype)
    if v is None:
        if ldv is None:
            raise AssertionError("ldv must be provided when v is None")
        v = (1 - torch.exp(ldv.float())).to(q.dtype)
    b = q.shape[0]
    nb = cu_seqlens.shape[0] - 1 if cu_seqlens is not None else b
    s0 = _prep_state(initial_state, nb, q.shape[2], q.shape[3], v.shape[3])
    d, e = q.shape[3], v.shape[3]
    if _pad_to_tensor_path(q, d, e, ldk, ldv, flags):
        # Narrow heads: the tensor-core kernels work on 128-wide tiles, the scan kernels that would
        # serve these shapes cost ~40x more per token at this size.  Zero features add nothing to any
        # product and a zero log decay leaves them alone, so the operands are padded to 128 features
        # here (one extra pass over each) and the results cut back; autograd carries the gradients
        # through the padding and the slices.
        pd, pe = 128 - d, 128 - e
        fill = 80.0 if (flags & _lib.FLAG_LD_LOGSIGMOID) else 0.0   # logsigmoid(80) = 0 in fp32
        pad = torch.nn.functional.pad
        qp, kp, vp = pad(q, (0, pd)), pad(k, (0, pd)), pad(v, (0, pe))
        lkp = None if ldk is None else pad(ldk, (0, pd), value=fill)
        lvp = None if ldv is None else pad(ldv, (0, pe), value=fill)
        s0p = None if s0 is None else pad(s0, (0, pe, 0, pd))
        o, sf = LavdFunction.apply(qp, kp, vp, lkp, lvp, s0p, cu_seqlens, flags)
        return o[..., :e], sf[..., :d, :e]
    return LavdFunction.apply(q, k, v, ldk, ldv, s0, cu_seqlens, flags)


def _pad_to_tensor_path(q, d, e, ldk, ldv, flags) -> bool:
    """16-bit inputs with head dimensions below 128 (and D * E >= 2048: below that the scan kernels
    are no slower), one decay, at least one chunk of tokens: worth padding to the 128-wide tiles."""
    if (flags & _lib.FLAG_FORCE_RECURRENCE) or q.dtype not in (torch.bfloat16, torch.float16):
        return False
    if (ldk is None) == (ldv is None) or q.shape[1] < 128:
        return False
    return d <= 128 and e <= 128 and (d, e) != (128, 128) and d * e >= 2048


def lavd_parallel_cuda(q: torch.Tensor, k: Optional[torch.Tensor] = None,
                       v: Optional[torch.Tensor] = None, ldk: Optional[torch.Tensor] = None,
                       ldv: Optional[torch.Tensor] = None, use_ldk: bool = True,
                       use_ldv: bool = False, initial_state: Optional[torch.Tensor] = None,
                       cu_seqlens: Optional[torch.LongTensor] = None, save_states: bool = True,
                       save_ld: bool = True, save_a: bool = True, use_chunk_loop: bool = False,
                       decay_activation: Optional[str] = None,
                       **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
    """Signature of lavd_parallel_triton (lavd_parallel_triton.py:1415-1430); use_ldk / use_ldv are
    derived from ldk / ldv being given, as there (:1462-1470)."""
    return _lavd(q, k, v, ldk, ldv, initial_state, cu_seqlens, _act_flag(decay_activation))


def lavd_recurrence_cuda(q: torch.Tensor, k: Optional[torch.Tensor] = None,
                         v: Optional[torch.Tensor] = None, ldk: Optional[torch.Tensor] = None,
                         ldv: Optional[torch.Tensor] = None, use_ldk: bool = True,
                         use_ldv: bool = False, initial_state: Optional[torch.Tensor] = None,
                         cu_seqlens: Optional[torch.LongTensor] = None,
                         decay_activation: Optional[str] = None,
                         **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
    """Signature of lavd_recurrence_triton: always the fp32 scan kernels."""
    return _lavd(q, k, v, ldk, ldv, initial_state, cu_seqlens,
                 _lib.FLAG_FORCE_RECURRENCE | _act_flag(decay_activation))


def lavd_fn(q: torch.Tensor, k: Optional[torch.Tensor] = None, v: Optional[torch.Tensor] = None,
            ldk: Optional[torch.Tensor] = None, ldv: Optional[torch.Tensor] = None,
            initial_state: Optional[torch.Tensor] = None,
            cu_seqlens: Optional[torch.LongTensor] = None, save_states: bool = True,
            save_ld: bool = True, save_a: bool = True, use_chunk_loop: bool = False,
            decay_activation: Optional[str] = None, **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dispatch of vector_decay/__init__.py:44-64."""
    fn = lavd_parallel_cuda if q.shape[1] > 1 else lavd_recurrence_cuda
    return fn(q=q, k=k, v=v, ldk=ldk, ldv=ldv, initial_state=initial_state, cu_seqlens=cu_seqlens,
              save_states=save_states, save_ld=save_ld, save_a=save_a,
              use_chunk_loop=use_chunk_loop, decay_activation=decay_activation)


def lavd_decode_step(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     ldk: Optional[torch.Tensor], state: torch.Tensor,
                     ldv: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                     inplace: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """One decode step with vector decay: q,k (B,1,H,D), v (B,1,H,E), ldk (B,1,H,D) fp32 and/or
    ldv (B,1,H,E) fp32, fp32 state (B,H,D,E).  No autograd; in place by default."""
    lib = _lib.load()
    _lib.require_cuda(q, k, v, ldk, ldv, state)
    b, n, h, d = q.shape
    e = v.shape[-1]
    if n != 1:
        raise ValueError("decode takes exactly one token per sequence")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape) != (b, h, d, e):
        raise ValueError("state must be a contiguous fp32 (B,H,D,E) tensor")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    lk, lv = _ld32(ldk), _ld32(ldv)
    new_state = state if inplace else torch.empty_like(state)
    o = out if out is not None else torch.empty(b, 1, h, e, dtype=q.dtype, device=q.device)
    with torch.cuda.device(q.device):
        rc = lib.la_decode_vector(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(lk), _lib.ptr(lv),
                                  _lib.ptr(state), _lib.ptr(new_state), _lib.ptr(o), b, h, d, e,
                                  _lib.dtype_code(q), _lib.stream_of(q))
    _lib.check(rc, "la_decode_vector")
    return o, new_state


lavd_parallel_triton = lavd_parallel_cuda
lavd_recurrence_triton = lavd_recurrence_cuda
