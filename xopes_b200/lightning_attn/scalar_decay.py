"""Lightning attention with data-dependent scalar decay (lasd) on the CUDA library.

Mirror of xopes/ops/lightning_attn/scalar_decay/__init__.py:10-52 and of the autograd wrappers
LasdParallelFunction (scalar_decay/lasd_parallel_triton.py:757-870) and LasdRecurrenceFunction
(scalar_decay/lasd_recurrence_triton.py:501-596): same names, keyword arguments, B x N x H x D
layout, (o, final_state) return and gradient order.  The `_triton` names of the reference stay as
aliases because its tests and benchmarks import them.

Differences, all deliberate:
  * final_state is returned in fp32 (what lasd_torch returns, scalar_decay/lasd_torch.py:105),
    not in k.dtype;
  * ld may be (B,N,H) or a per-head (H,) vector, as lightning_attn_func's docstring advertises
    (lightning_attn/__init__.py:35);
  * cu_seqlens is honoured by the chunk-parallel path too, with lasd_torch's semantics
    (scalar_decay/lasd_torch.py:61-103);
  * save_states / use_chunk_loop are accepted and ignored: states are never materialised;
  * decay_activation="logsigmoid" (an addition): ld then holds the pre-activations x of the usual
    decay producer ld = logsigmoid(x) (benchmarks/lightning_attention/benchmark.py:308-317), the
    kernels apply the activation where they read the decay and the gradient returned for ld is
    d/dx.  Same result as passing F.logsigmoid(x), without the two elementwise passes.
"""
from typing import Optional, Tuple

import torch

from .. import _lib


def _prep_ld(ld: torch.Tensor, b: int, n: int, h: int):
    ld32 = ld.detach()
    if ld32.dtype != torch.float32:
        ld32 = ld32.float()
    if ld32.dim() == 1:
        if ld32.shape[0] != h:
            raise ValueError(f"ld of shape {tuple(ld.shape)} does not match H={h}")
        return ld32, (0, 0, ld32.stride(0))
    if ld32.dim() == 3 and tuple(ld32.shape) == (b, n, h):
        return ld32, tuple(ld32.stride())
    raise ValueError(f"ld must have shape (B,N,H)=({b},{n},{h}) or (H,), got {tuple(ld.shape)}")


def _prep_state(state: Optional[torch.Tensor], nb: int, h: int, d: int, e: int):
    """(B,H,D,E), (1,H,D,E) or (H,D,E) -> contiguous fp32 (nb,H,D,E)
    (scalar_decay/lasd_parallel_triton.py:855-859)."""
    if state is None:
        return None
    s = state
    if s.dim() == 4 and s.shape[0] == 1 and nb != 1:
        s = s.squeeze(0)
    if s.dim() == 3:
        s = s.unsqueeze(0).expand(nb, h, d, e)
    if tuple(s.shape) != (nb, h, d, e):
        raise ValueError(f"initial_state has shape {tuple(state.shape)}, expected ({nb},{h},{d},{e})")
    return s


def _act_flag(decay_activation: Optional[str]) -> int:
    if decay_activation is None:
        return 0
    if decay_activation != "logsigmoid":
        raise ValueError(f"decay_activation must be None or 'logsigmoid', got {decay_activation!r}")
    return _lib.FLAG_LD_LOGSIGMOID


def _cu(cu_seqlens, device):
    if cu_seqlens is None:
        return None, 0
    cu = cu_seqlens.to(device=device, dtype=torch.int64).contiguous()
    return cu, cu.numel() - 1


def _segmentation(lib, q, ld32, strides, cu, b, n, h, d, e, flags):
    """Decide whether the forward should run segmented (few long sequences on the tensor path,
    xopes_b200/lightning_attn/segmented.py).  Returns (doc bounds, cap, ld over the flattened
    stream, its strides) or None.  Only for calls without cu_seqlens: the bounds must be known on
    the host without a device round trip."""
    from . import segmented as sg
    if cu is not None or (flags & _lib.FLAG_FORCE_RECURRENCE) or d != 128 or e != 128:
        return None
    if lib.la_lasd_path(n, d, e, _lib.dtype_code(q), flags) != 1:
        return None
    sms = sg.num_sms(q.device)
    cap = sg.auto_cap(b * n, h, sms)
    bounds = [(i * n, (i + 1) * n) for i in range(b)]
    if not sg.worth_segmenting(bounds, h, cap, sms):
        return None
    sb, sn, sh = strides
    if sn == 0 and sb == 0:            # per-head constant
        return bounds, cap, ld32, (0, 0, sh)
    if sb == n * sn or b == 1:          # batch and sequence strides collapse into one stream stride
        return bounds, cap, ld32, (0, sn, sh)
    return None


class LasdFunction(torch.autograd.Function):
    """forward(q, k, v, ld, initial_state, cu_seqlens, flags) -> (o, final_state)."""

    @staticmethod
    def forward(ctx, q, k, v, ld, initial_state, cu_seqlens, flags):
        lib = _lib.load()
        _lib.require_cuda(q, k, v, ld, initial_state, cu_seqlens)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        b, n, h, d = q.shape
        e = v.shape[-1]
        cu, m = _cu(cu_seqlens, q.device)
        if cu is not None and b != 1:
            raise AssertionError("cu_seqlens is only supported for batch size 1")
        nb = m if cu is not None else b
        ld32, (sb, sn, sh) = _prep_ld(ld, b, n, h)
        s0 = None
        if initial_state is not None:
            s0 = initial_state.detach().to(torch.float32).contiguous()
        seg = _segmentation(lib, q, ld32, (sb, sn, sh), cu, b, n, h, d, e, flags)
        if seg is not None:
            from .segmented import lasd_forward_segmented
            bounds, cap, ld_flat, strides = seg
            o, sf, s_seg = lasd_forward_segmented(q.view(1, b * n, h, d), k.view(1, b * n, h, d),
                                                  v.view(1, b * n, h, e), ld_flat, strides, s0, bounds, cap,
                                                  flags & _lib.FLAG_LD_LOGSIGMOID)
            o = o.view(b, n, h, e)
            # the states entering the segments (64 KB per segment and head) are kept for the backward
            ctx.save_for_backward(q, k, v, ld, s0, cu, s_seg)
            ctx.flags = flags
            ctx.seg = (bounds, cap, strides)
            ctx.state_dtype = None if initial_state is None else initial_state.dtype
            ctx.set_materialize_grads(False)
            return o, sf
        o = torch.empty(b, n, h, e, dtype=q.dtype, device=q.device)
        sf = torch.empty(nb, h, d, e, dtype=torch.float32, device=q.device)
        with torch.cuda.device(q.device):
            rc = lib.la_lasd_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ld32), sb, sn, sh,
                                 _lib.ptr(s0), _lib.ptr(cu), _lib.ptr(o), _lib.ptr(sf),
                                 b, n, h, d, e, m, _lib.dtype_code(q), flags, _lib.stream_of(q))
        _lib.check(rc, "la_lasd_fwd")
        ctx.save_for_backward(q, k, v, ld, s0, cu, None)
        ctx.flags = flags
        ctx.seg = None
        ctx.state_dtype = None if initial_state is None else initial_state.dtype
        ctx.set_materialize_grads(False)
        return o, sf

    @staticmethod
    def backward(ctx, do, dfinal_state):
        lib = _lib.load()
        q, k, v, ld, s0, cu, s_seg = ctx.saved_tensors
        b, n, h, d = q.shape
        e = v.shape[-1]
        m = 0 if cu is None else cu.numel() - 1
        nb = m if cu is not None else b
        if do is None:
            do = torch.zeros(b, n, h, e, dtype=q.dtype, device=q.device)
        do = do.contiguous().to(q.dtype)
        dsf = None if dfinal_state is None else dfinal_state.to(torch.float32).contiguous()
        ld32, (sb, sn, sh) = _prep_ld(ld, b, n, h)
        want_dld = ctx.needs_input_grad[3]
        want_ds0 = s0 is not None and ctx.needs_input_grad[4]
        if ctx.seg is not None:
            # few long sequences: the same cut into segments as the forward, in both directions
            from .segmented import lasd_backward_segmented
            bounds, cap, strides = ctx.seg
            dq, dk, dv, dld, ds0 = lasd_backward_segmented(
                q.view(1, b * n, h, d), k.view(1, b * n, h, d), v.view(1, b * n, h, e), ld32, strides, s0,
                do.view(1, b * n, h, e), dsf, bounds, cap, want_dld, want_ds0,
                ctx.flags & _lib.FLAG_LD_LOGSIGMOID, s_in=s_seg)
            dq, dk, dv = dq.view(b, n, h, d), dk.view(b, n, h, d), dv.view(b, n, h, e)
            if want_dld:
                dld = dld.view(b, n, h)
                if ld.dim() == 1:
                    dld = dld.sum(dim=(0, 1))
                dld = dld.to(ld.dtype)
            if want_ds0:
                ds0 = ds0.to(ctx.state_dtype)
            return dq, dk, dv, dld, ds0, None, None
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dld = torch.empty(b, n, h, dtype=torch.float32, device=q.device) if want_dld else None
        ds0 = torch.empty(nb, h, d, e, dtype=torch.float32, device=q.device) if want_ds0 else None
        ws, ws_bytes = None, 0
        if want_dld:
            ws_bytes = lib.la_lasd_bwd_workspace_bytes(b, n, h, d, e, m, 1)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
        with torch.cuda.device(q.device):
            rc = lib.la_lasd_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ld32), sb, sn, sh,
                                 _lib.ptr(s0), _lib.ptr(do), _lib.ptr(dsf), _lib.ptr(cu),
                                 _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(dld),
                                 _lib.ptr(ds0), _lib.ptr(ws), ws_bytes, b, n, h, d, e, m,
                                 _lib.dtype_code(q), ctx.flags, _lib.stream_of(q))
        _lib.check(rc, "la_lasd_bwd")
        if want_dld:
            if ld.dim() == 1:
                dld = dld.sum(dim=(0, 1))
            dld = dld.to(ld.dtype)
        if want_ds0:
            ds0 = ds0.to(ctx.state_dtype)
        return dq, dk, dv, dld, ds0, None, None


def _lasd(q, k, v, ld, initial_state, cu_seqlens, flags):
    if ld is None:
        raise ValueError("lasd needs a log-decay tensor ld")
    b = q.shape[0]
    nb = cu_seqlens.shape[0] - 1 if cu_seqlens is not None else b
    s0 = _prep_state(initial_state, nb, q.shape[2], q.shape[3], v.shape[3])
    return LasdFunction.apply(q, k, v, ld, s0, cu_seqlens, flags)


def lasd_parallel_cuda(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                       ld: Optional[torch.Tensor] = None,
                       initial_state: Optional[torch.Tensor] = None,
                       cu_seqlens: Optional[torch.LongTensor] = None, save_states: bool = True,
                       use_chunk_loop: bool = False, decay_activation: Optional[str] = None,
                       **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunk-parallel lasd (signature of lasd_parallel_triton, lasd_parallel_triton.py:824-834).
    Runs the tcgen05 chunk kernels where they apply (16-bit inputs, D = E = 128), the fp32 scan
    kernels otherwise."""
    return _lasd(q, k, v, ld, initial_state, cu_seqlens, _act_flag(decay_activation))


def lasd_recurrence_cuda(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ld: torch.Tensor,
                         initial_state: Optional[torch.Tensor] = None,
                         cu_seqlens: Optional[torch.LongTensor] = None,
                         decay_activation: Optional[str] = None,
                         **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
    """Token-by-token lasd (signature of lasd_recurrence_triton, lasd_recurrence_triton.py:555-563):
    always the fp32 scan kernels."""
    return _lasd(q, k, v, ld, initial_state, cu_seqlens,
                 _lib.FLAG_FORCE_RECURRENCE | _act_flag(decay_activation))


def lasd_fn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ld: Optional[torch.Tensor] = None,
            initial_state: Optional[torch.Tensor] = None,
            cu_seqlens: Optional[torch.LongTensor] = None, save_states: bool = True,
            use_chunk_loop: bool = False, decay_activation: Optional[str] = None,
            **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dispatch of scalar_decay/__init__.py:38-52: chunk-parallel for N > 1, recurrence for N == 1."""
    fn = lasd_parallel_cuda if v.shape[1] > 1 else lasd_recurrence_cuda
    return fn(q=q, k=k, v=v, ld=ld, initial_state=initial_state, cu_seqlens=cu_seqlens,
              save_states=save_states, use_chunk_loop=use_chunk_loop, decay_activation=decay_activation)


def lasd_decode_step(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ld: torch.Tensor,
                     state: torch.Tensor, out: Optional[torch.Tensor] = None,
                     inplace: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """One decode step: q,k (B,1,H,D), v (B,1,H,E), ld (B,1,H) or (H,), fp32 state (B,H,D,E).

    No autograd.  With inplace=True the state tensor is updated where it lies (the reference
    allocates a new state each call, lasd_recurrence_triton.py:132) and returned."""
    lib = _lib.load()
    _lib.require_cuda(q, k, v, ld, state)
    b, n, h, d = q.shape
    e = v.shape[-1]
    if n != 1:
        raise ValueError("decode takes exactly one token per sequence")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape) != (b, h, d, e):
        raise ValueError("state must be a contiguous fp32 (B,H,D,E) tensor")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    ld32, (sb, _, sh) = _prep_ld(ld, b, 1, h)
    new_state = state if inplace else torch.empty_like(state)
    o = out if out is not None else torch.empty(b, 1, h, e, dtype=q.dtype, device=q.device)
    with torch.cuda.device(q.device):
        rc = lib.la_decode_scalar(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(ld32), sb, sh,
                                  _lib.ptr(state), _lib.ptr(new_state), _lib.ptr(o), b, h, d, e,
                                  _lib.dtype_code(q), _lib.stream_of(q))
    _lib.check(rc, "la_decode_scalar")
    return o, new_state


# names the reference's tests and benchmarks import
lasd_parallel_triton = lasd_parallel_cuda
lasd_recurrence_triton = lasd_recurrence_cuda
