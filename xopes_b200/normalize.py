"""Fused normalisation + gate on the CUDA library: the op that follows lightning attention in a
model block (the reference's "normalize with gate", xopes/ops/normalize/README.md).

normalize_gate_fn mirrors the signature of normalize_torch / normalize_triton
(xopes/ops/normalize/normalize/normalize_torch.py:9-22) for the branch a linear-attention block
uses -- an optional gate, no residual:

    a = act(gate);  z = x * a if gate_pos == "pre" else x;  zc = z - mean(z) if use_mean
    y = c * zc / sqrt(sum(zc^2) + eps) * weight + bias      per group of x.shape[-1] / num_groups features
    o = y * a if gate_pos == "post" else y

One CUDA pass each way instead of an activation, a product, a norm and another product.  The
residual branch of the reference op (which excludes the gate) is outside this library's scope.
"""
from typing import Optional

import torch

from . import _lib

_ACTS = {"none": 0, "relu": 1, "sigmoid": 2, "silu": 3}
_POS = {"pre": 0, "post": 1}


class NormalizeGateFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, gate, act, pos, c, eps, use_mean, num_groups):
        lib = _lib.load()
        _lib.require_cuda(x, weight, bias, gate)
        xc = x.contiguous()
        gc = None if gate is None else gate.contiguous().to(x.dtype)
        d = x.shape[-1]
        e = d // num_groups
        rows = x.numel() // d
        w32 = None if weight is None else weight.detach().float().contiguous()
        b32 = None if bias is None else bias.detach().float().contiguous()
        out = torch.empty_like(xc)
        with torch.cuda.device(x.device):
            rc = lib.la_normalize_gate_fwd(_lib.ptr(xc), _lib.ptr(gc), _lib.ptr(w32), _lib.ptr(b32), _lib.ptr(out),
                                           rows, num_groups, e, _lib.dtype_code(xc), act, pos, c, eps,
                                           1 if use_mean else 0, _lib.stream_of(xc))
        _lib.check(rc, "la_normalize_gate_fwd")
        ctx.save_for_backward(xc, gc, w32, b32)
        ctx.cfg = (act, pos, c, eps, use_mean, num_groups, rows, e)
        ctx.dtypes = (None if weight is None else weight.dtype, None if bias is None else bias.dtype,
                      None if gate is None else gate.dtype)
        return out

    @staticmethod
    def backward(ctx, do):
        lib = _lib.load()
        xc, gc, w32, b32 = ctx.saved_tensors
        act, pos, c, eps, use_mean, num_groups, rows, e = ctx.cfg
        do = do.contiguous().to(xc.dtype)
        dx = torch.empty_like(xc)
        dg = None if gc is None else torch.empty_like(gc)
        dw = None if w32 is None else torch.zeros_like(w32)
        db = None if b32 is None else torch.zeros_like(b32)
        with torch.cuda.device(xc.device):
            rc = lib.la_normalize_gate_bwd(_lib.ptr(xc), _lib.ptr(gc), _lib.ptr(w32), _lib.ptr(b32), _lib.ptr(do),
                                           _lib.ptr(dx), _lib.ptr(dg), _lib.ptr(dw), _lib.ptr(db), rows, num_groups,
                                           e, _lib.dtype_code(xc), act, pos, c, eps, 1 if use_mean else 0,
                                           _lib.stream_of(xc))
        _lib.check(rc, "la_normalize_gate_bwd")
        wd, bd, gd = ctx.dtypes
        return (dx, None if dw is None else dw.to(wd), None if db is None else db.to(bd),
                None if dg is None else dg.to(gd), None, None, None, None, None, None)


def normalize_gate_fn(x: torch.Tensor, weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                      residual: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                      gate_act: str = "sigmoid", gate_pos: str = "pre", c: float = 1.0, eps: float = 1e-6,
                      use_mean: bool = False, num_groups: int = 1, return_residual: bool = False) -> torch.Tensor:
    """Arguments as normalize_torch (normalize_torch.py:9-22).  residual / return_residual raise
    NotImplementedError (the reference excludes them together with a gate, :56-58)."""
    if residual is not None or return_residual:
        raise NotImplementedError("the residual branch of normalize is outside this library's scope")
    if x.shape[-1] % num_groups != 0:
        raise AssertionError("The last dimension of x must be divisible by num_groups")
    if gate_act not in _ACTS:
        raise AssertionError(f"act {gate_act} not supported")
    if gate_pos not in _POS:
        raise ValueError(f"gate_pos must be 'pre' or 'post', got {gate_pos!r}")
    return NormalizeGateFunction.apply(x, weight, bias, gate, _ACTS[gate_act], _POS[gate_pos], float(c), float(eps),
                                       bool(use_mean), int(num_groups))
