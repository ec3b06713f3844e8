"""Host-side mirror of xopes/ops/lightning_attn (the reference's operator interface for this path).

lightning_attn_func has the signature and dispatch of xopes/ops/lightning_attn/__init__.py:12-77.
Decay types outside this library's scope ("positional", "element") raise NotImplementedError;
an unknown string raises ValueError as in the reference (:62).
"""
from typing import Optional, Tuple

import torch

from .constant_decay import lacd_fn
from .seq_parallel import SeqParExchangeError, lasd_seqpar_backward, lasd_seqpar_forward
from .scalar_decay import (lasd_decode_step, lasd_fn, lasd_parallel_cuda, lasd_parallel_triton,
                           lasd_recurrence_cuda, lasd_recurrence_triton)
from .vector_decay import (lavd_decode_step, lavd_fn, lavd_parallel_cuda, lavd_parallel_triton,
                           lavd_recurrence_cuda, lavd_recurrence_triton)


def lightning_attn_func(q: torch.Tensor, k: Optional[torch.Tensor] = None,
                        v: Optional[torch.Tensor] = None, ld: Optional[torch.Tensor] = None,
                        ldk: Optional[torch.Tensor] = None, ldv: Optional[torch.Tensor] = None,
                        initial_state: Optional[torch.Tensor] = None,
                        cu_seqlens: Optional[torch.LongTensor] = None, save_states: bool = True,
                        save_ld: bool = True, save_a: bool = True, use_chunk_loop: bool = False,
                        decay_type: str = "constant", **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
    if decay_type == "constant":
        fn = lacd_fn
    elif decay_type == "vector":
        fn = lavd_fn
    elif decay_type == "scalar":
        fn = lasd_fn
    elif decay_type in ("positional", "element"):
        raise NotImplementedError(f"decay type {decay_type!r} is outside this library's scope")
    else:
        raise ValueError(f"Invalid decay type: {decay_type}")
    return fn(q=q, k=k, v=v, ld=ld, ldk=ldk, ldv=ldv, initial_state=initial_state,
              cu_seqlens=cu_seqlens, save_states=save_states, save_ld=save_ld, save_a=save_a,
              use_chunk_loop=use_chunk_loop, **kwargs)


__all__ = [
    "lightning_attn_func", "lacd_fn", "lasd_fn", "lavd_fn", "lasd_parallel_cuda",
    "lasd_recurrence_cuda", "lavd_parallel_cuda", "lavd_recurrence_cuda", "lasd_parallel_triton",
    "lasd_recurrence_triton", "lavd_parallel_triton", "lavd_recurrence_triton",
    "lasd_decode_step", "lavd_decode_step", "lasd_seqpar_forward", "lasd_seqpar_backward",
    "SeqParExchangeError",
]
