"""Lightning attention with a per-head constant decay (lacd), served by the lasd kernels.

Mirror of xopes/ops/lightning_attn/constant_decay/__init__.py:11-53.  A constant decay is the
scalar-decay operator with ld[b, n, h] = ld[h] (constant_decay/lacd_torch.py:40-59), so the (H,)
vector goes to the lasd entry points with strides (0, 0, 1) and is never expanded in memory;
ld=None means no decay (lacd_torch.py:44-45).  The gradient of a learnable (H,) decay is the lasd
gradient summed over batch and sequence (constant_decay/lacd_parallel_triton.py:726-735).
"""
from typing import Optional, Tuple

import torch

from .scalar_decay import lasd_fn


def lacd_fn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ld: Optional[torch.Tensor] = None,
            initial_state: Optional[torch.Tensor] = None,
            cu_seqlens: Optional[torch.LongTensor] = None, save_states: bool = True,
            use_chunk_loop: bool = False, **kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
    if kwargs.get("decay_activation") is not None:
        raise ValueError("decay_activation applies to data-dependent decays (scalar, vector), not to a constant one")
    h = q.shape[2]
    if ld is None:
        ld = torch.zeros(h, dtype=torch.float32, device=q.device)
    elif ld.dim() != 1:
        ld = ld.reshape(h)
    return lasd_fn(q=q, k=k, v=v, ld=ld, initial_state=initial_state, cu_seqlens=cu_seqlens,
                   save_states=save_states, use_chunk_loop=use_chunk_loop)


lacd_parallel_triton = lacd_fn
lacd_recurrence_triton = lacd_fn
