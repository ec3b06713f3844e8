"""Chunk-level intermediate oracles of scalar-decay lightning attention (TEST INFRASTRUCTURE: only
tests/ may import this; it is never on the product path).

CPU restatement, in closed form per chunk, of the reference's chunk-level torch fixtures
(xopes/ops/lightning_attn/scalar_decay/torch_utils.py): `lasd_intra_torch` (:10-102, output of every
chunk computed from a zero state), `compute_states` (:105-216, each chunk's own state and the
scanned states between chunks, forward and reverse) and `lasd_inter_torch` (:220-267, what the
state entering a chunk adds to its outputs).  The reference loops over tokens; here each chunk is
one masked product.  Pinned: tests/golden/chunkfx_lasd.npz holds the reference functions'
own outputs (written by tests/golden/make_golden.py) and tests/test_oracle_golden.py checks this
file against them.

Conventions of the reference kept here.  Forward: decay is applied before a token is added, so a
chunk's own state is  sum_j exp(g - c_j) k_j v_j^T  (c inclusive cumulative log decay, g its total).
Reverse (`reverse=True`, the flow of the state gradient): walking a chunk from its last token to
its first, the step from token j+1 to token j applies exp(ld_{j+1}); the first token's own decay
is NOT applied inside a chunk, so a chunk's own reverse state is  sum_j exp(c_j - ld_0) k_j v_j^T,
and a scanned state is listed before the first decay of the chunk it has just left is applied.
"""
import torch


def _chunks(n, block):
    return [(s, min(s + block, n)) for s in range(0, n, block)]


def lasd_chunk_intra(q, k, v, ld, block=128, reverse=False):
    """Output of every chunk from a zero incoming state (lasd_intra_torch, torch_utils.py:10-102)."""
    q, k, v, ld = q.double(), k.double(), v.double(), ld.double()
    out = torch.zeros(*q.shape[:3], v.shape[-1], dtype=torch.double)
    for a, b in _chunks(q.shape[1], block):
        c = torch.cumsum(ld[:, a:b], 1)                                  # (B, m, H)
        if not reverse:
            w = torch.exp(c.unsqueeze(2) - c.unsqueeze(1))               # (B, i, j, H): exp(c_i - c_j)
            mask = torch.tril(torch.ones(b - a, b - a, dtype=torch.bool))
        else:
            w = torch.exp(c.unsqueeze(1) - c.unsqueeze(2))               # exp(c_j - c_i), j >= i
            mask = torch.triu(torch.ones(b - a, b - a, dtype=torch.bool))
        w = torch.where(mask.view(1, b - a, b - a, 1), w, torch.zeros((), dtype=torch.double))
        s = torch.einsum("bihd,bjhd->bijh", q[:, a:b], k[:, a:b]) * w
        out[:, a:b] = torch.einsum("bijh,bjhe->bihe", s, v[:, a:b])
    return out.float()


def lasd_chunk_states(k, v, ld, initial_state=None, block=128, reverse=False):
    """(local_states (B,H,L,D,E), global_states (B,H,L+1,D,E)) as compute_states returns them
    (torch_utils.py:105-216): slot i of global_states is the state entering chunk i in the
    direction of travel, the last slot the state after the whole sequence."""
    k, v, ld = k.double(), v.double(), ld.double()
    bsz, n, h, d = k.shape
    e = v.shape[-1]
    chunks = _chunks(n, block)
    local, total, first = [], [], []
    for a, b in chunks:
        c = torch.cumsum(ld[:, a:b], 1)
        g = c[:, -1]
        wgt = torch.exp(c - ld[:, a:a + 1]) if reverse else torch.exp(g.unsqueeze(1) - c)
        local.append(torch.einsum("bjhd,bjhe->bhde", k[:, a:b] * wgt.unsqueeze(-1), v[:, a:b]))
        total.append(g)
        first.append(ld[:, a])
    state = torch.zeros(bsz, h, d, e, dtype=torch.double) if initial_state is None else initial_state.double()
    dec = lambda x: torch.exp(x).view(bsz, h, 1, 1)  # noqa: E731
    if not reverse:
        glob = [state]
        for i in range(len(chunks)):
            state = dec(total[i]) * state + local[i]
            glob.append(state)
    else:
        # Travelling from the last chunk to the first.  The reference lists, as the state entering
        # chunk i, everything to its right referred to the first token of chunk i+1 WITHOUT that
        # token's own decay (it is applied with the next step, inside chunk i); only the last slot,
        # the state after the whole sequence, carries the decay of token 0.
        ent = [None] * len(chunks)
        nxt_first = torch.zeros_like(first[0])
        for i in range(len(chunks) - 1, -1, -1):
            ent[i] = state
            state = local[i] + dec(total[i] - first[i] + nxt_first) * state
            nxt_first = first[i]
        glob = ent + [dec(first[0]) * state]
    return torch.stack(local, 2).float(), torch.stack(glob, 2).float()


def lasd_chunk_inter(q, k, v, ld, initial_state=None, block=128):
    """What the states entering the chunks add to the outputs (lasd_inter_torch, torch_utils.py:220-267):
    o_inter[i] = exp(c_i) q_i^T S_in(chunk of i)."""
    _, glob = lasd_chunk_states(k, v, ld, initial_state, block, reverse=False)
    q, ld = q.double(), ld.double()
    out = torch.zeros(*q.shape[:3], v.shape[-1], dtype=torch.double)
    for i, (a, b) in enumerate(_chunks(q.shape[1], block)):
        c = torch.cumsum(ld[:, a:b], 1)
        out[:, a:b] = torch.exp(c).unsqueeze(-1) * torch.einsum("bihd,bhde->bihe", q[:, a:b], glob[:, :, i].double())
    return out.float()
