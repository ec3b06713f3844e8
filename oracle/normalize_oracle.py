"""CPU restatement of the reference's normalize op for the gate branch (TEST INFRASTRUCTURE: only
tests/ may import this).  Follows xopes/ops/normalize/normalize/normalize_torch.py:44-111 with the
activations of xopes/ops/act/_act_torch/act_torch.py:5-50, in float64.  Pinned by
tests/golden/normgate.npz (outputs and autograd gradients of the reference function itself, written
by tests/golden/make_golden.py)."""
import torch


def _act(g, act):
    if act == "relu":
        return torch.relu(g)
    if act == "sigmoid":
        return torch.sigmoid(g)
    if act == "silu":
        return g * torch.sigmoid(g)
    if act == "none":
        return g
    raise AssertionError(f"act {act} not supported")


def normalize_gate(x, weight=None, bias=None, gate=None, gate_act="sigmoid", gate_pos="pre", c=1.0, eps=1e-6,
                   use_mean=False, num_groups=1):
    """Forward, differentiable (use torch.autograd for the gradients); returns float64."""
    z = x.double()
    a = None
    if gate is not None:
        a = _act(gate.double(), gate_act)
        if gate_pos == "pre":
            z = z * a
    zg = z.reshape(*z.shape[:-1], num_groups, z.shape[-1] // num_groups)
    if use_mean:
        zg = zg - zg.mean(-1, keepdim=True)
    y = c * zg / torch.sqrt((zg * zg).sum(-1, keepdim=True) + eps)
    y = y.reshape(z.shape)
    if weight is not None:
        y = y * weight.double()
    if bias is not None:
        y = y + bias.double()
    if gate is not None and gate_pos == "post":
        y = y * a
    return y
