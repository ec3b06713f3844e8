"""GPU: the fused normalisation + gate kernels (xopes_b200.normalize_gate_fn, through the C ABI)
against the reference's own vectors (tests/golden/normgate.npz) in fp32 and against the CPU
oracle on the shape that follows lightning attention in a block (heads as groups of 128 features)
in bf16."""
import pytest
import torch

from oracle import normalize_oracle as norc
from util import TOL_BF16, TOL_FP32, assert_close, load_golden

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("use_mean", [False, True])
@pytest.mark.parametrize("pos", ["pre", "post"])
@pytest.mark.parametrize("act", ["none", "relu", "sigmoid", "silu"])
def test_normalize_gate_reference_vectors_fp32(act, pos, use_mean):
    from xopes_b200.normalize import normalize_gate_fn
    g = load_golden("normgate")
    groups = int(g["num_groups"])
    e = g["x"].shape[-1] // groups
    x, gate, w, b = (g[n].cuda().requires_grad_() for n in ("x", "gate", "weight", "bias"))
    o = normalize_gate_fn(x, w, b, gate=gate, gate_act=act, gate_pos=pos, c=e ** 0.5, eps=1e-5,
                          use_mean=use_mean, num_groups=groups)
    (o * g["do"].cuda()).sum().backward()
    tag = f"{act}_{pos}_{int(use_mean)}"
    tol = 2e-5  # fast exp / rsqrt in the kernel
    assert_close(tag + ".o", g[tag + ".o"], o, tol)
    assert_close(tag + ".dx", g[tag + ".dx"], x.grad, tol)
    assert_close(tag + ".dgate", g[tag + ".dgate"], gate.grad, tol)
    assert_close(tag + ".dweight", g[tag + ".dweight"], w.grad, tol)
    assert_close(tag + ".dbias", g[tag + ".dbias"], b.grad, tol)


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, TOL_BF16), (torch.float16, TOL_BF16), (torch.float32, 2e-5)])
@pytest.mark.parametrize("shape,groups", [((2, 300, 4 * 128), 4), ((3, 70, 2 * 64), 2), ((1, 50, 512), 1),
                                          ((2, 33, 3 * 200), 3)])
def test_normalize_gate_attention_block_shapes(shape, groups, dtype, tol):
    from xopes_b200.normalize import normalize_gate_fn
    gen = torch.Generator().manual_seed(3)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    x, gate, do = (cast(torch.randn(*shape, generator=gen)) for _ in range(3))
    w = 1 + 0.1 * torch.randn(shape[-1], generator=gen)
    e = shape[-1] // groups
    xc, gc = x.to(dtype).cuda().requires_grad_(), gate.to(dtype).cuda().requires_grad_()
    wc = w.cuda().requires_grad_()
    o = normalize_gate_fn(xc, wc, None, gate=gc, gate_act="sigmoid", gate_pos="pre", c=e ** 0.5, num_groups=groups)
    assert o.dtype == dtype
    (o.float() * do.cuda()).sum().backward()
    xr, gr, wr = (t.clone().requires_grad_() for t in (x, gate, w))
    ro = norc.normalize_gate(xr, wr, None, gr, "sigmoid", "pre", e ** 0.5, 1e-6, False, groups)
    rg = torch.autograd.grad((ro * do.double()).sum(), [xr, gr, wr])
    assert_close("o", ro.float(), o.float(), tol)
    assert_close("dx", rg[0].float(), xc.grad.float(), tol)
    assert_close("dgate", rg[1].float(), gc.grad.float(), tol)
    assert_close("dweight", rg[2].float(), wc.grad, tol)


def test_normalize_without_gate_and_refused_branches():
    from xopes_b200.normalize import normalize_gate_fn
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(5, 40, 256, generator=gen)
    xc = x.cuda().requires_grad_()
    o = normalize_gate_fn(xc, num_groups=2, use_mean=True)
    ro = norc.normalize_gate(x, num_groups=2, use_mean=True)
    assert_close("o", ro.float(), o, 2e-5)
    with pytest.raises(NotImplementedError):
        normalize_gate_fn(xc, residual=xc)
    with pytest.raises(AssertionError):
        normalize_gate_fn(xc, gate=xc, gate_act="softmax")
