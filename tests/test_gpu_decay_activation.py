"""GPU parity of the fused decay producer: with decay_activation="logsigmoid" the decay arguments hold
the pre-activations x of the usual producer ld = logsigmoid(x)
(benchmarks/lightning_attention/benchmark.py:308-317).  Checked against the CPU oracle fed with
logsigmoid(x); the gradient for x is the oracle's log-decay gradient times sigmoid(-x).  Every path
that reads a decay is visited: scan kernels (fp32), tensor-core chunk kernels (16-bit), varlen, the
segmented passes with their state-only pass, a per-head decay vector.

Tolerances: relative L2 <= 1e-5 for fp32, <= 1e-2 for 16-bit inputs."""
import pytest
import torch
import torch.nn.functional as F

from oracle import lightning_attn_oracle as orc
from util import TOL_BF16, TOL_FP32, assert_close

pytestmark = pytest.mark.gpu

DEV = "cuda"


def leaf(t, dtype=None):
    t = t.detach().clone()
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV).requires_grad_()


def _qkv(b, n, h, d, e, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    q = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    k = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    v = cast(torch.randn(b, n, h, e, generator=g))
    do = cast(torch.randn(b, n, h, e, generator=g))
    return g, q, k, v, do


# (shape, dtype, tol, document lengths or None): scan kernels, chunk kernels, varlen chunk kernels,
# and a call long and narrow enough to be cut into segments
LASD_CASES = [
    ((2, 65, 7, 33, 63), torch.float32, TOL_FP32, None),
    ((2, 512, 4, 128, 128), torch.bfloat16, TOL_BF16, None),
    ((2, 384, 2, 64, 96), torch.float16, TOL_BF16, None),
    ((1, 900, 2, 128, 128), torch.bfloat16, TOL_BF16, [300, 0, 472, 128]),
    ((1, 8192, 2, 128, 128), torch.bfloat16, TOL_BF16, None),
]


@pytest.mark.parametrize("shape,dtype,tol,lens", LASD_CASES)
def test_lasd_logsigmoid_producer(shape, dtype, tol, lens):
    import xopes_b200 as xb
    b, n, h, d, e = shape
    g, qf, kf, vf, dof = _qkv(b, n, h, d, e, dtype, 71)
    # pre-activations spanning strong decay (x << 0) to almost none (x >> 0)
    x = 3.0 * torch.randn(b, n, h, generator=g) + 3.0
    nb = len(lens) if lens else b
    s0 = 0.1 * torch.randn(nb, h, d, e, generator=g)
    dsf = torch.randn(nb, h, d, e, generator=g)
    cu = None if lens is None else torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    q, k, v, xc, s0c = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(x), leaf(s0)
    o, sf = xb.lasd_fn(q, k, v, xc, initial_state=s0c, cu_seqlens=None if cu is None else cu.to(DEV),
                       decay_activation="logsigmoid")
    ld = F.logsigmoid(x.double()).float()
    ro, rsf = orc.lasd_forward(qf, kf, vf, ld, s0, cu)
    assert_close("o", ro, o.float(), tol)
    assert_close("final_state", rsf, sf, tol)
    ((o.float() * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    rq, rk, rv, rld, rs0 = orc.lasd_backward(qf, kf, vf, ld, dof, s0, dsf, cu)
    assert_close("dq", rq, q.grad.float(), tol)
    assert_close("dk", rk, k.grad.float(), tol)
    assert_close("dv", rv, v.grad.float(), tol)
    assert_close("dx", (rld.double() * torch.sigmoid(-x.double())).float(), xc.grad, tol)
    assert_close("dinitial_state", rs0, s0c.grad, tol)


def test_lasd_logsigmoid_per_head_vector_and_eager_twin():
    """A per-head (H,) pre-activation: the gradient is summed over batch and tokens after the chain
    rule.  Also: the fused producer and the library fed with F.logsigmoid(x) agree."""
    import xopes_b200 as xb
    b, n, h, d, e = 2, 640, 4, 128, 128
    _, qf, kf, vf, dof = _qkv(b, n, h, d, e, torch.bfloat16, 5)
    x = torch.tensor([4.0, 2.0, 0.5, 6.0])
    q, k, v, xc = leaf(qf, torch.bfloat16), leaf(kf, torch.bfloat16), leaf(vf, torch.bfloat16), leaf(x)
    o, _ = xb.lasd_fn(q, k, v, xc, decay_activation="logsigmoid")
    (o.float() * dof.to(DEV)).sum().backward()
    q2, k2, v2, x2 = leaf(qf, torch.bfloat16), leaf(kf, torch.bfloat16), leaf(vf, torch.bfloat16), leaf(x)
    o2, _ = xb.lasd_fn(q2, k2, v2, F.logsigmoid(x2))
    (o2.float() * dof.to(DEV)).sum().backward()
    assert_close("o", o2.float().cpu(), o.float(), 1e-3)
    assert_close("dq", q2.grad.float().cpu(), q.grad.float(), 1e-3)
    assert_close("dx", x2.grad.cpu(), xc.grad, TOL_BF16)
    ld = F.logsigmoid(x).view(1, 1, h).expand(b, n, h).contiguous()
    *_, rld, _ = orc.lasd_backward(qf, kf, vf, ld, dof, None, None)
    assert_close("dx vs oracle", (rld * torch.sigmoid(-x)).sum(dim=(0, 1)), xc.grad, TOL_BF16)


LAVD_CASES = [
    ((2, 65, 3, 33, 63), torch.float32, TOL_FP32, True),
    ((2, 130, 2, 64, 32), torch.bfloat16, TOL_BF16, True),
    ((1, 515, 2, 128, 128), torch.bfloat16, TOL_BF16, False),
    ((1, 4096, 2, 128, 128), torch.bfloat16, TOL_BF16, False),   # cut into segments
]


@pytest.mark.parametrize("shape,dtype,tol,use_ldv", LAVD_CASES)
def test_lavd_logsigmoid_producer(shape, dtype, tol, use_ldv):
    import xopes_b200 as xb
    b, n, h, d, e = shape
    g, qf, kf, vf, dof = _qkv(b, n, h, d, e, dtype, 72)
    xk = 2.0 * torch.randn(b, n, h, d, generator=g) + 3.0
    xv = 2.0 * torch.randn(b, n, h, e, generator=g) + 3.0 if use_ldv else None
    s0 = 0.1 * torch.randn(b, h, d, e, generator=g)
    dsf = torch.randn(b, h, d, e, generator=g)
    q, k, v, xkc, s0c = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(xk), leaf(s0)
    xvc = leaf(xv) if use_ldv else None
    o, sf = xb.lavd_fn(q, k, v, ldk=xkc, ldv=xvc, initial_state=s0c, decay_activation="logsigmoid")
    ldk = F.logsigmoid(xk.double()).float()
    ldv = F.logsigmoid(xv.double()).float() if use_ldv else None
    ro, rsf = orc.lavd_forward(qf, kf, vf, ldk, ldv, s0)
    assert_close("o", ro, o.float(), tol)
    assert_close("final_state", rsf, sf, tol)
    ((o.float() * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    rq, rk, rv, rlk, rlv, rs0 = orc.lavd_backward(qf, kf, vf, ldk, ldv, dof, s0, dsf)
    assert_close("dq", rq, q.grad.float(), tol)
    assert_close("dk", rk, k.grad.float(), tol)
    assert_close("dv", rv, v.grad.float(), tol)
    assert_close("dxk", (rlk.double() * torch.sigmoid(-xk.double())).float(), xkc.grad, tol)
    if use_ldv:
        assert_close("dxv", (rlv.double() * torch.sigmoid(-xv.double())).float(), xvc.grad, tol)
    assert_close("dinitial_state", rs0, s0c.grad, tol)


def test_decay_activation_argument_checks():
    import xopes_b200 as xb
    q = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16, device=DEV)
    x = torch.zeros(1, 128, 2, device=DEV)
    with pytest.raises(ValueError):
        xb.lasd_fn(q, q, q, x, decay_activation="softplus")
    with pytest.raises(ValueError):   # the share mode needs the log decay itself
        xb.lavd_fn(q, None, q, ldk=torch.zeros(1, 128, 2, 128, device=DEV), decay_activation="logsigmoid")
    with pytest.raises(ValueError):
        xb.lightning_attn_func(q, q, q, ld=torch.zeros(2, device=DEV), decay_type="constant",
                               decay_activation="logsigmoid")


# ------------------------------------------------------------------------------------------------
# decays given in the 16-bit type of q, k, v (benchmarks/lightning_attention/benchmark.py:315-316):
# the kernels read them as they are.  Oracle: the same (exactly representable) values in fp32.
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape,dtype,use_ldv,act,mild", [
    ((2, 130, 2, 64, 32), torch.bfloat16, True, False, True),      # scan kernels, ldk and ldv
    ((2, 130, 2, 64, 32), torch.float16, True, True, True),        # scan kernels, activation fused
    ((1, 515, 2, 128, 128), torch.bfloat16, False, False, True),   # tensor path, ragged last chunk
    ((1, 515, 2, 128, 128), torch.float16, False, True, True),     # tensor path, activation fused
    ((2, 2048, 2, 128, 128), torch.bfloat16, False, False, False), # the benchmark's decay: two reference rows
    ((1, 4096, 2, 128, 128), torch.bfloat16, False, False, True),  # cut into segments (state-only pass)
])
def test_lavd_decays_in_16_bit(shape, dtype, use_ldv, act, mild):
    import xopes_b200 as xb
    b, n, h, d, e = shape
    g, qf, kf, vf, dof = _qkv(b, n, h, d, e, dtype, 73)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    if act:   # pre-activations, rounded to the 16-bit type
        xk = cast(2.0 * torch.randn(b, n, h, d, generator=g) + 4.0)
        xv = cast(2.0 * torch.randn(b, n, h, e, generator=g) + 4.0) if use_ldv else None
        ldk = F.logsigmoid(xk.double()).float()
        ldv = F.logsigmoid(xv.double()).float() if use_ldv else None
    else:
        xk = cast(F.logsigmoid(torch.randn(b, n, h, d, generator=g)) / (16.0 if mild else 1.0))
        xv = cast(F.logsigmoid(torch.randn(b, n, h, e, generator=g) + 1) / 4.0) if use_ldv else None
        ldk, ldv = xk, xv
    s0 = 0.1 * torch.randn(b, h, d, e, generator=g)
    dsf = torch.randn(b, h, d, e, generator=g)
    q, k, v, xkc, s0c = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(xk, dtype), leaf(s0)
    xvc = leaf(xv, dtype) if use_ldv else None
    o, sf = xb.lavd_fn(q, k, v, ldk=xkc, ldv=xvc, initial_state=s0c,
                       decay_activation="logsigmoid" if act else None)
    ro, rsf = orc.lavd_forward(qf, kf, vf, ldk, ldv, s0)
    assert_close("o", ro, o.float(), TOL_BF16)
    assert_close("final_state", rsf, sf, TOL_BF16)
    ((o.float() * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    rq, rk, rv, rlk, rlv, rs0 = orc.lavd_backward(qf, kf, vf, ldk, ldv, dof, s0, dsf)
    assert xkc.grad.dtype == dtype
    assert_close("dq", rq, q.grad.float(), TOL_BF16)
    assert_close("dk", rk, k.grad.float(), TOL_BF16)
    assert_close("dv", rv, v.grad.float(), TOL_BF16)
    chain = (lambda r, x: (r.double() * torch.sigmoid(-x.double())).float()) if act else (lambda r, x: r)
    assert_close("dldk", chain(rlk, xk), xkc.grad.float(), TOL_BF16)
    if use_ldv:
        assert_close("dldv", chain(rlv, xv), xvc.grad.float(), TOL_BF16)
    assert_close("dinitial_state", rs0, s0c.grad, TOL_BF16)


def test_16_bit_decays_are_rejected_for_fp32_inputs_at_the_c_abi():
    from xopes_b200 import _lib
    lib = _lib.load()
    t = torch.zeros(1, 128, 1, 128, device=DEV)
    o, sf = torch.empty_like(t), torch.empty(1, 1, 128, 128, device=DEV)
    rc = lib.la_lavd_fwd(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, None, None, o.data_ptr(),
                         sf.data_ptr(), 1, 128, 1, 128, 128, 0, _lib.LA_F32, _lib.FLAG_LD_16BIT,
                         torch.cuda.current_stream().cuda_stream)
    assert rc == -3  # LA_ERR_UNSUPPORTED
