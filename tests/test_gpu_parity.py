"""GPU parity: the CUDA path (through the Python mirror of the reference interface, which calls the
C ABI) against the committed reference vectors and against the CPU oracle on seeded inputs.

Tolerances: relative L2 <= 1e-5 for fp32 outputs, <= 1e-2 for 16-bit outputs, gradients and
final states."""
import ctypes

import pytest
import torch

from oracle import lightning_attn_oracle as orc
from util import TOL_BF16, TOL_FP32, assert_close, golden_cases, load_golden

pytestmark = pytest.mark.gpu

DEV = "cuda"

# The log-decay gradient is a reverse cumulative sum over the whole sequence of (q.dq - k.dk), two
# large terms that nearly cancel (the reference forms it the same way,
# log_decay_with_cumsum/dld_with_cumsum_triton.py:20-133).  It keeps the same 1e-2 bound as every
# other 16-bit output: when it is requested the kernels feed the state copy and the rescaled
# state-update operand to the tensor cores as high + low 16-bit halves, so that the inter-chunk parts
# of the two terms cancel (measured: 1e-3 .. 3e-3 from N = 128 to N = 16384).
def dld_tol(dtype, tol):
    return tol


def cuda(g):
    return {k: v.to(DEV) for k, v in g.items()}


def leaf(t, dtype=None):
    t = t.detach().clone()
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV).requires_grad_()


# ------------------------------------------------------------------------------------------------
# golden vectors (outputs of the reference's torch operators), fp32
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("which", ["parallel", "recurrence", "fn"])
@pytest.mark.parametrize("case", golden_cases("lasd_"))
def test_lasd_golden(case, which):
    import xopes_b200 as xb
    fn = {"parallel": xb.lasd_parallel_triton, "recurrence": xb.lasd_recurrence_triton,
          "fn": xb.lasd_fn}[which]
    g = load_golden(case)
    q, k, v, ld = leaf(g["q"]), leaf(g["k"]), leaf(g["v"]), leaf(g["ld"])
    s0 = leaf(g["initial_state"]) if "initial_state" in g else None
    cu = g["cu_seqlens"].to(DEV) if "cu_seqlens" in g else None
    o, sf = fn(q, k, v, ld, initial_state=s0, cu_seqlens=cu)
    assert_close("o", g["o"], o, TOL_FP32)
    assert_close("final_state", g["final_state"], sf, TOL_FP32)
    loss = (o * g["do"].to(DEV)).sum()
    if "dfinal_state" in g:
        loss = loss + (sf * g["dfinal_state"].to(DEV)).sum()
    loss.backward()
    for n, x in (("dq", q), ("dk", k), ("dv", v), ("dld", ld)):
        assert_close(n, g[n], x.grad, TOL_FP32)
    if s0 is not None:
        assert_close("dinitial_state", g["dinitial_state"], s0.grad, TOL_FP32)


@pytest.mark.parametrize("which", ["parallel", "recurrence"])
@pytest.mark.parametrize("case", golden_cases("lavd_"))
def test_lavd_golden(case, which):
    import xopes_b200 as xb
    fn = {"parallel": xb.lavd_parallel_triton, "recurrence": xb.lavd_recurrence_triton}[which]
    g = load_golden(case)
    q, v, ldk = leaf(g["q"]), leaf(g["v"]), leaf(g["ldk"])
    k = leaf(g["k"]) if "k" in g else None
    ldv = leaf(g["ldv"]) if "ldv" in g else None
    s0 = leaf(g["initial_state"]) if "initial_state" in g else None
    cu = g["cu_seqlens"].to(DEV) if "cu_seqlens" in g else None
    o, sf = fn(q, k, v, ldk=ldk, ldv=ldv, initial_state=s0, cu_seqlens=cu)
    assert_close("o", g["o"], o, TOL_FP32)
    assert_close("final_state", g["final_state"], sf, TOL_FP32)
    loss = (o * g["do"].to(DEV)).sum()
    if "dfinal_state" in g:
        loss = loss + (sf * g["dfinal_state"].to(DEV)).sum()
    loss.backward()
    assert_close("dq", g["dq"], q.grad, TOL_FP32)
    assert_close("dv", g["dv"], v.grad, TOL_FP32)
    assert_close("dldk", g["dldk"], ldk.grad, TOL_FP32)
    if k is not None:
        assert_close("dk", g["dk"], k.grad, TOL_FP32)
    if ldv is not None:
        assert_close("dldv", g["dldv"], ldv.grad, TOL_FP32)
    if s0 is not None:
        assert_close("dinitial_state", g["dinitial_state"], s0.grad, TOL_FP32)


# ------------------------------------------------------------------------------------------------
# the reference's own test shapes (tests/lightning_attn/scalar_decay/test.py:13-32), seeded inputs
# ------------------------------------------------------------------------------------------------
def _lasd_seeded(b, n, h, d, e, seed, dtype, use_state, use_dfinal, weak_decay):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, n, h, d, generator=g) * d ** -0.5
    k = torch.randn(b, n, h, d, generator=g) * d ** -0.5
    v = torch.randn(b, n, h, e, generator=g)
    if weak_decay:  # the reference test's decay: logsigmoid((1 + 0.01*randn) * 10)
        ld = torch.nn.functional.logsigmoid((1 + 0.01 * torch.randn(b, n, h, generator=g)) * 10)
    else:
        ld = torch.nn.functional.logsigmoid(torch.randn(b, n, h, generator=g) + 2.0)
    s0 = 0.1 * torch.randn(b, h, d, e, generator=g) if use_state else None
    do = torch.randn(b, n, h, e, generator=g)
    dsf = torch.randn(b, h, d, e, generator=g) if use_dfinal else None
    cast = lambda t: t.to(dtype).float()  # noqa: E731  values exactly representable in dtype
    return cast(q), cast(k), cast(v), ld, s0, cast(do), dsf


def _run_lasd_case(fn, b, n, h, d, e, seed, dtype, use_state, use_dfinal, weak_decay, tol):
    qf, kf, vf, ld, s0, dof, dsf = _lasd_seeded(b, n, h, d, e, seed, dtype, use_state, use_dfinal,
                                                weak_decay)
    q, k, v, ldc = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(ld)
    s0c = leaf(s0) if use_state else None
    o, sf = fn(q, k, v, ldc, initial_state=s0c)
    assert o.dtype == dtype and sf.dtype == torch.float32
    ro, rsf = orc.lasd_forward(qf, kf, vf, ld, s0)
    assert_close("o", ro, o.float(), tol)
    assert_close("final_state", rsf, sf, tol)
    loss = (o.float() * dof.to(DEV)).sum()
    if use_dfinal:
        loss = loss + (sf * dsf.to(DEV)).sum()
    loss.backward()
    rq, rk, rv, rld, rs0 = orc.lasd_backward(qf, kf, vf, ld, dof, s0, dsf)
    assert_close("dq", rq, q.grad.float(), tol)
    assert_close("dk", rk, k.grad.float(), tol)
    assert_close("dv", rv, v.grad.float(), tol)
    assert_close("dld", rld, ldc.grad, dld_tol(dtype, tol))
    if use_state:
        assert_close("dinitial_state", rs0, s0c.grad, tol)


REF_SHAPES = [(2, 256, 8, 128, 64), (2, 257, 8, 64, 32), (2, 65, 7, 33, 63), (2, 270, 8, 64, 32),
              (1, 300, 3, 255, 257), (2, 128, 4, 128, 128)]


@pytest.mark.parametrize("shape", REF_SHAPES)
@pytest.mark.parametrize("use_state,use_dfinal", [(True, True), (False, False)])
def test_lasd_reference_shapes_fp32(shape, use_state, use_dfinal):
    import xopes_b200 as xb
    _run_lasd_case(xb.lasd_parallel_triton, *shape, seed=2024, dtype=torch.float32,
                   use_state=use_state, use_dfinal=use_dfinal, weak_decay=True, tol=TOL_FP32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(2, 300, 4, 128, 128), (1, 128, 2, 128, 128), (2, 200, 3, 64, 64),
                                   (1, 1, 2, 128, 128), (1, 513, 2, 128, 128), (1, 129, 3, 128, 128),
                                   (2, 300, 2, 64, 128), (1, 257, 2, 128, 32), (2, 384, 3, 96, 40),
                                   (1, 700, 2, 8, 16)])
def test_lasd_16bit(shape, dtype):
    import xopes_b200 as xb
    _run_lasd_case(xb.lasd_fn, *shape, seed=7, dtype=dtype, use_state=True, use_dfinal=True,
                   weak_decay=False, tol=TOL_BF16)


def test_lasd_reference_training_shape_bf16():
    """The reference's training shape (tests/lightning_attn/scalar_decay/test.py:13-32:
    (8, 2048, 12, 64, 64)) at a quarter of its batch, in bf16: head dimension 64 on the tensor-core
    path, 24 (sequence, head) pairs."""
    import xopes_b200 as xb
    from xopes_b200 import _lib
    assert xb.load_library().la_lasd_path(2048, 64, 64, _lib.LA_BF16, _lib.FLAG_REQUIRE_TENSOR) == 1
    _run_lasd_case(xb.lasd_fn, 2, 2048, 12, 64, 64, seed=2024, dtype=torch.bfloat16, use_state=True,
                   use_dfinal=True, weak_decay=True, tol=TOL_BF16)


def test_config1_fp32_forward():
    """Benchmark configuration 1 in full: B2 N512 H8 D=E=64 fp32, per-head decay, no initial state."""
    import xopes_b200 as xb
    from xopes_b200 import workloads
    w = workloads.lasd_inputs(2, 512, 8, 64, 64, dtype=torch.float32, seed=0, decay_step=1.0,
                              use_state=False, use_do=False)
    o, sf = xb.lightning_attn_func(w["q"].to(DEV), w["k"].to(DEV), w["v"].to(DEV),
                                   ld=w["ld"].to(DEV), decay_type="scalar")
    ro, rsf = orc.lasd_forward(w["q"], w["k"], w["v"], w["ld"])
    assert_close("o", ro, o, TOL_FP32)
    assert_close("final_state", rsf, sf, TOL_FP32)
    # the default decay type ("constant") takes the same (H,) vector
    o2, sf2 = xb.lightning_attn_func(w["q"].to(DEV), w["k"].to(DEV), w["v"].to(DEV), ld=w["ld"].to(DEV))
    assert torch.equal(o, o2) and torch.equal(sf, sf2)


def test_per_head_decay_gradient_is_summed():
    import xopes_b200 as xb
    b, n, h, d, e = 2, 70, 3, 32, 32
    qf, kf, vf, _, s0, dof, dsf = _lasd_seeded(b, n, h, d, e, 5, torch.float32, True, True, False)
    ld_h = torch.log(1 - 2.0 ** (-3 - torch.arange(h, dtype=torch.float32)))
    q, k, v, ld = leaf(qf), leaf(kf), leaf(vf), leaf(ld_h)
    o, sf = xb.lasd_fn(q, k, v, ld, initial_state=s0.to(DEV))
    ((o * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    full = ld_h.view(1, 1, h).expand(b, n, h)
    _, _, _, rld, _ = orc.lasd_backward(qf, kf, vf, full, dof, s0, dsf)
    assert_close("dld", rld.sum((0, 1)), ld.grad, TOL_FP32)


def test_broadcast_initial_state_and_unused_state_output():
    import xopes_b200 as xb
    b, n, h, d, e = 3, 40, 2, 16, 16
    qf, kf, vf, ld, _, dof, _ = _lasd_seeded(b, n, h, d, e, 9, torch.float32, False, False, False)
    s0 = 0.1 * torch.randn(h, d, e, generator=torch.Generator().manual_seed(1))
    q, k, v, s0c = leaf(qf), leaf(kf), leaf(vf), leaf(s0)
    o, _ = xb.lasd_fn(q, k, v, ld.to(DEV), initial_state=s0c)
    (o * dof.to(DEV)).sum().backward()
    ro, _ = orc.lasd_forward(qf, kf, vf, ld, s0)
    assert_close("o", ro, o, TOL_FP32)
    rq, rk, rv, _, rs0 = orc.lasd_backward(qf, kf, vf, ld, dof, s0.unsqueeze(0).expand(b, h, d, e))
    assert_close("dq", rq, q.grad, TOL_FP32)
    assert_close("dinitial_state", rs0.sum(0), s0c.grad, TOL_FP32)


# ------------------------------------------------------------------------------------------------
# vector decay, seeded
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_FP32), (torch.bfloat16, TOL_BF16)])
@pytest.mark.parametrize("use_ldv", [False, True])
@pytest.mark.parametrize("shape", [(2, 130, 2, 64, 32), (1, 257, 2, 128, 128), (2, 65, 3, 33, 63)])
def test_lavd_seeded(shape, use_ldv, dtype, tol):
    import xopes_b200 as xb
    b, n, h, d, e = shape
    g = torch.Generator().manual_seed(31)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    qf = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    kf = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    vf = cast(torch.randn(b, n, h, e, generator=g))
    ldk = torch.nn.functional.logsigmoid(torch.randn(b, n, h, d, generator=g))
    ldv = torch.nn.functional.logsigmoid(torch.randn(b, n, h, e, generator=g) + 1) if use_ldv else None
    s0 = 0.1 * torch.randn(b, h, d, e, generator=g)
    dof = cast(torch.randn(b, n, h, e, generator=g))
    dsf = torch.randn(b, h, d, e, generator=g)
    q, k, v, lk, s0c = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(ldk), leaf(s0)
    lv = leaf(ldv) if use_ldv else None
    o, sf = xb.lavd_fn(q, k, v, ldk=lk, ldv=lv, initial_state=s0c)
    ro, rsf = orc.lavd_forward(qf, kf, vf, ldk, ldv, s0)
    assert_close("o", ro, o.float(), tol)
    assert_close("final_state", rsf, sf, tol)
    ((o.float() * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    rq, rk, rv, rlk, rlv, rs0 = orc.lavd_backward(qf, kf, vf, ldk, ldv, dof, s0, dsf)
    assert_close("dq", rq, q.grad.float(), tol)
    assert_close("dk", rk, k.grad.float(), tol)
    assert_close("dv", rv, v.grad.float(), tol)
    assert_close("dldk", rlk, lk.grad, tol)
    if use_ldv:
        assert_close("dldv", rlv, lv.grad, tol)
    assert_close("dinitial_state", rs0, s0c.grad, tol)


def _lavd_unsafe_flag(lib):
    import ctypes
    f = ctypes.c_int(-1)
    assert lib.la_debug_lavd_unsafe(torch.cuda.current_stream().cuda_stream, ctypes.byref(f)) == 0
    return f.value


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("regime", ["weak", "medium", "reference_benchmark", "strong"])
@pytest.mark.parametrize("shape,lens", [((2, 384, 2), None), ((1, 300, 3), None), ((1, 128, 1), None),
                                        ((1, 700, 2), [1, 127, 128, 129, 300, 15]), ((1, 2048, 2), None)])
def test_lavd_tensor_path(shape, lens, regime, dtype, lib):
    """Vector decay (ldk only) with D = E = 128 in 16 bit: the tcgen05 chunk kernels.  "weak" is the
    benchmark configuration's decay (logsigmoid(x)/16) and must stay on the one-reference kernels;
    "reference_benchmark" is the decay of the reference's own benchmark script
    (logsigmoid(N(0,1)), benchmarks/lightning_attention/benchmark.py:315), about 2^-74 per half
    chunk: it must be served by the two-reference tensor-core kernels (bf16), not by the scan;
    "strong" decays by far more than 2^-96 per 32 tokens and must fall back to the scan kernels."""
    import xopes_b200 as xb
    from xopes_b200 import _lib
    b, n, h = shape
    d = e = 128
    assert lib.la_lavd_path(n, d, e, _lib.dtype_code(torch.empty(0, dtype=dtype)), 1, 0, 0) == 1
    g = torch.Generator().manual_seed(17)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    x = torch.randn(b, n, h, d, generator=g)
    ldk = {"weak": torch.nn.functional.logsigmoid(x) / 16,
           "medium": torch.nn.functional.logsigmoid(x + 1),
           "reference_benchmark": torch.nn.functional.logsigmoid(x),
           "strong": torch.nn.functional.logsigmoid(x * 2 - 4)}[regime]
    qf = cast(torch.randn(b, n, h, d, generator=g))
    kf = cast((1 - torch.exp(ldk)) * torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    vf = cast(torch.randn(b, n, h, e, generator=g))
    nb = b if lens is None else len(lens)
    cu = None if lens is None else torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    s0 = 0.1 * torch.randn(nb, h, d, e, generator=g)
    dof = cast(torch.randn(b, n, h, e, generator=g))
    dsf = 0.1 * torch.randn(nb, h, d, e, generator=g)  # upstream state gradient on the scale of the state
    q, k, v, lk, s0c = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(ldk), leaf(s0)
    o, sf = xb.lavd_fn(q, k, v, ldk=lk, initial_state=s0c, cu_seqlens=None if cu is None else cu.to(DEV))
    flag_fwd = _lavd_unsafe_flag(lib)
    ro, rsf = orc.lavd_forward(qf, kf, vf, ldk, None, s0, cu)
    assert_close("o", ro, o.float(), TOL_BF16)
    assert_close("final_state", rsf, sf, TOL_BF16)
    ((o.float() * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    flag_bwd = _lavd_unsafe_flag(lib)
    if regime == "weak":
        assert flag_fwd == 0 and flag_bwd == 0, "benchmark-range decays must stay on the one-reference kernels"
    if regime == "reference_benchmark" and dtype == torch.bfloat16:
        assert flag_fwd <= 1 and flag_bwd <= 1, "logsigmoid(N(0,1)) decays must stay on the tensor cores"
        if n >= 2048:
            assert flag_fwd == 1 and flag_bwd == 1, "expected the two-reference kernels to serve this"
    if regime == "strong":
        assert flag_fwd == 2 and flag_bwd == 2, "out-of-range decays must fall back to the scan"
    rq, rk, rv, rlk, _, rs0 = orc.lavd_backward(qf, kf, vf, ldk, None, dof, s0, dsf, cu)
    assert_close("dq", rq, q.grad.float(), TOL_BF16)
    assert_close("dk", rk, k.grad.float(), TOL_BF16)
    assert_close("dv", rv, v.grad.float(), TOL_BF16)
    assert_close("dldk", rlk, lk.grad, TOL_BF16)
    assert_close("dinitial_state", rs0, s0c.grad, TOL_BF16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("regime", ["weak", "reference_benchmark", "strong"])
@pytest.mark.parametrize("shape,lens", [((2, 384, 2), None), ((1, 300, 3), None),
                                        ((1, 700, 2), [1, 127, 128, 129, 300, 15]), ((1, 2048, 2), None)])
def test_lavd_value_decay_on_the_tensor_path(shape, lens, regime, dtype, lib):
    """Vector decay on the value features only (ldv, no ldk), D = E = 128, 16 bit: the same tcgen05
    kernels with the roles of the passes exchanged (o and dv are the passes with the decay on the
    output features, dq and dk those with the decay on the contraction).  Same three levels as the
    key-decay case."""
    import xopes_b200 as xb
    from xopes_b200 import _lib
    b, n, h = shape
    d = e = 128
    assert lib.la_lavd_path(n, d, e, _lib.dtype_code(torch.empty(0, dtype=dtype)), 0, 1, 0) == 1
    assert lib.la_lavd_path(n, d, e, _lib.dtype_code(torch.empty(0, dtype=dtype)), 1, 1, 0) == 0
    g = torch.Generator().manual_seed(19)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    x = torch.randn(b, n, h, e, generator=g)
    ldv = {"weak": torch.nn.functional.logsigmoid(x) / 16,
           "reference_benchmark": torch.nn.functional.logsigmoid(x),
           "strong": torch.nn.functional.logsigmoid(x * 2 - 4)}[regime]
    qf = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    kf = cast(torch.randn(b, n, h, d, generator=g))
    vf = cast((1 - torch.exp(ldv)) * torch.randn(b, n, h, e, generator=g))
    nb = b if lens is None else len(lens)
    cu = None if lens is None else torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    s0 = 0.1 * torch.randn(nb, h, d, e, generator=g)
    dof = cast(torch.randn(b, n, h, e, generator=g))
    dsf = 0.1 * torch.randn(nb, h, d, e, generator=g)
    q, k, v, lv, s0c = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(ldv), leaf(s0)
    o, sf = xb.lavd_fn(q, k, v, ldv=lv, initial_state=s0c, cu_seqlens=None if cu is None else cu.to(DEV))
    flag_fwd = _lavd_unsafe_flag(lib)
    ro, rsf = orc.lavd_forward(qf, kf, vf, None, ldv, s0, cu)
    assert_close("o", ro, o.float(), TOL_BF16)
    assert_close("final_state", rsf, sf, TOL_BF16)
    ((o.float() * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    flag_bwd = _lavd_unsafe_flag(lib)
    if regime == "weak":
        assert flag_fwd == 0 and flag_bwd == 0
    if regime == "reference_benchmark" and dtype == torch.bfloat16:
        assert flag_fwd <= 1 and flag_bwd <= 1, "logsigmoid(N(0,1)) decays must stay on the tensor cores"
    if regime == "strong":
        assert flag_fwd == 2 and flag_bwd == 2, "out-of-range decays must fall back to the scan"
    rq, rk, rv, _, rlv, rs0 = orc.lavd_backward(qf, kf, vf, None, ldv, dof, s0, dsf, cu)
    assert_close("dq", rq, q.grad.float(), TOL_BF16)
    assert_close("dk", rk, k.grad.float(), TOL_BF16)
    assert_close("dv", rv, v.grad.float(), TOL_BF16)
    assert_close("dldv", rlv, lv.grad, TOL_BF16)
    assert_close("dinitial_state", rs0, s0c.grad, TOL_BF16)


def test_lavd_benchmark_length_slice():
    """A (B=1, H=2) slice of benchmark configuration 3 at its full length N = 16384 (bf16,
    ldk = logsigmoid(x)/16, k = (1 - exp(ldk)) k_raw, no initial state): every gradient the
    configuration asks for, including the log-decay gradient, within 1e-2."""
    import xopes_b200 as xb
    from xopes_b200 import workloads
    w = workloads.lavd_inputs(1, 16384, 2, 128, 128, torch.bfloat16, seed=3)
    q, k, v, lk = (w[x].to(DEV).requires_grad_() for x in ("q", "k", "v", "ldk"))
    o, sf = xb.lightning_attn_func(q, k, v, ldk=lk, decay_type="vector")
    o.backward(w["do"].to(DEV))
    f = {n: t.float() for n, t in w.items()}
    ro, rsf = orc.lavd_forward(f["q"], f["k"], f["v"], f["ldk"], None)
    rq, rk, rv, rlk, _, _ = orc.lavd_backward(f["q"], f["k"], f["v"], f["ldk"], None, f["do"])
    assert_close("o", ro, o.float(), TOL_BF16)
    assert_close("final_state", rsf, sf, TOL_BF16)
    assert_close("dq", rq, q.grad.float(), TOL_BF16)
    assert_close("dk", rk, k.grad.float(), TOL_BF16)
    assert_close("dv", rv, v.grad.float(), TOL_BF16)
    assert_close("dldk", rlk, lk.grad, TOL_BF16)


def test_lasd_benchmark_length_slice_with_decay_gradient():
    """A (B=1, H=2) slice at the length of benchmark configuration 2 (N = 8192, bf16) with a
    data-dependent decay whose gradient is requested, an initial state and a final-state gradient."""
    import xopes_b200 as xb
    _run_lasd_case(xb.lasd_fn, 1, 8192, 2, 128, 128, seed=13, dtype=torch.bfloat16, use_state=True,
                   use_dfinal=True, weak_decay=False, tol=TOL_BF16)


# ------------------------------------------------------------------------------------------------
# varlen
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_FP32), (torch.bfloat16, TOL_BF16)])
def test_lasd_varlen_documents_are_independent(dtype, tol):
    import xopes_b200 as xb
    lens = [1, 127, 128, 129, 300, 5, 256]
    n, h, d, e = sum(lens), 2, 128, 128
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    qf, kf, vf, ld, _, dof, _ = _lasd_seeded(1, n, h, d, e, 3, dtype, False, False, False)
    g = torch.Generator().manual_seed(4)
    s0 = 0.1 * torch.randn(len(lens), h, d, e, generator=g)
    dsf = torch.randn(len(lens), h, d, e, generator=g)
    q, k, v, ldc, s0c = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(ld), leaf(s0)
    o, sf = xb.lasd_fn(q, k, v, ldc, initial_state=s0c, cu_seqlens=cu.to(DEV))
    ro, rsf = orc.lasd_forward(qf, kf, vf, ld, s0, cu)
    assert_close("o", ro, o.float(), tol)
    assert_close("final_state", rsf, sf, tol)
    ((o.float() * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    rq, rk, rv, rld, rs0 = orc.lasd_backward(qf, kf, vf, ld, dof, s0, dsf, cu)
    assert_close("dq", rq, q.grad.float(), tol)
    assert_close("dk", rk, k.grad.float(), tol)
    assert_close("dv", rv, v.grad.float(), tol)
    assert_close("dld", rld, ldc.grad, dld_tol(dtype, tol))
    assert_close("dinitial_state", rs0, s0c.grad, tol)


@pytest.mark.parametrize("reverse_heavy", [False, True])
def test_lasd_extreme_decay(reverse_heavy):
    """Log decays of -2 to -8 per token: a 32-token batch decays by hundreds of bits, beyond what
    the factorised decay mask of the tensor-core path may represent, so its diagonal batches take
    the per-element path; mixed with mild heads that stay factorised."""
    import xopes_b200 as xb
    b, n, h, d, e = 2, 300, 4, 128, 128
    dtype = torch.bfloat16
    qf, kf, vf, ld, s0, dof, dsf = _lasd_seeded(b, n, h, d, e, 31, dtype, True, True, False)
    g = torch.Generator().manual_seed(32)
    ld = -(2.0 + 6.0 * torch.rand(b, n, h, generator=g))
    ld[:, :, 0] = -0.01 * torch.rand(b, n, generator=g)      # one mild head
    if reverse_heavy:
        ld[:, ::7, 1] = -40.0                                 # isolated near-resets
    q, k, v, ldc, s0c = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(ld), leaf(s0)
    o, sf = xb.lasd_fn(q, k, v, ldc, initial_state=s0c)
    ro, rsf = orc.lasd_forward(qf, kf, vf, ld, s0)
    assert_close("o", ro, o.float(), TOL_BF16)
    assert_close("final_state", rsf, sf, TOL_BF16)
    ((o.float() * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    rq, rk, rv, rld, rs0 = orc.lasd_backward(qf, kf, vf, ld, dof, s0, dsf)
    assert torch.isfinite(q.grad).all() and torch.isfinite(k.grad).all() and torch.isfinite(v.grad).all()
    assert_close("dq", rq, q.grad.float(), TOL_BF16)
    assert_close("dk", rk, k.grad.float(), TOL_BF16)
    assert_close("dv", rv, v.grad.float(), TOL_BF16)
    assert_close("dld", rld, ldc.grad, dld_tol(dtype, TOL_BF16))
    assert_close("dinitial_state", rs0, s0c.grad, TOL_BF16)


@pytest.mark.parametrize("shape", [(5, 400, 32, 128, 128), (3, 513, 30, 128, 128), (40, 256, 4, 128, 128)])
def test_lasd_more_pairs_than_sms(shape):
    """More (sequence, head) pairs than SMs: the chunk passes split the chunk space evenly over
    one CTA per SM and hand the running state of a cut sequence from one CTA to the next; with
    more than half as many, the merged dk/dv launch does."""
    import xopes_b200 as xb
    _run_lasd_case(xb.lasd_fn, *shape, seed=11, dtype=torch.bfloat16, use_state=True, use_dfinal=True,
                   weak_decay=False, tol=TOL_BF16)


@pytest.mark.parametrize("want_dld", [False, True])
@pytest.mark.parametrize("ndocs", [44, 19])  # 200 and 100 (document, head) pairs
def test_lasd_varlen_many_documents(want_dld, ndocs):
    """Ragged documents (empty, one token, several times a CTA's share of the chunk space) with
    more (document, head) pairs than SMs."""
    import xopes_b200 as xb
    g = torch.Generator().manual_seed(21)
    lens = [3000, 0, 1, 128] + [int(x) for x in torch.randint(0, 400, (ndocs,), generator=g)] + [0, 700]
    n, h, d, e = sum(lens), 4, 128, 128
    dtype = torch.bfloat16
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    qf, kf, vf, ld, _, dof, _ = _lasd_seeded(1, n, h, d, e, 5, dtype, False, False, False)
    s0 = 0.1 * torch.randn(len(lens), h, d, e, generator=g)
    dsf = torch.randn(len(lens), h, d, e, generator=g)
    q, k, v, s0c = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(s0)
    ldc = leaf(ld) if want_dld else ld.to(DEV)
    o, sf = xb.lasd_fn(q, k, v, ldc, initial_state=s0c, cu_seqlens=cu.to(DEV))
    ro, rsf = orc.lasd_forward(qf, kf, vf, ld, s0, cu)
    assert_close("o", ro, o.float(), TOL_BF16)
    assert_close("final_state", rsf, sf, TOL_BF16)
    ((o.float() * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    rq, rk, rv, rld, rs0 = orc.lasd_backward(qf, kf, vf, ld, dof, s0, dsf, cu)
    assert_close("dq", rq, q.grad.float(), TOL_BF16)
    assert_close("dk", rk, k.grad.float(), TOL_BF16)
    assert_close("dv", rv, v.grad.float(), TOL_BF16)
    if want_dld:
        assert_close("dld", rld, ldc.grad, dld_tol(dtype, TOL_BF16))
    assert_close("dinitial_state", rs0, s0c.grad, TOL_BF16)
    st = ctypes.c_int(-1)
    lib = xb._lib.load()
    assert lib.la_device_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(st)) == 0
    assert st.value == 0, f"a bounded wait ran out (code {st.value})"


# ------------------------------------------------------------------------------------------------
# decode
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("vector", [False, True])
@pytest.mark.parametrize("shape", [(4, 3, 128, 128), (2, 2, 64, 32), (2, 2, 33, 256)])
def test_decode_loop_in_place(shape, vector):
    """A short decode loop (configuration 4 scaled down): bf16 tokens, fp32 state carried in place;
    the oracle sees fp32 up-casts of the same bf16 inputs so that it carries an fp32 state too."""
    import xopes_b200 as xb
    from xopes_b200 import workloads
    b, h, d, e = shape
    w = workloads.decode_inputs(b, h, d, e, steps=5, vector=vector, seed=0)
    state = w["state"].to(DEV).clone()
    rstate = w["state"].clone()
    for t in w["steps"]:
        q, k, v = t["q"].to(DEV), t["k"].to(DEV), t["v"].to(DEV)
        if vector:
            o, s2 = xb.lavd_decode_step(q, k, v, t["ldk"].to(DEV), state)
            ro, rstate = orc.decode_step_vector(t["q"].float(), t["k"].float(), t["v"].float(),
                                                t["ldk"], rstate)
        else:
            o, s2 = xb.lasd_decode_step(q, k, v, w["ld"].to(DEV), state)
            ro, rstate = orc.decode_step_scalar(t["q"].float(), t["k"].float(), t["v"].float(),
                                                w["ld"], rstate)
        assert s2.data_ptr() == state.data_ptr()
        assert_close("o", ro, o.float(), TOL_BF16)
        assert_close("state", rstate, state, TOL_FP32)


def test_decode_matches_fn_with_one_token():
    import xopes_b200 as xb
    from xopes_b200 import workloads
    w = workloads.decode_inputs(3, 2, 128, 128, steps=1, vector=True, seed=1)
    t = w["steps"][0]
    q, k, v, ldk = (t[x].to(DEV) for x in ("q", "k", "v", "ldk"))
    s = w["state"].to(DEV)
    o1, s1 = xb.lavd_fn(q, k, v, ldk=ldk, initial_state=s)
    o2, s2 = xb.lavd_decode_step(q, k, v, ldk, s, inplace=False)
    assert_close("o", o1.float(), o2.float(), 1e-6)
    assert_close("state", s1, s2, 1e-6)
    ld = w["ld"].to(DEV)
    o1, s1 = xb.lasd_fn(q, k, v, ld, initial_state=s)
    o2, s2 = xb.lasd_decode_step(q, k, v, ld, s, inplace=False)
    assert_close("o", o1.float(), o2.float(), 1e-6)
    assert_close("state", s1, s2, 1e-6)


# ------------------------------------------------------------------------------------------------
# dispatcher and constant decay
# ------------------------------------------------------------------------------------------------
def test_lightning_attn_func_dispatch_matches_direct_calls():
    import xopes_b200 as xb
    b, n, h, d, e = 2, 140, 2, 32, 32
    qf, kf, vf, ld, s0, dof, _ = _lasd_seeded(b, n, h, d, e, 21, torch.float32, True, False, False)
    q, k, v = qf.to(DEV), kf.to(DEV), vf.to(DEV)
    o1, s1 = xb.lightning_attn_func(q, k, v, ld=ld.to(DEV), initial_state=s0.to(DEV), decay_type="scalar")
    o2, s2 = xb.lasd_fn(q, k, v, ld.to(DEV), initial_state=s0.to(DEV))
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    ldk = torch.nn.functional.logsigmoid(torch.randn(b, n, h, d, generator=torch.Generator().manual_seed(2)))
    o3, s3 = xb.lightning_attn_func(q, k, v, ldk=ldk.to(DEV), decay_type="vector")
    ro, rs = orc.lavd_forward(qf, kf, vf, ldk, None)
    assert_close("o", ro, o3, TOL_FP32)
    assert_close("state", rs, s3, TOL_FP32)
    with pytest.raises(NotImplementedError):
        xb.lightning_attn_func(q, k, v, decay_type="element")


def test_constant_decay_default_path_with_learnable_decay_and_no_decay():
    """decay_type="constant" (the dispatcher's default, constant_decay/lacd_torch.py): a per-head (H,)
    log decay, or none at all; the gradient of the (H,) vector is summed over batch and sequence."""
    import xopes_b200 as xb
    b, n, h, d, e = 2, 130, 3, 32, 48
    qf, kf, vf, _, _, dof, _ = _lasd_seeded(b, n, h, d, e, 22, torch.float32, False, False, False)
    ld_h = torch.log(1 - 2.0 ** (-2 - torch.arange(h, dtype=torch.float32)))
    q, k, v, ld = leaf(qf), leaf(kf), leaf(vf), leaf(ld_h)
    o, sf = xb.lightning_attn_func(q, k, v, ld=ld)
    (o * dof.to(DEV)).sum().backward()
    full = ld_h.view(1, 1, h).expand(b, n, h)
    ro, rsf = orc.lasd_forward(qf, kf, vf, full)
    rq, rk, rv, rld, _ = orc.lasd_backward(qf, kf, vf, full, dof)
    assert_close("o", ro, o, TOL_FP32)
    assert_close("state", rsf, sf, TOL_FP32)
    assert_close("dq", rq, q.grad, TOL_FP32)
    assert_close("dk", rk, k.grad, TOL_FP32)
    assert_close("dv", rv, v.grad, TOL_FP32)
    assert_close("dld", rld.sum((0, 1)), ld.grad, TOL_FP32)
    o0, s0 = xb.lightning_attn_func(q.detach(), k.detach(), v.detach())  # no decay at all
    ro0, rs0 = orc.lasd_forward(qf, kf, vf, torch.zeros(b, n, h))
    assert_close("o (no decay)", ro0, o0, TOL_FP32)
    assert_close("state (no decay)", rs0, s0, TOL_FP32)


@pytest.mark.parametrize("shape,which,lens,act", [
    ((2, 384, 2, 64, 64), "ldk", None, False),
    ((1, 300, 3, 64, 32), "ldk", None, True),
    ((2, 256, 2, 128, 64), "ldv", None, False),
    ((1, 700, 2, 96, 128), "ldk", [1, 127, 128, 129, 300, 15], False),
])
def test_lavd_narrow_heads_run_padded_on_the_tensor_path(shape, which, lens, act, lib):
    """Vector decay with head dimensions below 128 in 16 bit: the operands are zero-padded to the
    128-wide tiles of the tcgen05 kernels and the results cut back (the scan kernels are not
    involved: level 0)."""
    import xopes_b200 as xb
    b, n, h, d, e = shape
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(23)
    cast = lambda t: t.to(dtype).float()  # noqa: E731
    f = d if which == "ldk" else e
    x = torch.randn(b, n, h, f, generator=g) + (3.0 if act else 0.0)
    ld = torch.nn.functional.logsigmoid(x.double()).float() if act else torch.nn.functional.logsigmoid(x) / 16
    qf = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    kf = cast(torch.randn(b, n, h, d, generator=g) * d ** -0.5)
    vf = cast(torch.randn(b, n, h, e, generator=g))
    nb = b if lens is None else len(lens)
    cu = None if lens is None else torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int64)
    s0 = 0.1 * torch.randn(nb, h, d, e, generator=g)
    dof = cast(torch.randn(b, n, h, e, generator=g))
    dsf = 0.1 * torch.randn(nb, h, d, e, generator=g)
    q, k, v, lc, s0c = leaf(qf, dtype), leaf(kf, dtype), leaf(vf, dtype), leaf(x if act else ld), leaf(s0)
    kw = {which: lc}
    o, sf = xb.lavd_fn(q, k, v, initial_state=s0c, cu_seqlens=None if cu is None else cu.to(DEV),
                       decay_activation="logsigmoid" if act else None, **kw)
    assert tuple(o.shape) == (b, n, h, e) and tuple(sf.shape) == (nb, h, d, e)
    assert _lavd_unsafe_flag(lib) == 0
    ldk, ldv = (ld, None) if which == "ldk" else (None, ld)
    ro, rsf = orc.lavd_forward(qf, kf, vf, ldk, ldv, s0, cu)
    assert_close("o", ro, o.float(), TOL_BF16)
    assert_close("final_state", rsf, sf, TOL_BF16)
    ((o.float() * dof.to(DEV)).sum() + (sf * dsf.to(DEV)).sum()).backward()
    rq, rk, rv, rlk, rlv, rs0 = orc.lavd_backward(qf, kf, vf, ldk, ldv, dof, s0, dsf, cu)
    assert_close("dq", rq, q.grad.float(), TOL_BF16)
    assert_close("dk", rk, k.grad.float(), TOL_BF16)
    assert_close("dv", rv, v.grad.float(), TOL_BF16)
    rl = rlk if which == "ldk" else rlv
    if act:
        rl = (rl.double() * torch.sigmoid(-x.double())).float()
    assert tuple(lc.grad.shape) == (b, n, h, f)
    assert_close("dld", rl, lc.grad, TOL_BF16)
    assert_close("dinitial_state", rs0, s0c.grad, TOL_BF16)
