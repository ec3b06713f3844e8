"""CPU: the oracle reproduces the vectors the reference itself produced (tests/golden/*.npz,
written by tests/golden/make_golden.py from lasd_torch / lavd_torch and autograd through them)."""
import pytest

from oracle import chunk_fixtures as cfx
from oracle import lightning_attn_oracle as orc
from util import TOL_FP32, assert_close, golden_cases, load_golden


@pytest.mark.parametrize("case", golden_cases("lasd_"))
def test_lasd_oracle_matches_reference_vectors(case):
    g = load_golden(case)
    s0, cu, dsf = g.get("initial_state"), g.get("cu_seqlens"), g.get("dfinal_state")
    o, sf = orc.lasd_forward(g["q"], g["k"], g["v"], g["ld"], s0, cu)
    assert_close("o", g["o"], o, TOL_FP32)
    assert_close("final_state", g["final_state"], sf, TOL_FP32)
    dq, dk, dv, dld, ds0 = orc.lasd_backward(g["q"], g["k"], g["v"], g["ld"], g["do"], s0, dsf, cu)
    for n, x in (("dq", dq), ("dk", dk), ("dv", dv), ("dld", dld)):
        assert_close(n, g[n], x, TOL_FP32)
    if s0 is not None:
        assert_close("dinitial_state", g["dinitial_state"], ds0, TOL_FP32)


@pytest.mark.parametrize("case", golden_cases("lavd_"))
def test_lavd_oracle_matches_reference_vectors(case):
    g = load_golden(case)
    s0, cu, dsf = g.get("initial_state"), g.get("cu_seqlens"), g.get("dfinal_state")
    k, ldv = g.get("k"), g.get("ldv")
    o, sf = orc.lavd_forward(g["q"], k, g["v"], g["ldk"], ldv, s0, cu)
    assert_close("o", g["o"], o, TOL_FP32)
    assert_close("final_state", g["final_state"], sf, TOL_FP32)
    dq, dk, dv, dldk, dldv, ds0 = orc.lavd_backward(g["q"], k, g["v"], g["ldk"], ldv, g["do"], s0,
                                                    dsf, cu)
    assert_close("dq", g["dq"], dq, TOL_FP32)
    assert_close("dv", g["dv"], dv, TOL_FP32)
    assert_close("dldk", g["dldk"], dldk, TOL_FP32)
    if k is not None:
        assert_close("dk", g["dk"], dk, TOL_FP32)
    if ldv is not None:
        assert_close("dldv", g["dldv"], dldv, TOL_FP32)
    if s0 is not None:
        assert_close("dinitial_state", g["dinitial_state"], ds0, TOL_FP32)


def test_oracle_varlen_equals_per_document_runs():
    """lasd_torch(cu_seqlens) is per-document lasd_torch (scalar_decay/lasd_torch.py:77-103)."""
    g = load_golden("lasd_varlen")
    cu = g["cu_seqlens"]
    o, sf = orc.lasd_forward(g["q"], g["k"], g["v"], g["ld"], g["initial_state"], cu)
    for i in range(len(cu) - 1):
        a0, a1 = int(cu[i]), int(cu[i + 1])
        oi, si = orc.lasd_forward(g["q"][:, a0:a1], g["k"][:, a0:a1], g["v"][:, a0:a1],
                                  g["ld"][:, a0:a1], g["initial_state"][i:i + 1])
        assert_close("o", oi, o[:, a0:a1], 1e-6)
        assert_close("state", si[0], sf[i], 1e-6)


def test_chunk_fixture_oracle_matches_reference_vectors():
    """oracle/chunk_fixtures.py against the outputs of the reference's own chunk-level fixtures
    (scalar_decay/torch_utils.py: lasd_intra_torch, compute_states, lasd_inter_torch)."""
    g = load_golden("chunkfx_lasd")
    q, k, v, ld, s0, block = g["q"], g["k"], g["v"], g["ld"], g["initial_state"], int(g["block"])
    for rev, tag in ((False, "fwd"), (True, "rev")):
        assert_close("intra_" + tag, g["intra_" + tag], cfx.lasd_chunk_intra(q, k, v, ld, block, rev), TOL_FP32)
        loc, glob = cfx.lasd_chunk_states(k, v, ld, s0, block, rev)
        assert_close("local_" + tag, g["local_" + tag], loc, TOL_FP32)
        assert_close("global_" + tag, g["global_" + tag], glob, TOL_FP32)
    assert_close("inter", g["inter"], cfx.lasd_chunk_inter(q, k, v, ld, s0, block), TOL_FP32)
    # the pieces add up: intra + inter is the full forward
    o, _ = orc.lasd_forward(q, k, v, ld, s0)
    assert_close("intra + inter", o, g["intra_fwd"] + g["inter"], TOL_FP32)


def test_normalize_gate_oracle_matches_reference_vectors():
    """oracle/normalize_oracle.py against outputs and autograd gradients of the reference's
    normalize_torch with a gate (every activation, both gate positions, with / without mean)."""
    import torch
    from oracle import normalize_oracle as norc
    g = load_golden("normgate")
    groups = int(g["num_groups"])
    e = g["x"].shape[-1] // groups
    for act in ("none", "relu", "sigmoid", "silu"):
        for pos in ("pre", "post"):
            for use_mean in (False, True):
                x, gate, w, b = (g[n].clone().requires_grad_() for n in ("x", "gate", "weight", "bias"))
                o = norc.normalize_gate(x, w, b, gate, act, pos, e ** 0.5, 1e-5, use_mean, groups)
                grads = torch.autograd.grad((o * g["do"].double()).sum(), [x, gate, w, b])
                tag = f"{act}_{pos}_{int(use_mean)}"
                assert_close(tag + ".o", g[tag + ".o"], o.float(), TOL_FP32)
                for n, got in zip(("dx", "dgate", "dweight", "dbias"), grads):
                    assert_close(f"{tag}.{n}", g[f"{tag}.{n}"], got.float(), TOL_FP32)
