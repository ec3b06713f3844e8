"""Helpers shared by the tests."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# acceptance tolerances on relative L2 error: fp32 outputs, 16-bit outputs / gradients / states
TOL_FP32 = 1e-5
TOL_BF16 = 1e-2


def rel_l2(ref, x):
    ref = ref.detach().double().cpu()
    x = x.detach().double().cpu()
    return float((ref - x).norm() / (ref.norm() + 1e-8))


def assert_close(name, ref, x, tol):
    """Relative-L2 acceptance; like the reference's assert_close (xopes/utils/test_utils.py:14-28)
    a tiny absolute error also passes, which covers all-zero references."""
    assert ref.shape == x.shape, f"{name}: shape {tuple(x.shape)} vs reference {tuple(ref.shape)}"
    assert torch.isfinite(x.detach().float()).all(), f"{name}: non-finite values"
    err = rel_l2(ref, x)
    max_abs = float((ref.detach().double().cpu() - x.detach().double().cpu()).abs().max())
    assert err <= tol or max_abs <= 1e-7, f"{name}: rel-L2 {err:.3e} > {tol:.1e} (max abs {max_abs:.3e})"


def golden_cases(prefix):
    return sorted(f[:-4] for f in os.listdir(GOLDEN) if f.startswith(prefix) and f.endswith(".npz"))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: torch.from_numpy(z[k]) for k in z.files}
