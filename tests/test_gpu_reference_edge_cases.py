"""Edge cases the reference's own test file pins for Newton-Schulz, mirrored on the GPU kernels, and the fp32 bound
of BASELINE config 1 settled against a float64 run of the same iteration.

- polar factor by SVD, atol 0.1 (tests/test_muon_utils.py:82-102 of the reference);
- an input with condition number 1e12: ten polar_express / deepseekv4 steps must land closer to the polar factor
  than five quintic steps (:212-250 there);
- sixteen polar_express steps give an almost orthogonal matrix (:252-262 there; fp32 path);
- config 1 (1024 x 4096, five "simple" steps, fp32 path): the kernels and the reference's stored CPU result are
  both compared with a float64 run as a third party; the kernels must be within 1e-4 of it, or at least no
  further from it than the reference's own fp32 result is.
"""

import os

import numpy as np
import pytest
import torch

from emerging_optimizers_b200 import _native as nat
from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils
from emerging_optimizers_b200.utils import fp32_matmul_precision


pytestmark = pytest.mark.gpu


def _randn(*shape, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).cuda()


def _rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


@pytest.mark.parametrize("precision", ["highest", "medium"])
@pytest.mark.parametrize("shape", [(512, 512), (512, 256), (256, 512)])
def test_five_quintic_steps_are_close_to_the_svd_polar_factor(shape, precision):
    x = _randn(*shape, seed=11)
    with fp32_matmul_precision(precision):
        out = muon_utils.newton_schulz(x, steps=5, coefficient_type="quintic", use_syrk=(precision == "medium"))
    U, _, Vh = torch.linalg.svd(x.double(), full_matrices=False)
    torch.testing.assert_close(out.float(), (U @ Vh).float(), atol=1e-1, rtol=1e-7)
    assert nat.read_device_status() == 0


def _ill_conditioned(dim1, dim2, seed):
    """U diag(logspace(6, -6)) V^T with random orthonormal U, V: condition number 1e12."""
    k = min(dim1, dim2)
    u, _ = torch.linalg.qr(_randn(dim1, k, seed=seed).double())
    v, _ = torch.linalg.qr(_randn(dim2, k, seed=seed + 1).double())
    s = torch.logspace(6, -6, k, dtype=torch.float64, device="cuda")
    return (u @ torch.diag(s) @ v.T).float(), (u @ v.T).float()


@pytest.mark.parametrize("coefficient_type", ["polar_express", "deepseekv4"])
@pytest.mark.parametrize("shape", [(512, 512), (512, 256), (256, 512)])
def test_ten_steps_of_the_long_schedules_beat_five_quintic_steps_on_condition_number_1e12(shape, coefficient_type):
    x, polar = _ill_conditioned(*shape, seed=21)
    # fp32 path (the precision the reference's test runs at): three-plane split products must not lose the tiny
    # singular directions that this ordering depends on
    with fp32_matmul_precision("highest"):
        long_run = muon_utils.newton_schulz(x, steps=10, coefficient_type=coefficient_type)
        quintic = muon_utils.newton_schulz(x, steps=5, coefficient_type="quintic")
    d_long, d_quintic = float((long_run - polar).norm()), float((quintic - polar).norm())
    assert d_long < d_quintic, (d_long, d_quintic)
    # The same inputs in float64 arithmetic: the fp32 path must show the same gap, not merely the same sign.
    sets = muon_utils._COEFFICIENT_SETS
    mode = "repeat_last"
    ref_long = _ns_float64(x, list(muon_utils.get_coefficient_iterator(10, sets[coefficient_type], mode=mode)))
    ref_quintic = _ns_float64(x, list(muon_utils.get_coefficient_iterator(5, sets["quintic"], mode="cycle")))
    r_long, r_quintic = float((ref_long - polar.double()).norm()), float((ref_quintic - polar.double()).norm())
    print(f"{shape} {coefficient_type}: fp32 path {d_long:.4f} / {d_quintic:.4f}, float64 {r_long:.4f} / {r_quintic:.4f}")
    assert d_long == pytest.approx(r_long, rel=2e-2)
    assert d_quintic == pytest.approx(r_quintic, rel=2e-2)
    # The bf16 path is not asked for this ordering (the reference runs the test at "highest" only): singular values
    # below the bf16 rounding step (2^-9 of the largest) are noise there, and ten steps amplify that noise further
    # than five do.  It must still return finite values of the right size.
    with fp32_matmul_precision("medium"):
        long_bf16 = muon_utils.newton_schulz(x, steps=10, coefficient_type=coefficient_type, use_syrk=True)
    assert bool(torch.isfinite(long_bf16).all()) and float(long_bf16.norm()) <= 2.0 * min(shape) ** 0.5
    assert nat.read_device_status() == 0


@pytest.mark.parametrize("shape", [(512, 256), (256, 512)])
def test_sixteen_polar_express_steps_are_almost_orthogonal(shape):
    x = _randn(*shape, seed=31)
    with fp32_matmul_precision("highest"):
        out = muon_utils.newton_schulz(x, steps=16, coefficient_type="polar_express")
    o = out.double()
    gram = o @ o.T if shape[0] <= shape[1] else o.T @ o
    eye = torch.eye(gram.size(0), dtype=torch.float64, device="cuda")
    assert float((gram - eye).abs().max()) <= 1e-5
    assert nat.read_device_status() == 0


def _ns_float64(x, schedule):
    """The iteration of muon_utils.py:215-269 of the reference in float64 (norm, products and sums)."""
    X = x.double()
    tall = X.size(-2) > X.size(-1)
    if tall:
        X = X.mT
    X = X / X.norm()
    for a, b, c in schedule:
        A = X @ X.mT
        B = b * A + c * (A @ A)
        X = a * X + B @ X
    return X.mT if tall else X


def test_config1_fp32_path_is_no_further_from_float64_than_the_reference_is(golden_dir):
    rec = np.load(os.path.join(golden_dir, "config1.npz"))
    x = _randn(1024, 4096, seed=0)
    assert float(x.double().sum()) == pytest.approx(float(rec["x_sum"]), rel=1e-12)  # the reference saw these bits
    with fp32_matmul_precision("highest"):
        y = muon_utils.newton_schulz(x, steps=5, coefficient_type="simple")
    y64 = _ns_float64(x, [muon_utils._COEFFICIENT_SETS["simple"][0]] * 5)
    golden = torch.from_numpy(rec["highest.sample"]).cuda()  # the reference's CPU fp32 result, every 16th row / column
    err_kernel_full = _rel(y, y64)
    err_kernel = _rel(y[::16, ::16], y64[::16, ::16])
    err_reference = _rel(golden, y64[::16, ::16])
    print(f"config 1 fp32: kernels vs float64 {err_kernel_full:.3e} (sample {err_kernel:.3e}); "
          f"reference CPU fp32 vs float64 (sample) {err_reference:.3e}; kernels vs reference {_rel(y[::16, ::16], golden):.3e}")  # fmt: skip
    assert err_kernel <= max(1e-4, err_reference)
    assert err_kernel_full <= max(1e-4, 1.1 * err_reference)
    assert nat.read_device_status() == 0
