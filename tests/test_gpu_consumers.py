"""The optimizers, hooks and utilities built on Newton-Schulz, on the sm_100a kernels, against vectors produced by
the reference itself on CPU (tests/golden/make_golden.py, section "consumers").

What is compared is the *change* of each weight (after - initial), so that the large unchanged part of the weight
does not hide an error of the update; for Spel the weight itself (every step replaces it by a polar factor).
"""

import pytest
import torch

from emerging_optimizers_b200 import _native
from emerging_optimizers_b200.orthogonalized_optimizers import _consumers as consumer_switch
from emerging_optimizers_b200.orthogonalized_optimizers import polargrad, spectral_clipping_utils
from emerging_optimizers_b200.utils import fp32_matmul_precision
from tests import _consumers


pytestmark = pytest.mark.gpu

# Relative Frobenius tolerance of the weight change, per precision.  "highest" runs the three-plane bf16 split
# (fp32-accurate products); "medium" rounds A, S and X to bf16 at the same points as the reference's CPU bf16 path,
# so what is left is fp32 accumulation order flipping single bf16 roundings.
# Measured on a B200: at most 3e-6 at "highest" and 3e-3 at "medium" (Spel after three steps; most cases are
# bitwise equal at "medium" because the inner dimensions here are short).
TOL = {"highest": 1e-4, "medium": 1e-2}


# MOP takes its polar factor from the library SVD, not from the kernels of this package: covered on the CPU side only.
@pytest.mark.parametrize("precision", ["highest", "medium"])
@pytest.mark.parametrize("name", [n for n in _consumers.OPTIMIZER_CASES if n != "mop"])
def test_optimizer_steps_match_reference(name, precision):
    want = _consumers.golden()
    got, init = _consumers.run_case(name, precision, "cuda")
    tol = TOL[precision]
    for key, val in got.items():
        ref = torch.from_numpy(want[f"{name}.{precision}.{key}"])
        assert val.shape == ref.shape, key
        if key.endswith("momentum_buffer") and name != "muown":
            # plain EMA of the gradients: no kernel of this package is involved.  (Muown's buffer averages the
            # direction part of the gradient, which depends on the weights the previous steps produced.)
            assert _consumers.rel_fro(val, ref) <= 1e-6, key
        elif ".after" in key and name != "spel":
            w0 = init[int(key[1 : key.index(".")])]
            assert _consumers.rel_fro(val - w0, ref - w0) <= tol, (key, _consumers.rel_fro(val - w0, ref - w0))
        else:
            assert _consumers.rel_fro(val, ref) <= tol, (key, _consumers.rel_fro(val, ref))
    assert _native.read_device_status() == 0


@pytest.mark.parametrize("name", ["scion", "spel", "namo"])
def test_syrk_switch_gives_the_same_steps(name):
    """With the process-wide switch on, Scion / Spel / AdaptiveMuon run their symmetric products on the
    lower-triangular kernel: same products, same rounding, so the same weights."""
    plain, _ = _consumers.run_case(name, "medium", "cuda")
    consumer_switch.USE_SYRK = True
    try:
        syrk, _ = _consumers.run_case(name, "medium", "cuda")
    finally:
        consumer_switch.USE_SYRK = False
    for key in plain:
        assert torch.equal(plain[key], syrk[key]), key


@pytest.mark.parametrize("name", sorted(_consumers.CASES["spectral"]))
def test_spectral_functions_match_reference(name):
    fn, shape, seed, kw = _consumers.CASES["spectral"][name]
    x = _consumers.randn(*shape, seed=seed, scale=0.2).cuda()
    with fp32_matmul_precision("highest"):
        y = getattr(spectral_clipping_utils, fn)(x, **kw)
    ref = torch.from_numpy(_consumers.golden()[f"spectral.{name}"])
    assert y.shape == ref.shape
    assert _consumers.rel_fro(y.cpu(), ref) <= 1e-4, _consumers.rel_fro(y.cpu(), ref)


def test_spectral_clip_bounds_singular_values():
    x = _consumers.randn(256, 384, seed=7, scale=0.1).cuda()
    with fp32_matmul_precision("highest"):
        clipped = spectral_clipping_utils.spectral_clip(x, 0.8, 1.6)
        capped = spectral_clipping_utils.spectral_hardcap(x, 1.2)
    sv = torch.linalg.svdvals(x)
    assert sv.min() < 0.7 and sv.max() > 1.7  # the input really exceeds both bounds
    s = torch.linalg.svdvals(clipped)
    assert s.min() >= 0.8 - 5e-2 and s.max() <= 1.6 + 5e-2
    s = torch.linalg.svdvals(capped)
    assert s.max() <= 1.2 + 5e-2
    assert torch.allclose(s.sort().values, sv.clamp_max(1.2).sort().values, atol=5e-2)


@pytest.mark.parametrize("name", sorted(_consumers.CASES["one_sided"]))
def test_one_sided_polar_update_matches_reference(name):
    shape, seed, kw = _consumers.CASES["one_sided"][name]
    x = _consumers.randn(*shape, seed=seed).cuda()
    y = polargrad.one_sided_polargrad_orth_fn(x, **kw)
    ref = torch.from_numpy(_consumers.golden()[f"one_sided.{name}"])
    assert _consumers.rel_fro(y.cpu(), ref) <= 1e-4


@pytest.mark.parametrize("precision", ["highest", "medium"])
@pytest.mark.parametrize("name", sorted(_consumers.CASES["split_qkv"]["cases"]))
def test_split_qkv_muon_matches_reference_per_piece(name, precision):
    want = _consumers.golden()
    got, init = _consumers.run_split_qkv(name, precision, "cuda")
    for key, val in got.items():
        ref = torch.from_numpy(want[f"split_qkv.{name}.{precision}.{key}"])
        err = _consumers.rel_fro(val - init[key], ref - init[key])
        assert err <= TOL[precision], (key, err)
    assert _native.read_device_status() == 0


def test_split_qkv_per_head_runs_one_batched_call_per_step():
    """80 heads of 128 x 1024 inside one fused weight: the heads go through the library as one stack."""
    from emerging_optimizers_b200.orthogonalized_optimizers import SplitQkvMuon

    heads, head_dim, hidden = (64, 8, 8), 128, 1024
    w = torch.nn.Parameter(_consumers.randn(sum(heads) * head_dim, hidden, seed=9, scale=0.02).cuda())
    w.is_qkv = True
    opt = SplitQkvMuon(
        [w], lr=0.02, qkv_split_shapes=[h * head_dim // 8 for h in heads], num_query_groups=8, per_head=True,
        head_dim=head_dim, coefficient_type="polar_express", num_ns_steps=8, scale_mode="shape_scaling",
    )  # fmt: skip
    w.grad = _consumers.randn(*w.shape, seed=10, scale=1e-3).cuda()
    before = w.detach().clone()
    n0 = _native.launch_count
    opt.step()
    launches = _native.launch_count - n0
    assert launches == 4, launches  # sum of squares (2 kernels), normalise + cast, all eight iterations in one
    # every head's update is a 128 x 1024 polar factor (scale factor 1 for a wide matrix under "shape_scaling")
    upd = (before * (1 - 0.02 * 0.01) - w.detach()) / 0.02
    per_head = upd.view(8, -1, hidden).reshape(-1, head_dim, hidden)
    gram = per_head @ per_head.mT
    eye = torch.eye(head_dim, device="cuda")
    assert float((gram - eye).abs().max()) < 0.1
    assert _native.read_device_status() == 0
