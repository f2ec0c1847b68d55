"""Host logic of the optimizers, hooks and utilities built on top of Newton-Schulz, against vectors produced by
the reference itself (tests/golden/make_golden.py, section "consumers").

There is no CPU Newton-Schulz in the package, so on this side ``muon_utils.newton_schulz`` is replaced by the
test-only torch restatement; everything around it (momentum, second moments, scale factors, hooks, retraction,
spectral clipping algebra, eigen-decomposition route) is the package's own code.  The GPU counterpart of this file
runs the same cases on the kernels.
"""

import re

import pytest
import torch

from emerging_optimizers_b200 import registry
from emerging_optimizers_b200.orthogonalized_optimizers import (
    MOP,
    AdaptiveMuon,
    Muon,
    MuonHyperball,
    PolarGrad,
    Scion,
    Spel,
    muon_utils,
    polargrad,
    spectral_clipping_utils,
)
from emerging_optimizers_b200.weight_update_hooks import (
    HyperballHook,
    NoOpWeightUpdateHook,
    RadialBrakeHook,
    RelativeUpdateHook,
)
from tests import _consumers
from tests._torch_ref import newton_schulz_torch


def _cpu_newton_schulz(x, steps, coefficient_type="quintic", **kwargs):
    bf16 = torch.get_float32_matmul_precision() == "medium"
    return newton_schulz_torch(x, steps, coefficient_type, bf16=bf16)


@pytest.fixture
def cpu_ns(monkeypatch):
    monkeypatch.setattr(muon_utils, "newton_schulz", _cpu_newton_schulz)


@pytest.mark.parametrize("precision", ["highest", "medium"])
@pytest.mark.parametrize("name", _consumers.OPTIMIZER_CASES)
def test_optimizer_steps_match_reference(cpu_ns, name, precision):
    want = _consumers.golden()
    got, _ = _consumers.run_case(name, precision, "cpu")
    # Same torch CPU operations in the same order as the reference: agreement to rounding at "highest"; on the
    # bf16 path a one-ulp difference somewhere flips a few bf16 roundings downstream.
    tol = 1e-5 if precision == "highest" else 2e-3
    for key, val in got.items():
        ref = torch.from_numpy(want[f"{name}.{precision}.{key}"])
        assert val.shape == ref.shape, key
        assert _consumers.rel_fro(val, ref) <= tol, (key, _consumers.rel_fro(val, ref))


@pytest.mark.parametrize("name", sorted(_consumers.CASES["spectral"]))
def test_spectral_functions_match_reference(cpu_ns, name):
    fn, shape, seed, kw = _consumers.CASES["spectral"][name]
    x = _consumers.randn(*shape, seed=seed, scale=0.2)
    prev = torch.get_float32_matmul_precision()
    torch.set_float32_matmul_precision("highest")
    try:
        y = getattr(spectral_clipping_utils, fn)(x, **kw)
    finally:
        torch.set_float32_matmul_precision(prev)
    ref = torch.from_numpy(_consumers.golden()[f"spectral.{name}"])
    assert y.shape == ref.shape == x.shape
    assert _consumers.rel_fro(y, ref) <= 1e-5


@pytest.mark.parametrize("name", sorted(_consumers.CASES["one_sided"]))
def test_one_sided_polar_update_matches_reference(name):
    shape, seed, kw = _consumers.CASES["one_sided"][name]
    x = _consumers.randn(*shape, seed=seed)
    y = polargrad.one_sided_polargrad_orth_fn(x, **kw)
    ref = torch.from_numpy(_consumers.golden()[f"one_sided.{name}"])
    assert _consumers.rel_fro(y, ref) <= 1e-5
    plain = {k: v for k, v in kw.items() if k != "side"}
    wrapper = polargrad.left_polargrad_orth_fn if kw["side"] == "left" else polargrad.right_polargrad_orth_fn
    assert torch.equal(wrapper(x, **plain), y)


def test_one_sided_polar_update_is_a_polar_factor():
    x = _consumers.randn(12, 40, seed=1)
    u = polargrad.left_polargrad_orth_fn(x, alpha=0.0)
    assert torch.allclose(u @ u.T, torch.eye(12), atol=1e-4)
    nuc = torch.linalg.svdvals(x).sum()
    assert torch.allclose(polargrad.left_polargrad_orth_fn(x), u * nuc, rtol=1e-4, atol=1e-5)
    centered = polargrad.right_polargrad_orth_fn(x.T.contiguous(), center_rows=True)
    assert centered.mean(dim=0).abs().max() < 1e-5
    with pytest.raises(ValueError, match="side must be 'left' or 'right'"):
        polargrad.one_sided_polargrad_orth_fn(x, side="both")


def test_registry_and_constructor_errors():
    for name, cls in (
        ("scion", Scion), ("spel", Spel), ("polargrad", PolarGrad), ("adaptive_muon", AdaptiveMuon),
        ("muon_hyperball", MuonHyperball), ("muon", Muon), ("mop", MOP),
    ):  # fmt: skip
        assert registry.get_optimizer_cls(name) is cls
    w = [torch.nn.Parameter(torch.ones(4, 8))]
    for cls in (Scion, Spel):
        with pytest.raises(ValueError, match="num_ns_steps must be at least 1, got 0"):
            cls(w, num_ns_steps=0)
    with pytest.raises(ValueError, match="num_ns_steps must be at least 1"):
        AdaptiveMuon(w, 1e-3, 0.9, 0.0, num_ns_steps=0)
    with pytest.raises(ValueError, match="num_ns_steps must be positive, got -1"):
        PolarGrad(w, num_ns_steps=-1)
    PolarGrad(w, num_ns_steps=0)
    with pytest.raises(ValueError, match='moment2_method="namo" is incompatible'):
        AdaptiveMuon(w, 1e-3, 0.9, 0.1, moment2_method="namo", weight_decay_method="l2")
    with pytest.raises(KeyError, match="manages its own HyperballHook"):
        MuonHyperball(w, hyperball_radius=1.0, weight_update_hook=NoOpWeightUpdateHook())
    with pytest.raises(ValueError, match="almost zero norm"):
        MuonHyperball([torch.nn.Parameter(torch.zeros(4, 8))], hyperball_radius=1.0)
    with pytest.raises(ValueError, match=re.escape("hyperball_radius=1.0 was specified")):
        MuonHyperball(w, hyperball_radius=1.0)
    MuonHyperball(w, hyperball_radius=32**0.5)
    scion = Scion(w)
    assert scion.defaults["weight_decay"] == 1 and scion.weight_decay_method == "decoupled" and not scion.nesterov


def test_adaptive_muon_state_shapes_and_errors(cpu_ns):
    shapes = {"adamuon": {(8, 4): (8, 4), (4, 8): (4, 8)}, "normuon": {(8, 4): (8, 1), (4, 8): (1, 8), (6, 6): (6, 1)},
              "namo": {(8, 4): (1,), (4, 8): (1,)}}  # fmt: skip
    for method, table in shapes.items():
        params = [torch.nn.Parameter(torch.randn(*s)) for s in table]
        opt = AdaptiveMuon(params, 1e-2, 0.9, 0.0, moment2_method=method)
        for p in params:
            p.grad = torch.randn_like(p)
        opt.step()
        for p in params:
            assert tuple(opt.state[p]["moment2_buffer"].shape) == table[tuple(p.shape)]
            assert set(opt.state[p]) == {"momentum_buffer", "moment2_buffer"}
        assert opt.param_groups[0]["beta2"] == 0.95 and opt.param_groups[0]["eps"] == 1e-8
    for method in ("adamuon", "namo"):
        p = torch.nn.Parameter(torch.randn(2, 3, 4))
        p.grad = torch.randn_like(p)
        with pytest.raises(ValueError, match="only supports 2D parameters"):
            AdaptiveMuon([p], 1e-2, 0.9, 0.0, moment2_method=method).step()
    p = torch.nn.Parameter(torch.randn(4, 8))
    p.grad = torch.randn_like(p)
    with pytest.raises(TypeError, match="Invalid second moment method: nope"):
        AdaptiveMuon([p], 1e-2, 0.9, 0.0, moment2_method="nope").step()
    with pytest.raises(ValueError, match="closure is not supported"):
        AdaptiveMuon([p], 1e-2, 0.9, 0.0).step(lambda: 0.0)


def test_normuon_keeps_the_norm_of_the_raw_update(cpu_ns):
    p = torch.nn.Parameter(_consumers.randn(16, 24, seed=3))
    opt = AdaptiveMuon([p], 1e-2, 0.9, 0.0, moment2_method="normuon", scale_mode="unit_rms_norm", fp32_matmul_prec="highest")
    p.grad = _consumers.randn(16, 24, seed=4)
    before = p.detach().clone()
    opt.step()
    raw = _cpu_newton_schulz(opt.state[p]["momentum_buffer"], 5, "quintic")
    applied = (before - p.detach()) / 1e-2 / (16 / 24) ** 0.5
    assert torch.allclose(applied.norm(), raw.norm(), rtol=1e-4)


def test_spel_retracts_to_near_orthogonal(cpu_ns):
    p = torch.nn.Parameter(_consumers.randn(16, 32, seed=5, scale=0.1))
    opt = Spel([p], lr=0.1, fp32_matmul_prec="highest", coefficient_type="polar_express", num_ns_steps=8)
    for k in range(2):
        p.grad = _consumers.randn(16, 32, seed=6 + k)
        opt.step()
    assert torch.allclose(p.detach() @ p.detach().T, torch.eye(16), atol=5e-2)


@pytest.mark.parametrize("precision", ["highest", "medium"])
@pytest.mark.parametrize("name", sorted(_consumers.CASES["split_qkv"]["cases"]))
def test_split_qkv_muon_matches_reference_per_piece(cpu_ns, name, precision):
    want = _consumers.golden()
    got, _ = _consumers.run_split_qkv(name, precision, "cpu")
    for key, val in got.items():
        ref = torch.from_numpy(want[f"split_qkv.{name}.{precision}.{key}"])
        assert _consumers.rel_fro(val, ref) <= (1e-5 if precision == "highest" else 2e-3), key


@pytest.mark.parametrize("groups,split,per_head,head_dim", [
    (1, (6, 2, 2), False, None), (3, (4, 2, 2), False, None), (3, (4, 2, 2), True, 2), (2, (8, 4, 4), True, 4),
    (4, (2, 2, 2), True, 1), (1, (5, 3, 7), False, None),
])  # fmt: skip
def test_split_qkv_routes_every_row_to_its_own_logical_matrix(groups, split, per_head, head_dim):
    """The layout algebra on its own: with an 'orthogonalizer' that just tags every matrix it is handed, each row of
    the fused weight must come back tagged by the logical matrix the explicit index arithmetic assigns it to, and
    the values themselves must return to their rows."""
    from emerging_optimizers_b200.orthogonalized_optimizers import SplitQkvMuon

    hidden, per_group = 5, sum(split)
    rows = groups * per_group
    grad = torch.arange(rows * hidden, dtype=torch.float32).reshape(rows, hidden)
    p = torch.nn.Parameter(torch.zeros(rows, hidden))
    p.is_qkv = True
    opt = SplitQkvMuon([p], qkv_split_shapes=split, num_query_groups=groups, per_head=per_head, head_dim=head_dim)
    seen = []

    def tagger(x):
        # one call may carry a stack of equally shaped matrices: tag each matrix by the rows it contains
        mats = x if x.dim() == 3 else x.unsqueeze(0)
        for m in mats:
            seen.append(sorted(int(v) // hidden for v in m[:, 0].tolist()))
        return x.clone()

    opt.scaled_orthogonalize_fn = tagger
    out = opt.orthogonalize(p, grad)
    assert torch.equal(out, grad)  # identity on the values: every row went back to where it came from
    want = []
    offset = 0
    for block in split:
        rows_of_block = [g * per_group + offset + r for g in range(groups) for r in range(block)]
        if per_head:
            want += [rows_of_block[i : i + head_dim] for i in range(0, len(rows_of_block), head_dim)]
        else:
            want.append(rows_of_block)
        offset += block
    assert sorted(seen) == sorted(want)


def test_split_qkv_muon_argument_checks(cpu_ns):
    from emerging_optimizers_b200.orthogonalized_optimizers import SplitQkvMuon

    w = torch.nn.Parameter(torch.randn(30, 16))
    with pytest.raises(ValueError, match="three positive row counts"):
        SplitQkvMuon([w], qkv_split_shapes=(8, 8))
    with pytest.raises(ValueError, match="num_query_groups must be at least 1"):
        SplitQkvMuon([w], qkv_split_shapes=(8, 8, 8), num_query_groups=0)
    with pytest.raises(ValueError, match="per_head needs a head_dim"):
        SplitQkvMuon([w], qkv_split_shapes=(8, 8, 8), per_head=True, head_dim=3)
    opt = SplitQkvMuon([{"params": [w], "is_qkv": True}], qkv_split_shapes=(8, 8, 8))
    w.grad = torch.randn_like(w)
    with pytest.raises(ValueError, match="expected num_query_groups"):
        opt.step()


# ---------------------------------------------------------------------------------------------------------------
# weight-update hooks on their own
# ---------------------------------------------------------------------------------------------------------------


@pytest.mark.parametrize("shape", [(5,), (4, 6), (2, 3, 4)])
def test_hyperball_hook_norms(shape):
    hook = HyperballHook(radius=3.0)
    p, u = torch.randn(*shape), torch.randn(*shape) * 7
    assert hook.pre_weight_update_inplace(p, u) is None
    assert torch.allclose(u.norm(), torch.tensor(3.0), rtol=1e-6)
    p.add_(u, alpha=-0.1)
    hook.post_weight_update_inplace(p, None)
    assert torch.allclose(p.norm(), torch.tensor(3.0), rtol=1e-6)
    tiny = torch.full(shape, 1e-20)
    hook.pre_weight_update_inplace(p, tiny)
    assert tiny.count_nonzero() == 0
    bf = torch.randn(*shape).bfloat16()
    hook.post_weight_update_inplace(bf, None)
    assert bf.dtype == torch.bfloat16 and abs(float(bf.float().norm()) - 3.0) < 0.05


@pytest.mark.parametrize("shape", [(5,), (4, 6)])
def test_relative_update_hook(shape):
    hook = RelativeUpdateHook()
    p, u = torch.randn(*shape) * 2, torch.randn(*shape) * 0.01
    direction = u / u.norm()
    p0 = p.clone()
    hook.pre_weight_update_inplace(p, u)
    assert torch.allclose(u.norm(), p.norm(), rtol=1e-6) and torch.allclose(u / u.norm(), direction, atol=1e-6)
    hook.post_weight_update_inplace(p, None)
    assert torch.equal(p, p0)
    for dead_p, dead_u in ((torch.zeros(*shape), torch.ones(*shape)), (torch.ones(*shape), torch.zeros(*shape))):
        hook.pre_weight_update_inplace(dead_p, dead_u)
        assert dead_u.count_nonzero() == 0


@pytest.mark.parametrize("outward,inward", [(0.5, 1.0), (0.0, 0.0), (0.25, 0.75), (1.0, 1.0)])
def test_radial_brake_hook_keeps_the_configured_fraction(outward, inward):
    hook = RadialBrakeHook(outward_scale=outward, inward_scale=inward)
    for factor, kept in ((1.5, outward), (0.5, inward)):
        p = torch.randn(6, 8)
        n0 = p.norm()
        direction = p / n0
        state = hook.pre_weight_update_inplace(p, torch.zeros_like(p))
        assert torch.allclose(state, n0)
        p.mul_(factor)  # a purely radial update
        hook.post_weight_update_inplace(p, state)
        assert torch.allclose(p.norm(), n0 + kept * (factor - 1.0) * n0, rtol=1e-5)
        assert torch.allclose(p / p.norm(), direction, atol=1e-6)
    # a change of norm below eps is dropped altogether; a weight that became zero stays zero
    hook = RadialBrakeHook(eps=1e-3)
    p = torch.ones(4)
    s = hook.pre_weight_update_inplace(p, p)
    p.mul_(1.0 + 1e-4)
    hook.post_weight_update_inplace(p, s)
    assert torch.allclose(p.norm(), torch.tensor(2.0), rtol=1e-6)
    p = torch.ones(4)
    s = hook.pre_weight_update_inplace(p, p)
    p.zero_()
    hook.post_weight_update_inplace(p, s)
    assert p.count_nonzero() == 0


@pytest.mark.parametrize(
    "cls,kwargs,message",
    [
        (HyperballHook, dict(radius=1.0, eps=0.0), "eps must be finite and positive"),
        (HyperballHook, dict(radius=1.0, eps=float("inf")), "eps must be finite and positive"),
        (HyperballHook, dict(radius=float("nan")), "radius must be finite and at least eps"),
        (HyperballHook, dict(radius=1e-20), "radius must be finite and at least eps"),
        (RadialBrakeHook, dict(outward_scale=1.5), r"outward_scale must be in \[0, 1\]"),
        (RadialBrakeHook, dict(inward_scale=-0.1), r"inward_scale must be in \[0, 1\]"),
        (RadialBrakeHook, dict(eps=float("nan")), "eps must be finite and positive"),
        (RelativeUpdateHook, dict(eps=0.0), "eps must be positive"),
    ],
)
def test_hook_constructor_validation(cls, kwargs, message):
    with pytest.raises(ValueError, match=message):
        cls(**kwargs)
