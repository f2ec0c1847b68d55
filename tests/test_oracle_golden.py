"""The numpy oracle against vectors produced by the reference itself (tests/golden/make_golden.py)."""

import json
import os

import numpy as np
import pytest

from oracle import ns_oracle as orc


def rel_fro(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


def _cases(golden_dir):
    with open(os.path.join(golden_dir, "ns_cases.json")) as f:
        return json.load(f)


def test_tables_match_reference(golden_dir):
    with open(os.path.join(golden_dir, "tables.json")) as f:
        tables = json.load(f)
    for name, rec in tables["schedules"].items():
        got = list(orc.coefficient_iterator(12, orc.COEFFICIENT_SETS[name], rec["mode"]))
        assert [list(t) for t in got] == rec["steps12"], name
        assert (name in orc.REPEAT_LAST_TYPES) == (rec["mode"] == "repeat_last")
    for key, val in tables["scale_factors"].items():
        mode, dims = key.split(":")
        m, n = (int(v) for v in dims.split("x"))
        assert orc.muon_scale_factor(m, n, mode) == pytest.approx(val, rel=1e-15)


@pytest.mark.parametrize("precision,tol", [("highest", 2e-5), ("medium", 1.2e-2)])
def test_newton_schulz_matches_reference(golden_dir, precision, tol):
    data = np.load(os.path.join(golden_dir, f"ns_{precision}.npz"))
    for name, meta in _cases(golden_dir).items():
        kw = dict(meta["kwargs"])
        if "custom_coefficient_sets" in kw:
            kw["custom_coefficient_sets"] = [tuple(t) for t in kw["custom_coefficient_sets"]]
        y = orc.newton_schulz(data[f"{name}.x"], precision=precision, **kw)
        ref = data[f"{name}.y"]
        assert y.shape == ref.shape and y.dtype == np.float32
        assert rel_fro(y, ref) <= tol, (name, rel_fro(y, ref))


def test_config1_matches_reference(golden_dir):
    torch = pytest.importorskip("torch")
    rec = np.load(os.path.join(golden_dir, "config1.npz"))
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(1024, 4096, generator=g, dtype=torch.float32).numpy()
    assert float(x.astype(np.float64).sum()) == pytest.approx(float(rec["x_sum"]), rel=1e-12)
    assert float((x.astype(np.float64) ** 2).sum()) == pytest.approx(float(rec["x_sumsq"]), rel=1e-12)
    # Five "simple" steps amplify fp32 round-off on this 1024 x 4096 input: two fp32 BLAS libraries with different
    # summation orders already differ by about 9e-5 here, hence the looser fp32 bound than for the small cases.
    for precision, tol in (("highest", 2e-4), ("medium", 1.2e-2)):
        y = orc.newton_schulz(x, 5, "simple", precision=precision)
        assert rel_fro(y[::16, ::16], rec[f"{precision}.sample"]) <= tol
        sv = np.linalg.svd(y.astype(np.float64), compute_uv=False)
        band = float(rec[f"{precision}.sv_max"]) - float(rec[f"{precision}.sv_min"])
        assert sv.min() >= float(rec[f"{precision}.sv_min"]) - 0.02 * band - tol
        assert sv.max() <= float(rec[f"{precision}.sv_max"]) + 0.02 * band + tol
        assert np.linalg.norm(y.astype(np.float64)) == pytest.approx(float(rec[f"{precision}.fro"]), rel=5e-3)


def test_deferred_normalisation_is_as_accurate_on_large_matrices_only(golden_dir):
    """Why the kernels defer the normalisation only from 2^22 elements per matrix: on the 1024 x 4096 input the
    variant is as close to the reference's result as the normalise-first path, on the small golden cases single
    roundings of the un-normalised first iterate show and the 2e-2 bound does not hold."""
    torch = pytest.importorskip("torch")
    rec = np.load(os.path.join(golden_dir, "config1.npz"))
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(1024, 4096, generator=g, dtype=torch.float32).numpy()
    plain = rel_fro(orc.newton_schulz(x, 5, "simple", precision="medium")[::16, ::16], rec["medium.sample"])
    deferred = rel_fro(orc.newton_schulz_deferred_norm(x, 5, "simple")[::16, ::16], rec["medium.sample"])
    assert deferred <= 1.2e-2 and deferred <= 1.1 * plain + 5e-4

    data = np.load(os.path.join(golden_dir, "ns_medium.npz"))
    cases = json.load(open(os.path.join(golden_dir, "ns_cases.json")))
    worst = 0.0
    for name, meta in cases.items():
        kw = dict(meta["kwargs"])
        if kw.pop("normalize_in_double", False):
            continue
        if "custom_coefficient_sets" in kw:
            kw["custom_coefficient_sets"] = [tuple(t) for t in kw["custom_coefficient_sets"]]
        assert data[f"{name}.x"][0].size < (1 << 22) if data[f"{name}.x"].ndim == 3 else data[f"{name}.x"].size < (1 << 22)
        worst = max(worst, rel_fro(orc.newton_schulz_deferred_norm(data[f"{name}.x"], **kw), data[f"{name}.y"]))
    assert worst > 2e-2  # below the threshold the reference's rounding points have to be kept


def test_muon_step_matches_reference(golden_dir):
    data = np.load(os.path.join(golden_dir, "muon_steps.npz"))
    with open(os.path.join(golden_dir, "muon_cases.json")) as f:
        meta = json.load(f)
    for name, kw in meta["cases"].items():
        kw = dict(kw)
        precision = kw.pop("fp32_matmul_prec", "medium")
        n = len(meta["shapes"])
        params = [data[f"{name}.p{i}.init"].copy() for i in range(n)]
        moms = [np.zeros_like(p) for p in params]
        for step in range(2):
            grads = [data[f"{name}.p{i}.grad{step}"] for i in range(n)]
            before = [p.copy() for p in params]
            orc.muon_step(params, grads, moms, precision=precision, **kw)
            for i in range(n):
                ref_after = data[f"{name}.p{i}.after{step}"]
                # Compare the applied update, not the parameter (the update is ~lr times smaller than p).
                upd, ref_upd = params[i] - before[i], ref_after - before[i]
                tol = 2e-2 if precision == "medium" else 1e-4
                assert rel_fro(upd, ref_upd) <= tol, (name, step, i, rel_fro(upd, ref_upd))
                assert rel_fro(moms[i], data[f"{name}.p{i}.mom{step}"]) <= 1e-6
                # Keep following the reference trajectory so that errors do not compound across steps.
                params[i][...] = ref_after
                moms[i][...] = data[f"{name}.p{i}.mom{step}"]


def test_tp_matches_reference(golden_dir):
    data = np.load(os.path.join(golden_dir, "ns_tp.npz"))
    x = data["x_full"]
    world = 2
    full = orc.newton_schulz(x, 5, "quintic")
    for pdim in (0, 1):
        src = x if pdim == 1 else np.ascontiguousarray(x.T)
        shards = np.array_split(src, world, axis=pdim)
        outs = orc.newton_schulz_tp_distributed(shards, 5, "quintic", pdim)
        full_p = full if pdim == 1 else full.T
        for r in range(world):
            assert rel_fro(outs[r], data[f"p{pdim}.distributed.rank{r}"]) <= 2e-5
            assert rel_fro(data[f"p{pdim}.duplicated.rank{r}"], np.array_split(full_p, world, axis=pdim)[r]) <= 2e-5


def test_bf16_round_is_round_to_nearest_even():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(0)
    x = np.concatenate(
        [rng.standard_normal(4096).astype(np.float32) * s for s in (1e-20, 1e-3, 1.0, 1e10)]
        + [np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, np.inf, -np.inf], dtype=np.float32)]
    )
    want = torch.from_numpy(x).bfloat16().float().numpy()
    assert np.array_equal(orc.bf16_round(x), want)


def test_integer_syrk_is_exact():
    rng = np.random.default_rng(1)
    a = rng.integers(-3, 4, size=(40, 24)).astype(np.float32)
    c = rng.integers(-3, 4, size=(40, 40)).astype(np.float32)
    c = c + c.T
    d = orc.syrk_ex(a, c, alpha=0.5, beta=0.25)
    assert np.array_equal(d, orc.bf16_round(0.5 * (a @ a.T) + 0.25 * c))
    assert np.array_equal(d, d.T)


@pytest.mark.parametrize("precision,tol", [("highest", 2e-5), ("medium", 1.2e-2)])
def test_torch_cpu_restatement_matches_reference(golden_dir, precision, tol):
    """The torch-operator restatement timed as the CPU baseline (oracle/ns_torch_cpu.py) against the reference's
    vectors; only the cases its reduced signature covers (preset schedules, default orientation and eps)."""
    torch = pytest.importorskip("torch")
    from oracle import ns_torch_cpu

    data = np.load(os.path.join(golden_dir, f"ns_{precision}.npz"))
    checked = 0
    for name, meta in _cases(golden_dir).items():
        kw = dict(meta["kwargs"])
        if set(kw) - {"steps", "coefficient_type"} or kw["coefficient_type"] == "custom":
            continue
        y = ns_torch_cpu.newton_schulz(torch.from_numpy(data[f"{name}.x"]), kw["steps"], kw["coefficient_type"], precision)
        ref = data[f"{name}.y"]
        assert tuple(y.shape) == ref.shape and y.dtype == torch.float32
        assert rel_fro(y.contiguous().numpy(), ref) <= tol, (name, rel_fro(y.contiguous().numpy(), ref))
        checked += 1
    assert checked >= 12
