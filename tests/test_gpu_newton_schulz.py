"""Newton-Schulz and Muon on the GPU against the reference's golden vectors, the numpy oracle and, at full size,
a library-GEMM restatement of the reference arithmetic.

Tolerances (relative Frobenius error of the result): 2e-2 on the bf16 ("medium") path, 1e-4 on the fp32 path,
except where a comment says why a case needs more.
"""

import json
import os

import numpy as np
import pytest
import torch

from emerging_optimizers_b200 import _native as nat
from emerging_optimizers_b200.orthogonalized_optimizers import Muon, muon_utils
from emerging_optimizers_b200.utils import fp32_matmul_precision
from oracle import ns_oracle as orc
from tests._torch_ref import int_tensor, newton_schulz_torch, randn_tensor, rel_fro


pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2
FP32_TOL = 1e-4


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert nat.read_device_status() == 0


def _golden_cases(golden_dir):
    with open(os.path.join(golden_dir, "ns_cases.json")) as f:
        cases = json.load(f)
    for kw in cases.values():
        if "custom_coefficient_sets" in kw["kwargs"]:
            kw["kwargs"]["custom_coefficient_sets"] = [tuple(t) for t in kw["kwargs"]["custom_coefficient_sets"]]
    return cases


@pytest.mark.parametrize("use_syrk", [False, True])
def test_bf16_path_matches_reference_golden(golden_dir, use_syrk):
    data = np.load(os.path.join(golden_dir, "ns_medium.npz"))
    for name, meta in _golden_cases(golden_dir).items():
        x = torch.from_numpy(data[f"{name}.x"]).cuda()
        with fp32_matmul_precision("medium"):
            y = muon_utils.newton_schulz(x, use_syrk=use_syrk, **meta["kwargs"])
        assert y.dtype == torch.float32 and tuple(y.shape) == tuple(x.shape)
        err = rel_fro(y.cpu(), torch.from_numpy(data[f"{name}.y"]))
        assert err <= BF16_TOL, (name, err)


@pytest.mark.parametrize("precision", ["highest", "high"])
def test_fp32_path_matches_reference_golden(golden_dir, precision):
    data = np.load(os.path.join(golden_dir, "ns_highest.npz"))
    for name, meta in _golden_cases(golden_dir).items():
        x = torch.from_numpy(data[f"{name}.x"]).cuda()
        with fp32_matmul_precision(precision):
            y = muon_utils.newton_schulz(x, **meta["kwargs"])
        err = rel_fro(y.cpu(), torch.from_numpy(data[f"{name}.y"]))
        assert err <= FP32_TOL, (name, err)


def test_config1_against_reference(golden_dir):
    """BASELINE config 1: 1024 x 4096 N(0,1) seed 0, five "simple" steps."""
    rec = np.load(os.path.join(golden_dir, "config1.npz"))
    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn(1024, 4096, generator=g, dtype=torch.float32)
    assert float(x.double().sum()) == pytest.approx(float(rec["x_sum"]), rel=1e-12)
    xg = x.cuda()
    # fp32 bound 1e-4 against the reference's stored CPU fp32 result.  Measured 9.1e-5, nearly all of it the
    # reference's own distance from a float64 run of the same steps (8.8e-5; the kernels are 1.3e-5 from it, see
    # tests/test_gpu_reference_edge_cases.py).
    for precision, tol, use_syrk in (("highest", 1e-4, False), ("medium", BF16_TOL, True), ("medium", BF16_TOL, False)):
        with fp32_matmul_precision(precision):
            y = muon_utils.newton_schulz(xg, 5, "simple", use_syrk=use_syrk)
        err = rel_fro(y[::16, ::16].cpu(), torch.from_numpy(rec[f"{precision}.sample"]))
        assert err <= tol, (precision, err)
        sv = torch.linalg.svdvals(y.double())
        lo, hi = float(rec[f"{precision}.sv_min"]), float(rec[f"{precision}.sv_max"])
        slack = tol * max(1.0, hi)
        assert float(sv.min()) >= lo - slack and float(sv.max()) <= hi + slack, (precision, float(sv.min()), float(sv.max()))
        assert float(y.double().norm()) == pytest.approx(float(rec[f"{precision}.fro"]), rel=5e-3)


def test_oracle_agrees_on_seeded_inputs():
    for shape, ctype, steps in (((256, 512), "quintic", 5), ((512, 256), "polar_express", 8), ((4, 128, 384), "simple", 5)):
        x = randn_tensor(*shape, seed=31, scale=1e-3)
        with fp32_matmul_precision("medium"):
            y = muon_utils.newton_schulz(x, steps, ctype, use_syrk=True)
        want = orc.newton_schulz(x.cpu().numpy(), steps, ctype, precision="medium")
        assert rel_fro(y.cpu(), torch.from_numpy(want)) <= BF16_TOL
        with fp32_matmul_precision("highest"):
            y = muon_utils.newton_schulz(x, steps, ctype)
        want = orc.newton_schulz(x.cpu().numpy(), steps, ctype, precision="highest")
        assert rel_fro(y.cpu(), torch.from_numpy(want)) <= FP32_TOL


def test_syrk_step_equals_gemm_step_bitwise_on_integers():
    """Small integers and power-of-two coefficients make every bf16 product exact (the reference's own trick,
    tests/test_muon_utils.py:503-524 there)."""
    x = int_tensor(128, 256, seed=32, lo=-1, hi=2)
    a, b, c = 2**-1, 2**-2, 2**-3
    got_gemm = muon_utils.newton_schulz_step(x, a, b, c)
    got_syrk = muon_utils.newton_schulz_step_tsyrk(x, a, b, c)
    A = x.float() @ x.float().T
    B = (b * A + c * (A @ A)).bfloat16().float()
    want = (a * x.float() + B @ x.float()).bfloat16()
    assert torch.equal(got_gemm, got_syrk)
    assert torch.equal(got_gemm, want)
    xb = int_tensor(3, 128, 256, seed=33, lo=-1, hi=2)
    assert torch.equal(
        muon_utils.batched_newton_schulz_step(xb, a, b, c), muon_utils.batched_newton_schulz_step_tsyrk(xb, a, b, c)
    )
    # cubic path (c == 0): X' = a X + b A X
    got = muon_utils.newton_schulz_step(x, a, b, 0.0)
    assert torch.equal(got, (a * x.float() + b * (A.bfloat16().float() @ x.float())).bfloat16())


def test_batched_equals_per_matrix_bitwise():
    x = randn_tensor(5, 128, 320, seed=34)
    with fp32_matmul_precision("medium"):
        yb = muon_utils.newton_schulz(x, 5, "quintic", use_syrk=True)
        for i in range(x.size(0)):
            assert torch.equal(yb[i], muon_utils.newton_schulz(x[i], 5, "quintic", use_syrk=True))


def test_tall_input_equals_transposed_wide_input():
    x = randn_tensor(640, 256, seed=35)
    with fp32_matmul_precision("medium"):
        y_tall = muon_utils.newton_schulz(x, 5, "quintic", use_syrk=True)
        y_wide = muon_utils.newton_schulz(x.T.contiguous(), 5, "quintic", use_syrk=True)
    assert tuple(y_tall.shape) == (640, 256)
    assert torch.equal(y_tall, y_wide.T)


def test_polar_express_16_steps_is_orthogonal():
    x = randn_tensor(128, 256, seed=36)
    with fp32_matmul_precision("highest"):
        o = muon_utils.newton_schulz(x, 16, "polar_express")
    eye = torch.eye(128, device="cuda", dtype=torch.float64)
    assert float((o.double() @ o.double().T - eye).abs().max()) <= 1e-4


def test_steps_zero_returns_normalised_input():
    x = randn_tensor(64, 96, seed=37)
    with fp32_matmul_precision("highest"):
        y = muon_utils.newton_schulz(x, 0, "simple")
    assert torch.allclose(y, x / x.norm(), rtol=1e-6, atol=0)
    assert y.data_ptr() != x.data_ptr()


def test_replaced_step_function_is_used():
    calls = []
    orig = muon_utils.newton_schulz_step_tsyrk

    def spy(X, a, b, c, tp_group=None):
        calls.append(X.dtype)
        return orig(X, a, b, c, tp_group=tp_group)

    muon_utils.newton_schulz_step_tsyrk = spy
    try:
        x = randn_tensor(64, 128, seed=38)
        with fp32_matmul_precision("medium"):
            y = muon_utils.newton_schulz(x, 3, "simple", use_syrk=True)
            # 13 x 21 is not TMA-aligned: the SYRK step functions are skipped, as in the reference
            muon_utils.newton_schulz(randn_tensor(13, 21, seed=39), 3, "simple", use_syrk=True)
    finally:
        muon_utils.newton_schulz_step_tsyrk = orig
    assert calls == [torch.bfloat16] * 3
    with fp32_matmul_precision("medium"):
        assert torch.equal(y, muon_utils.newton_schulz(x, 3, "simple", use_syrk=True))


@pytest.mark.parametrize("shape", [(256, 640), (640, 256), (3, 128, 384), (2, 384, 128), (256, 256)])
@pytest.mark.parametrize("ctype,steps", [("quintic", 5), ("cubic5", 5), ("polar_express", 1)])
def test_single_call_loop_equals_step_by_step_bitwise(shape, ctype, steps):
    """The one-call iteration loop of the library against the same kernels driven step by step from Python
    (selected here by wrapping a step function, which is how a caller opts out of the single call)."""
    x = randn_tensor(*shape, seed=40)
    names = ["newton_schulz_step", "batched_newton_schulz_step", "newton_schulz_step_tsyrk", "batched_newton_schulz_step_tsyrk"]
    for use_syrk in (False, True):
        with fp32_matmul_precision("medium"):
            fast = muon_utils.newton_schulz(x, steps, ctype, use_syrk=use_syrk)
            saved = {n: getattr(muon_utils, n) for n in names}
            try:
                for n, fn in saved.items():
                    setattr(muon_utils, n, (lambda f: lambda X, a, b, c, tp_group=None: f(X, a, b, c, tp_group=tp_group))(fn))
                slow = muon_utils.newton_schulz(x, steps, ctype, use_syrk=use_syrk)
            finally:
                for n, fn in saved.items():
                    setattr(muon_utils, n, fn)
        assert fast.shape == slow.shape and torch.equal(fast, slow)


@pytest.mark.parametrize("shape", [(256, 640), (640, 256), (3, 128, 384), (2, 384, 128), (13, 21), (2, 21, 13)])
@pytest.mark.parametrize("ctype,steps", [("simple", 5), ("cubic5", 5), ("polar_express", 2), ("quintic", 1)])
def test_fp32_single_call_loop_equals_step_by_step_bitwise(shape, ctype, steps):
    """The same for the fp32 path: the library's one-call loop issues the kernels the step functions issue."""
    x = randn_tensor(*shape, seed=41)
    names = ["newton_schulz_step", "batched_newton_schulz_step"]
    with fp32_matmul_precision("highest"):
        n0 = nat.launch_count
        fast = muon_utils.newton_schulz(x, steps, ctype)
        per_call = nat.launch_count - n0
        saved = {n: getattr(muon_utils, n) for n in names}
        try:
            for n, fn in saved.items():
                setattr(muon_utils, n, (lambda f: lambda X, a, b, c, tp_group=None: f(X, a, b, c, tp_group=tp_group))(fn))
            n0 = nat.launch_count
            slow = muon_utils.newton_schulz(x, steps, ctype)
            per_step = nat.launch_count - n0
        finally:
            for n, fn in saved.items():
                setattr(muon_utils, n, fn)
    assert fast.shape == slow.shape and fast.dtype == torch.float32 and torch.equal(fast, slow)
    assert per_call == per_step  # same kernels, counted the same way
    assert nat.read_device_status() == 0


@pytest.mark.parametrize("shape", [(511, 513), (511, 257), (257, 513)])
def test_fp32_path_elementwise_on_powers_of_two(shape):
    """The construction of the reference's tightest Newton-Schulz test (tests/test_muon_utils.py:182-210): entries
    that are powers of two, odd sizes, integer custom coefficients, two steps.  Every term is positive, so there is
    no cancellation and the comparison can be elementwise and purely relative (atol 0).  The reference holds its
    fp32 GEMMs to rtol 1e-6 there; the split-bf16 products accumulate in the tensor cores' fp32 adders and are held
    to 1e-5 against a float64 restatement."""
    g = torch.Generator(device="cpu").manual_seed(50)
    x = (2.0 ** torch.randint(-10, -5, shape, generator=g).float()).cuda()
    sets = [(3.0, 5.0, 7.0), (11.0, 13.0, 17.0)]
    with fp32_matmul_precision("highest"):
        y = muon_utils.newton_schulz(x, steps=2, coefficient_type="custom", custom_coefficient_sets=sets)
    X = x.double()
    if shape[0] > shape[1]:
        X = X.mT
    X = X / X.norm()
    for a, b, c in sets:
        A = X @ X.mT
        X = a * X + (b * A + c * A @ A) @ X
    if shape[0] > shape[1]:
        X = X.mT
    rel = ((y.double() - X).abs() / X.abs()).max().item()
    assert rel <= 1e-5, rel
    assert nat.read_device_status() == 0


@pytest.mark.parametrize("shape", [(1024, 4096), (4096, 512), (640, 2048), (256, 8192)])
def test_fp32_k_split_gram_agrees_with_step_by_step(shape):
    """A single small matrix: the one-call fp32 loop slices the contraction dimension of the Gram product across
    CTAs and sums the partial matrices in fp32; the step functions do not.  Same products, different summation
    order, so agreement to fp32 round-off (amplified by five "simple" steps) rather than bit for bit."""
    x = randn_tensor(*shape, seed=42)
    names = ["newton_schulz_step", "batched_newton_schulz_step"]
    with fp32_matmul_precision("highest"):
        fast = muon_utils.newton_schulz(x, 5, "simple")
        saved = {n: getattr(muon_utils, n) for n in names}
        try:
            for n, fn in saved.items():
                setattr(muon_utils, n, (lambda f: lambda X, a, b, c, tp_group=None: f(X, a, b, c, tp_group=tp_group))(fn))
            slow = muon_utils.newton_schulz(x, 5, "simple")
        finally:
            for n, fn in saved.items():
                setattr(muon_utils, n, fn)
    assert rel_fro(fast, slow) <= 2e-5, rel_fro(fast, slow)
    assert nat.read_device_status() == 0


@pytest.mark.parametrize(
    "shape", [(4, 128, 512), (3, 64, 1024), (2, 128, 8192), (5, 120, 520), (128, 4096), (300, 128, 256), (1, 8, 256)]
)
@pytest.mark.parametrize("ctype,steps", [("simple", 5), ("cubic5", 5), ("polar_express", 1), ("quintic", 2)])
def test_fused_small_matrix_kernel_equals_general_kernels(shape, ctype, steps, monkeypatch):
    """Matrices with at most 128 rows run all iterations in one persistent kernel that keeps A, A^2 and S in shared
    memory; same products, same rounding points, so the result must equal the general kernels' bit for bit."""
    x = randn_tensor(*shape, seed=41, scale=1e-3)
    with fp32_matmul_precision("medium"):
        fused = muon_utils.newton_schulz(x, steps, ctype, use_syrk=True)
        monkeypatch.setattr(nat, "FUSED_SMALL_MATRICES", False)
        general = muon_utils.newton_schulz(x, steps, ctype, use_syrk=True)
    assert fused.dtype == torch.float32 and fused.shape == general.shape
    assert torch.equal(fused, general)
    ref = newton_schulz_torch(x, steps, ctype, bf16=True)
    assert rel_fro(fused, ref) <= BF16_TOL


def test_muon_steps_match_reference_golden(golden_dir):
    data = np.load(os.path.join(golden_dir, "muon_steps.npz"))
    with open(os.path.join(golden_dir, "muon_cases.json")) as f:
        meta = json.load(f)
    n = len(meta["shapes"])
    for name, kw in meta["cases"].items():
        tol = BF16_TOL if kw.get("fp32_matmul_prec", "medium") == "medium" else FP32_TOL
        for use_syrk in (False, True):
            params = [torch.nn.Parameter(torch.from_numpy(data[f"{name}.p{i}.init"]).cuda()) for i in range(n)]
            opt = Muon(params, use_syrk=use_syrk, **kw)
            assert opt.use_syrk == use_syrk
            for step in range(2):
                before = [p.detach().clone() for p in params]
                for i, p in enumerate(params):
                    p.grad = torch.from_numpy(data[f"{name}.p{i}.grad{step}"]).cuda()
                opt.step()
                for i, p in enumerate(params):
                    ref_after = torch.from_numpy(data[f"{name}.p{i}.after{step}"]).cuda()
                    err = rel_fro(p.detach() - before[i], ref_after - before[i])
                    assert err <= tol, (name, step, i, err)
                    mom = opt.state[p]["momentum_buffer"]
                    assert rel_fro(mom, torch.from_numpy(data[f"{name}.p{i}.mom{step}"]).cuda()) <= 1e-6
                    # follow the reference trajectory so that step 1 starts from identical state
                    p.data.copy_(ref_after)
                    mom.copy_(torch.from_numpy(data[f"{name}.p{i}.mom{step}"]).cuda())


@pytest.mark.parametrize("shape", [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336)])
def test_llama_layer_shapes_against_library_gemm_restatement(shape):
    """BASELINE config 3 matrix shapes (gradients ~ N(0, 1e-3) rounded to bf16), bf16 path, SYRK kernels, compared
    with the same arithmetic done by library GEMMs on the same device."""
    x = randn_tensor(*shape, seed=2, scale=1e-3).bfloat16().float()
    with fp32_matmul_precision("medium"):
        y = muon_utils.newton_schulz(x, 5, "simple", use_syrk=True)
    ref = newton_schulz_torch(x, 5, "simple", bf16=True)
    assert rel_fro(y, ref) <= BF16_TOL
    # the reference's singular-value band for five "simple" steps (about [0.68, 1.14]) via the Gram matrix
    g = y.T @ y if shape[0] > shape[1] else y @ y.T
    ev = torch.linalg.eigvalsh(g.double())
    ev_ref = torch.linalg.eigvalsh((ref.T @ ref if shape[0] > shape[1] else ref @ ref.T).double())
    assert float(ev.min().clamp_min(0).sqrt()) >= float(ev_ref.min().clamp_min(0).sqrt()) - 2e-2
    assert float(ev.max().sqrt()) <= float(ev_ref.max().sqrt()) + 2e-2


def test_config4_single_device_full_size():
    """BASELINE config 4 on one device: 8192 x 28672, N(0,1) seed 3, five "simple" steps on the bf16 path."""
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(8192, 28672, generator=g, device="cuda", dtype=torch.float32)
    with fp32_matmul_precision("medium"):
        y = muon_utils.newton_schulz(x, 5, "simple", use_syrk=True)
    ref = newton_schulz_torch(x, 5, "simple", bf16=True)
    assert rel_fro(y, ref) <= BF16_TOL
    del ref
    # size-independent property: Y Y^T has its spectrum inside the five-"simple"-step band squared
    gram = y @ y.T
    ev = torch.linalg.eigvalsh(gram.double())
    assert 0.6**2 <= float(ev.min()) and float(ev.max()) <= 1.2**2


def test_config5_per_head_batch():
    """BASELINE config 5 per-device slice, reduced batch: (B, 128, 8192) heads, N(0, 1e-3), five "simple" steps."""
    x = randn_tensor(80, 128, 8192, seed=4, scale=1e-3).bfloat16().float()
    with fp32_matmul_precision("medium"):
        y = muon_utils.newton_schulz(x, 5, "simple", use_syrk=True)
    ref = newton_schulz_torch(x, 5, "simple", bf16=True)
    per_head = ((y - ref).double().flatten(1).norm(dim=1) / ref.double().flatten(1).norm(dim=1)).max()
    assert float(per_head) <= BF16_TOL
    want = orc.newton_schulz(x[:2].cpu().numpy(), 5, "simple", precision="medium")
    assert rel_fro(y[:2].cpu(), torch.from_numpy(want)) <= BF16_TOL


@pytest.mark.parametrize("shape", [(1024, 4096), (4096, 1024), (2, 1024, 4096)])
def test_deferred_normalisation_is_exact_when_the_norm_is_a_power_of_two(shape, monkeypatch):
    """Large matrices skip the normalisation pass: bf16(x) is iterated and 1 / |x|^2, 1 / |x| are applied in the first
    two epilogues.  With entries +-1 and 2^22 of them per matrix the norm is 2^11, every scaling is exact, and the
    result must equal the normalise-first path bit for bit."""
    g = torch.Generator(device="cpu").manual_seed(80)
    x = (torch.randint(0, 2, shape, generator=g).float() * 2 - 1).cuda()
    for use_syrk in (False, True):
        with fp32_matmul_precision("medium"):
            folded = muon_utils.newton_schulz(x, 5, "simple", use_syrk=use_syrk)
            monkeypatch.setattr(muon_utils, "FOLD_NORMALIZATION_MIN_NUMEL", 0)
            plain = muon_utils.newton_schulz(x, 5, "simple", use_syrk=use_syrk)
            monkeypatch.undo()
        assert torch.equal(folded, plain)
    assert nat.read_device_status() == 0


def test_deferred_normalisation_stays_within_the_bf16_tolerance_on_random_input(monkeypatch):
    """Against the library-GEMM restatement (which rounds the first iterate where the normalise-first path does, so
    that path agrees with it more closely by construction) both stay within the bf16 tolerance; against the fp32
    path of the same call, which favours neither, the two are equally accurate."""
    x = randn_tensor(2048, 4096, seed=81)
    for ctype, steps in (("simple", 5), ("quintic", 5), ("cubic5", 5), ("polar_express", 1)):
        with fp32_matmul_precision("medium"):
            folded = muon_utils.newton_schulz(x, steps, ctype, use_syrk=True)
            monkeypatch.setattr(muon_utils, "FOLD_NORMALIZATION_MIN_NUMEL", 0)
            plain = muon_utils.newton_schulz(x, steps, ctype, use_syrk=True)
            monkeypatch.undo()
        with fp32_matmul_precision("highest"):
            exact = muon_utils.newton_schulz(x, steps, ctype)
        ref = newton_schulz_torch(x, steps, ctype, bf16=True)
        assert not torch.equal(folded, plain)  # the first iterate is rounded at a different point ...
        assert rel_fro(folded, ref) <= BF16_TOL and rel_fro(plain, ref) <= BF16_TOL
        assert rel_fro(folded, exact) <= 1.25 * rel_fro(plain, exact) + 5e-4  # ... with the same accuracy
    assert nat.read_device_status() == 0


def test_deferred_normalisation_in_the_per_head_kernel(monkeypatch):
    """Stacks of 128 x 8192 heads (2^20 elements each) skip the normalisation pass too: exact with a power-of-two
    norm, and as close to the library-GEMM restatement as the normalise-first path on random input."""
    g = torch.Generator(device="cpu").manual_seed(82)
    ones = (torch.randint(0, 2, (3, 128, 8192), generator=g).float() * 2 - 1).cuda()  # norm 2^10 per head
    x = randn_tensor(6, 128, 8192, seed=83, scale=1e-3)
    with fp32_matmul_precision("medium"):
        folded_ones = muon_utils.newton_schulz(ones, 5, "simple", use_syrk=True)
        folded = muon_utils.newton_schulz(x, 5, "quintic", use_syrk=True)
        monkeypatch.setattr(muon_utils, "FOLD_NORMALIZATION_MIN_NUMEL", 0)
        plain_ones = muon_utils.newton_schulz(ones, 5, "simple", use_syrk=True)
        plain = muon_utils.newton_schulz(x, 5, "quintic", use_syrk=True)
        monkeypatch.undo()
    assert torch.equal(folded_ones, plain_ones)
    assert not torch.equal(folded, plain)
    for i in range(x.size(0)):
        ref = newton_schulz_torch(x[i], 5, "quintic", bf16=True)
        assert rel_fro(folded[i], ref) <= BF16_TOL and rel_fro(plain[i], ref) <= BF16_TOL
    assert nat.read_device_status() == 0


def test_status_mirror_makes_an_earlier_failure_loud():
    """The mirror of the status word is refreshed by every call; a non-zero value raises at the next call once."""
    from emerging_optimizers_b200 import _native as nat

    x = randn_tensor(512, 1024, seed=5)
    with fp32_matmul_precision("medium"):
        muon_utils.newton_schulz(x, steps=2, coefficient_type="simple")
        torch.cuda.synchronize()
        mirror = nat._STATUS_MIRRORS[x.device.index]
        assert int(mirror[0]) == 0  # the call left a fresh copy of a clean status word
        mirror[0] = 0x11  # what the copy would hold after a kernel gave up a wait
        with pytest.raises(nat.NativeLibraryError, match="0x11"):
            muon_utils.newton_schulz(x, steps=2, coefficient_type="simple")
        y = muon_utils.newton_schulz(x, steps=2, coefficient_type="simple")  # raised once, works again
    assert torch.isfinite(y).all()


def test_deferred_normalisation_matches_its_cpu_statement():
    """From 2^22 elements the kernels defer the normalisation; the oracle states that variant on the CPU with the
    same rounding points.  What is left between the two is the fp32 summation order, which five "simple" steps on
    bf16 operands amplify to about half a percent (the same distance as between these kernels and library GEMMs)."""
    x = randn_tensor(2048, 4096, seed=77)
    assert x.numel() >= muon_utils.FOLD_NORMALIZATION_MIN_NUMEL
    with fp32_matmul_precision("medium"):
        y = muon_utils.newton_schulz(x, 5, "simple", use_syrk=True)
    want = orc.newton_schulz_deferred_norm(x.cpu().numpy(), 5, "simple")
    err = rel_fro(y, torch.from_numpy(want).cuda())
    print(f"kernels vs CPU statement of the deferred normalisation: {err:.3e}")
    assert err <= 1e-2
