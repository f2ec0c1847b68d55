"""Parity of the CUDA kernels, called through the C ABI (ctypes), against the numpy oracle and, for integer-valued
inputs where bf16 products and fp32 sums are exact, bit for bit against fp32 matmul."""

import numpy as np
import pytest
import torch

from emerging_optimizers_b200 import _native as nat
from emerging_optimizers_b200 import triton_kernels as tk
from oracle import ns_oracle as orc
from tests._torch_ref import int_tensor, randn_tensor, rel_fro


pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert nat.read_device_status() == 0


def _exact_ref(a, c, alpha, beta):
    ref = alpha * (a.float() @ a.float().mT)
    if c is not None:
        ref = ref + beta * c.float()
    return ref.bfloat16()


@pytest.mark.parametrize(
    "n,k",
    [(8, 8), (128, 64), (136, 72), (256, 256), (384, 1024), (512, 256), (1000, 136), (2048, 1024), (2304, 192)],
)
@pytest.mark.parametrize("trans", [False, True])
def test_syrk_integer_inputs_bit_exact(n, k, trans):
    a = int_tensor(n, k, seed=n + k) if not trans else int_tensor(k, n, seed=n + k).T
    got = tk.tsyrk_ex(a)
    assert got.is_contiguous() and got.dtype == torch.bfloat16
    assert torch.equal(got, _exact_ref(a, None, 1.0, 0.0))
    assert torch.equal(got, got.T)


@pytest.mark.parametrize("n,k", [(128, 64), (520, 264), (1024, 512)])
@pytest.mark.parametrize("trans", [False, True])
def test_syrk_with_c_alpha_beta_bit_exact(n, k, trans):
    a = int_tensor(n, k, seed=1) if not trans else int_tensor(k, n, seed=1).T
    c = int_tensor(n, n, seed=2)
    c = (c + c.T).contiguous()
    for cc in (c, c.T):
        got = tk.tsyrk_ex(a, cc, alpha=2**-1, beta=2**-2)
        assert torch.equal(got, _exact_ref(a, c, 0.5, 0.25))
    out = torch.full((n, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ret = tk.tsyrk_ex_small_matrix(a, c, alpha=0.5, beta=0.25, out=out)
    assert ret is out and torch.equal(out, _exact_ref(a, c, 0.5, 0.25))


def test_syrk_skip_upper_leaves_upper_untouched():
    n, k = 520, 136
    a = int_tensor(n, k, seed=3)
    out = torch.full((n, n), -7.0, dtype=torch.bfloat16, device="cuda")
    tk.tsyrk_ex_small_matrix(a, skip_upper_triangle=True, out=out)
    ref = _exact_ref(a, None, 1.0, 0.0)
    assert torch.equal(torch.tril(out), torch.tril(ref))
    upper = torch.triu(torch.ones(n, n, dtype=torch.bool, device="cuda"), diagonal=1)
    assert bool((out[upper] == -7.0).all())


@pytest.mark.parametrize("batch,n,k", [(1, 128, 64), (3, 512, 256), (5, 136, 72), (7, 1032, 264)])
@pytest.mark.parametrize("trans", [False, True])
def test_batched_syrk_bit_exact(batch, n, k, trans):
    a = int_tensor(batch, n, k, seed=4) if not trans else int_tensor(batch, k, n, seed=4).mT
    c = int_tensor(batch, n, n, seed=5)
    c = (c + c.mT).contiguous()
    assert tk.can_use_batched_tsyrk(a, c)
    got = tk.batched_tsyrk_ex(a)
    assert torch.equal(got, _exact_ref(a, None, 1.0, 0.0))
    got = tk.batched_tsyrk_ex(a, c, alpha=0.25, beta=0.5)
    assert torch.equal(got, _exact_ref(a, c, 0.25, 0.5))
    assert torch.equal(got, got.mT)


def test_syrk_random_inputs_match_oracle():
    a = (randn_tensor(384, 1024, seed=6) / 32).bfloat16()
    c = randn_tensor(384, 384, seed=7)
    c = (c + c.T).bfloat16()
    got = tk.tsyrk_ex(a, c, alpha=1.5, beta=-0.75).float().cpu().numpy()
    want = orc.syrk_ex(a.float().cpu().numpy(), c.float().cpu().numpy(), alpha=1.5, beta=-0.75)
    # fp32 accumulation order differs from the oracle's BLAS: allow one bf16 ulp on isolated elements.
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= 2e-3
    assert np.array_equal(got, got.T)


@pytest.mark.parametrize("a_mn", [0, 1])
@pytest.mark.parametrize("b_mn", [0, 1])
@pytest.mark.parametrize("m,n,k,batch", [(128, 256, 64, 1), (200, 304, 72, 1), (256, 512, 1024, 3), (1024, 2048, 520, 1)])
def test_gemm_all_operand_layouts_bit_exact(a_mn, b_mn, m, n, k, batch):
    lead = (batch,) if batch > 1 else ()
    a = int_tensor(*lead, m, k, seed=8) if not a_mn else int_tensor(*lead, k, m, seed=8).mT
    b = int_tensor(*lead, k, n, seed=9) if b_mn else int_tensor(*lead, n, k, seed=9).mT
    c = int_tensor(*lead, m, n, seed=10)
    out = torch.empty(*lead, m, n, dtype=torch.bfloat16, device="cuda")
    nat.gemm(a, b, c, out, alpha=0.5, beta=0.25)
    ref = (0.5 * (a.float() @ b.float()) + 0.25 * c.float()).bfloat16()
    assert torch.equal(out, ref)
    out32 = torch.empty(*lead, m, n, dtype=torch.float32, device="cuda")
    nat.gemm(a, b, c, out32, alpha=0.5, beta=0.25, post_scale=3.0, round_bf16=True)
    assert torch.equal(out32, ref.float() * 3.0)


@pytest.mark.parametrize("tile_m", [128, 256])
def test_both_tile_heights_bit_exact(tile_m):
    """The launcher picks 128- or 256-row tiles per problem; both must give the same bits on every layout."""
    nat.set_option("gemm_tile_m", tile_m)
    try:
        for n, k, trans in ((256, 64, False), (1000, 136, False), (2048, 1024, True), (2304, 192, True)):
            a = int_tensor(n, k, seed=n) if not trans else int_tensor(k, n, seed=n).T
            c = int_tensor(n, n, seed=1)
            c = (c + c.T).contiguous()
            assert torch.equal(tk.tsyrk_ex(a, c, alpha=0.5, beta=0.25), _exact_ref(a, c, 0.5, 0.25))
        for m, n, k, a_mn, b_mn, batch in ((256, 256, 64, 0, 0, 1), (512, 768, 256, 0, 1, 1), (200, 304, 72, 1, 1, 1),
                                           (1024, 2048, 520, 1, 0, 1), (256, 512, 1024, 0, 1, 3)):  # fmt: skip
            lead = (batch,) if batch > 1 else ()
            a = int_tensor(*lead, m, k, seed=8) if not a_mn else int_tensor(*lead, k, m, seed=8).mT
            b = int_tensor(*lead, k, n, seed=9) if b_mn else int_tensor(*lead, n, k, seed=9).mT
            c = int_tensor(*lead, m, n, seed=10)
            out = torch.empty(*lead, m, n, dtype=torch.bfloat16, device="cuda")
            nat.gemm(a, b, c, out, alpha=0.5, beta=0.25)
            assert torch.equal(out, (0.5 * (a.float() @ b.float()) + 0.25 * c.float()).bfloat16())
        x = (randn_tensor(1024, 4096, seed=14) / 64).bfloat16()
        first = tk.tsyrk_ex(x)
        nat.set_option("gemm_tile_m", 128)
        assert torch.equal(first, tk.tsyrk_ex(x))  # same bits from either tile height
    finally:
        nat.set_option("gemm_tile_m", 0)


def test_config2_batched_syrk_full_size_properties():
    """BASELINE config 2 shape: 32 x (2048 x 8192), entries N(0, 1/8192) so that diag(A) is about 1."""
    g = torch.Generator(device="cuda").manual_seed(1)
    x = (torch.randn(32, 2048, 8192, generator=g, device="cuda") / 8192**0.5).bfloat16()
    a = tk.batched_tsyrk_ex(x)
    assert torch.equal(a, a.mT)
    # fp32-accumulated reference on a batch subset, tolerance 1e-2 relative as the config states
    for b in (0, 17, 31):
        ref = x[b].float() @ x[b].float().T
        assert rel_fro(a[b].float(), ref) <= 1e-2
        assert torch.allclose(a[b].float(), ref, rtol=1e-2, atol=1e-2)
    # size-independent check on every matrix: trace(A_b) = ||X_b||_F^2
    tr = a.float().diagonal(dim1=-2, dim2=-1).sum(-1)
    ss = (x.float() ** 2).sum(dim=(-2, -1))
    assert torch.allclose(tr, ss, rtol=2e-3)


@pytest.mark.parametrize("shape", [(1024, 4096), (3, 100, 36), (7, 13), (2, 64, 64)])
def test_sumsq_and_normalize_match_numpy(shape):
    x = randn_tensor(*shape, seed=11, scale=1e-3)
    ss = nat.sumsq(x).cpu().numpy()
    xn = x.cpu().numpy()
    want = (xn.astype(np.float64) ** 2).reshape(-1 if len(shape) == 2 else shape[0], *shape[-2:]).sum(axis=(-2, -1))
    assert np.allclose(ss, want.reshape(ss.shape), rtol=1e-12)
    y32 = nat.normalize(x, nat.sumsq(x), 1e-15, True, torch.float32).cpu().numpy()
    assert np.allclose(y32, orc.frobenius_normalize(xn), rtol=2e-7, atol=0)
    y16 = nat.normalize(x, nat.sumsq(x), 1e-15, True, torch.bfloat16).float().cpu().numpy()
    assert np.array_equal(y16, orc.bf16_round(y32))
    # a transposed view normalises to the transposed result
    yt = nat.normalize(x.mT, nat.sumsq(x.mT), 1e-15, True, torch.float32)
    assert torch.equal(yt.mT.contiguous().cpu(), torch.from_numpy(y32))


def test_normalize_eps_clamp_and_double_mode():
    x = torch.zeros(4, 8, device="cuda")
    y = nat.normalize(x, nat.sumsq(x), 1e-15, True, torch.float32)
    assert torch.equal(y, x)
    tiny = randn_tensor(8, 16, seed=12, scale=1e-25)
    ss = nat.sumsq(tiny)
    assert float(ss) > 0.0  # float64 accumulation: squares of 1e-25 do not underflow
    y = nat.normalize(tiny, ss, 1e-15, False, torch.float32).cpu().numpy()
    assert np.allclose(y, orc.frobenius_normalize(tiny.cpu().numpy(), in_double=True), rtol=1e-6)


def test_run_to_run_determinism():
    a = (randn_tensor(1024, 2048, seed=13) / 45).bfloat16()
    first = tk.tsyrk_ex(a)
    for _ in range(10):
        assert torch.equal(tk.tsyrk_ex(a), first)


@pytest.mark.parametrize("shape", [(256, 640), (640, 256), (100, 72)])
def test_kronecker_factor_update_matches_fp64(shape):
    """L <- lerp(L, G G^T, 1 - beta), R <- lerp(R, G^T G, 1 - beta): fp32 round-off against float64, symmetric."""
    from emerging_optimizers_b200.legacy_soap import update_kronecker_factors

    g = randn_tensor(*shape, seed=70)
    L0 = randn_tensor(shape[0], shape[0], seed=71)
    R0 = randn_tensor(shape[1], shape[1], seed=72)
    L0, R0 = L0 + L0.T, R0 + R0.T
    L, R = L0.clone(), R0.clone()
    update_kronecker_factors([L, R], g, 0.95)
    g64 = g.double()
    L_ref = 0.95 * L0.double() + 0.05 * (g64 @ g64.T)
    R_ref = 0.95 * R0.double() + 0.05 * (g64.T @ g64)
    assert rel_fro(L, L_ref) <= 2e-6 and rel_fro(R, R_ref) <= 2e-6
    assert torch.equal(L, L.T) and torch.equal(R, R.T)
    if shape[0] != shape[1]:
        with pytest.raises(ValueError, match="Kronecker factor must be"):
            update_kronecker_factors([R, L], g, 0.95)
    assert nat.read_device_status() == 0


@pytest.mark.parametrize("n", [64, 200, 512, 1000, 4096])
def test_mirror_of_the_lower_triangle(n):
    """eo_tp_gram_mirror (both of its kernels: 64 x 64 blocks with vector accesses, 32 x 32 blocks for odd sizes)."""
    ld = (n + 7) // 8 * 8
    g = torch.Generator(device="cpu").manual_seed(n)
    a = torch.randn(n, ld, generator=g).to(torch.bfloat16).cuda()
    want = torch.tril(a[:, :n]) + torch.tril(a[:, :n], -1).T
    nat.tp_gram_mirror(a, n, ld)
    assert torch.equal(a[:, :n], want)
    assert nat.read_device_status() == 0


@pytest.mark.parametrize(
    "m,n,k,tri,a_mn,b_mn",
    [
        (3072, 3328, 6144, False, 0, 0),  # 156 tiles on 74 CTA pairs: the last 8 are cut in two
        (3072, 3328, 24640, False, 0, 1),  # ... in eight, K not a multiple of the piece length
        (3000, 3304, 9216, False, 1, 1),  # ragged edges, three pieces
        (4352, 4352, 15360, True, 0, 0),  # SYRK: 153 lower-triangle tiles, the last 5 in five pieces
    ],
)
def test_split_tail_of_the_pair_kernel(m, n, k, tri, a_mn, b_mn):
    """Large products run on CTA pairs and split the K range of the tiles of their last, nearly empty round.

    Exact on integer-valued inputs; on random inputs equal to the unsplit kernel up to the rounding of the partial
    sums, the same bits for a batched launch as for per-matrix launches, and the same bits from run to run.
    """
    if tri:
        a = int_tensor(m, k, seed=21)
        c = int_tensor(m, m, seed=22)
        c = (c + c.T).contiguous()
        assert torch.equal(tk.tsyrk_ex(a, c, alpha=0.5, beta=0.25), _exact_ref(a, c, 0.5, 0.25))
        x = (randn_tensor(2, m, k, seed=23) / 8).bfloat16()
        run = lambda t: tk.batched_tsyrk_ex(t) if t.dim() == 3 else tk.tsyrk_ex(t)  # noqa: E731
    else:
        a = int_tensor(m, k, seed=21) if not a_mn else int_tensor(k, m, seed=21).mT
        b = int_tensor(k, n, seed=22) if b_mn else int_tensor(n, k, seed=22).mT
        c = int_tensor(m, n, seed=23)
        out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        nat.gemm(a, b, c, out, alpha=0.5, beta=0.25)
        assert torch.equal(out, (0.5 * (a.float() @ b.float()) + 0.25 * c.float()).bfloat16())
        x = (randn_tensor(2, m, k, seed=24) / 8).bfloat16()
        y = (randn_tensor(2, k, n, seed=25) / 8).bfloat16()

        def run(t):
            yy = y if t.dim() == 3 else y[0]
            o = torch.empty(*t.shape[:-1], n, dtype=torch.bfloat16, device="cuda")
            return nat.gemm(t, yy, None, o)

    both = run(x)
    one = run(x[0].contiguous())
    assert torch.equal(both[0], one)  # the split does not depend on the batch size
    assert torch.equal(run(x), both)  # nor on which CTA finishes a tile
    nat.set_option("gemm_split_k", 0)
    try:
        unsplit = run(x[0].contiguous())
    finally:
        nat.set_option("gemm_split_k", 1)
    assert rel_fro(one.float(), unsplit.float()) <= 2e-3  # both are bf16 roundings of nearly the same fp32 sums
    assert not torch.equal(one, unsplit)  # the split really happened: some roundings differ


def test_split_tail_on_two_streams_at_once():
    """The partial sums of the split tail live in a workspace per stream: products that overlap on two streams must
    not see each other's pieces."""
    xs = [(randn_tensor(4352, 15360, seed=40 + i) / 8).bfloat16() for i in range(2)]
    want = [tk.tsyrk_ex(x) for x in xs]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    got = [[], []]
    for _ in range(6):
        for i, s in enumerate(streams):
            with torch.cuda.stream(s):
                got[i].append(tk.tsyrk_ex(xs[i]))
    torch.cuda.synchronize()
    for i in range(2):
        for g in got[i]:
            assert torch.equal(g, want[i])
