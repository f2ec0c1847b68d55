"""The grouped fused Muon step on the GPU: its elementwise kernels against torch, the fused step against the
per-parameter step, and layer-parallel Muon against the single-process step (bitwise)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from emerging_optimizers_b200 import _native as nat
from emerging_optimizers_b200.distributed import LayerParallelMuon
from emerging_optimizers_b200.orthogonalized_optimizers import Muon, muon, muon_utils
from emerging_optimizers_b200.utils import fp32_matmul_precision
from tests._torch_ref import randn_tensor, rel_fro


pytestmark = pytest.mark.gpu

SHAPES = [(256, 256), (64, 256), (64, 256), (896, 256), (256, 896), (256, 256), (40, 24)]
KW = dict(lr=0.02, momentum=0.95, weight_decay=0.1, nesterov=True, weight_decay_method="decoupled",
          num_ns_steps=5, scale_mode="shape_scaling", coefficient_type="simple", fp32_matmul_prec="medium")  # fmt: skip


def _params(device="cuda"):
    return [torch.nn.Parameter(randn_tensor(*s, seed=50 + i, scale=0.02, device=device)) for i, s in enumerate(SHAPES)]


def _set_grads(params, step):
    for i, p in enumerate(params):
        p.grad = randn_tensor(*p.shape, seed=1000 * step + i, scale=1e-3, device=p.device).bfloat16().float()


@pytest.mark.parametrize("nesterov", [True, False])
@pytest.mark.parametrize("l2", [0.0, 0.05])
@pytest.mark.parametrize("numel_shape", [(64, 256), (13, 21), (1024, 1030)])
def test_elementwise_kernels_match_torch(nesterov, l2, numel_shape):
    g = randn_tensor(*numel_shape, seed=1, scale=1e-3)
    m = randn_tensor(*numel_shape, seed=2, scale=1e-3)
    p = randn_tensor(*numel_shape, seed=3, scale=0.02)
    mu = 0.95
    g_ref = g.add(p, alpha=l2) if l2 else g  # what WeightDecayMixin's l2 method does to the gradient
    m_ref = m.clone().lerp_(g_ref, 1 - mu)
    u_ref = g_ref.lerp(m_ref, mu) if nesterov else m_ref
    m_new = m.clone()
    ss = nat.muon_momentum(g, m_new, p, mu, nesterov, l2)
    assert torch.equal(m_new, m_ref)  # the momentum buffer is bit for bit what torch.lerp_ leaves
    assert torch.allclose(ss, (u_ref.double() ** 2).sum().reshape(1), rtol=1e-6)
    out = torch.empty(numel_shape, dtype=torch.bfloat16, device="cuda")
    nat.muon_normalize(g, m_new, p, mu, nesterov, l2, ss, 1e-15, out)
    want = (u_ref / u_ref.norm()).bfloat16()
    # one bf16 ulp where the quotient sits on a rounding boundary
    assert rel_fro(out.float(), want.float()) <= 2e-3
    # apply: p <- (p + shrink p) - lr ((u scale) extra)
    for u in (out, out.float()):
        p1 = p.clone()
        nat.muon_apply(p1, u, -0.002, 1.5, 0.2, 0.02)
        p_ref = p.clone()
        p_ref.add_(p_ref, alpha=-0.002)
        p_ref.add_(u.float() * 1.5 * 0.2, alpha=-0.02)
        assert torch.equal(p1, p_ref)
    assert nat.read_device_status() == 0


@pytest.mark.parametrize("method", ["decoupled", "independent", "palm", "l2"])
@pytest.mark.parametrize("use_syrk", [False, True])
def test_fused_step_equals_per_parameter_step(method, use_syrk, monkeypatch):
    kw = dict(KW, weight_decay_method=method)
    a, b = _params(), _params()
    fused, plain = Muon(a, use_syrk=use_syrk, **kw), Muon(b, use_syrk=use_syrk, **kw)
    assert fused._fused_step_applies()
    for step in range(3):
        _set_grads(a, step)
        _set_grads(b, step)
        fused.step()
        monkeypatch.setattr(muon, "FUSED_STEP", False)
        assert not plain._fused_step_applies()
        plain.step()
        monkeypatch.setattr(muon, "FUSED_STEP", True)
        for i, (pa, pb) in enumerate(zip(a, b)):
            # same arithmetic in a different launch structure; the applied update must agree to fp32 round-off
            assert torch.allclose(pa, pb, rtol=0, atol=2e-7), (step, i, float((pa - pb).abs().max()))
            assert torch.allclose(fused.state[pa]["momentum_buffer"], plain.state[pb]["momentum_buffer"], rtol=1e-6, atol=0)
    assert nat.read_device_status() == 0


def test_fused_step_not_used_when_customised(monkeypatch):
    class Sub(Muon):
        def orthogonalize(self, p, grad, **kwargs):
            return super().orthogonalize(p, grad, **kwargs)

    params = _params()
    assert not Sub(params, **KW)._fused_step_applies()
    assert not Muon(params, **dict(KW, fp32_matmul_prec="highest"))._fused_step_applies()
    opt = Muon(params, **KW)
    monkeypatch.setattr(muon_utils, "newton_schulz_step", lambda *a, **k: None)
    assert not opt._fused_step_applies()


def test_batch_composition_does_not_change_a_matrix_result():
    """A matrix orthogonalized alone (narrow tiles are chosen for a small problem) and inside a stack of 16 (wide
    tiles) must give the same bits: layer-parallel ownership changes the batch a matrix lands in."""
    x = randn_tensor(16, 1024, 4096, seed=60, scale=1e-3)
    with fp32_matmul_precision("medium"):
        yb = muon_utils.newton_schulz(x, 5, "simple", use_syrk=True)
        for i in (0, 7, 15):
            assert torch.equal(yb[i], muon_utils.newton_schulz(x[i], 5, "simple", use_syrk=True))
            assert torch.equal(yb[i], muon_utils.newton_schulz(x[i : i + 1], 5, "simple", use_syrk=True)[0])


def test_layer_parallel_single_rank_equals_muon_bitwise():
    a, b = _params(), _params()
    ref, lp = Muon(a, use_syrk=True, **KW), LayerParallelMuon(b, use_syrk=True, **KW)
    for step in range(2):
        _set_grads(a, step)
        _set_grads(b, step)
        ref.step()
        lp.step()
        for pa, pb in zip(a, b):
            assert torch.equal(pa, pb)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _lp_worker(rank, world, port, out, exchange="updates"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    dev = f"cuda:{rank}"
    params = _params(dev)
    opt = LayerParallelMuon(params, use_syrk=True, bucket_numel=100_000, exchange=exchange, **KW)
    for step in range(2):
        _set_grads(params, step)
        opt.step()
    torch.cuda.synchronize()
    out[rank] = {"params": [p.detach().cpu() for p in params], "owned": opt.owned_indices(),
                 "status": nat.read_device_status(torch.device(dev))}  # fmt: skip
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("exchange", ["updates", "parameters", "mixed"])
def test_layer_parallel_two_gpus_equals_single_process_bitwise(exchange):
    world = 2
    ref_params = _params()
    ref = Muon(ref_params, use_syrk=True, **KW)
    for step in range(2):
        _set_grads(ref_params, step)
        ref.step()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_lp_worker, args=(world, _free_port(), out, exchange), nprocs=world, join=True)
        results = dict(out)
    assert sorted(results[0]["owned"] + results[1]["owned"]) == list(range(len(SHAPES)))
    for r in range(world):
        assert results[r]["status"] == 0
        for i, p in enumerate(ref_params):
            assert torch.equal(results[r]["params"][i], p.detach().cpu()), (r, i)


def test_per_head_muon_subclass_pattern():
    """The reference's recipe for per-head / split-QKV orthogonalization (examples/per-head-muon.ipynb and the
    docstring at orthogonalized_optimizer.py:68-87 there): a Muon subclass overrides ``orthogonalize``, views the
    (heads * d, n) gradient as (heads, d, n) and orthogonalizes every head on its own - here one batched call that
    lands on the fused small-matrix kernel.  It must equal orthogonalizing each head separately."""
    heads, d, n = 6, 128, 512

    class PerHeadMuon(Muon):
        def orthogonalize(self, p, grad, **kwargs):
            out = self.scaled_orthogonalize_fn(grad.view(heads, d, n))
            return out.reshape(heads * d, n)

    kw = dict(KW, scale_mode="spectral")
    w = randn_tensor(heads * d, n, seed=70, scale=0.02)
    g = randn_tensor(heads * d, n, seed=71, scale=1e-3).bfloat16().float()
    p = torch.nn.Parameter(w.clone())
    p.grad = g.clone()
    opt = PerHeadMuon([p], use_syrk=True, **kw)
    assert not opt._fused_step_applies()  # customised: the per-parameter path is taken
    opt.step()

    # the same step written out head by head
    mom = torch.zeros_like(w).lerp_(g, 1 - kw["momentum"])
    upd = g.lerp(mom, kw["momentum"])
    want = w.clone()
    want.add_(want, alpha=-kw["weight_decay"] * kw["lr"])
    with fp32_matmul_precision("medium"):
        per_head = torch.cat(
            [muon_utils.newton_schulz(upd[h * d : (h + 1) * d], 5, "simple", use_syrk=True) for h in range(heads)]
        )
    scale = max(d, n) ** 0.5  # "spectral" scale from the size of one head, not of the fused parameter
    want.add_(per_head * scale * 1.0, alpha=-kw["lr"])
    assert torch.equal(p.detach(), want)
    assert nat.read_device_status() == 0


def test_fused_step_with_deferred_normalisation_on_large_matrices(monkeypatch):
    """Matrices of 2^22 elements and more go through the one-pass prepare kernel (momentum update + un-normalised
    bf16 update + sum of squares) and take their 1 / norm factors in the first two epilogues of the iteration.
    Momentum buffers are the same bits as with the two-pass form; the weights agree with it within what one bf16
    rounding of the first iterate moves them, and with the library-GEMM restatement of the step."""
    shapes = [(1024, 4096), (1024, 4096), (4096, 1024)]

    def make():
        return [torch.nn.Parameter(randn_tensor(*s, seed=90 + i, scale=0.02, device="cuda")) for i, s in enumerate(shapes)]

    def grads(ps, step):
        for i, p in enumerate(ps):
            p.grad = randn_tensor(*p.shape, seed=2000 * (step + 1) + i, scale=1e-3, device="cuda").bfloat16().float()

    a, b = make(), make()
    p0 = [p.detach().clone() for p in a]
    deferred, two_pass = Muon(a, use_syrk=True, **KW), Muon(b, use_syrk=True, **KW)
    for step in range(2):
        grads(a, step)
        grads(b, step)
        deferred.step()
        monkeypatch.setattr(muon_utils, "FOLD_NORMALIZATION_MIN_NUMEL", 0)
        two_pass.step()
        monkeypatch.undo()
        for pa, pb in zip(a, b):
            assert torch.equal(deferred.state[pa]["momentum_buffer"], two_pass.state[pb]["momentum_buffer"])
    for pa, pb, q in zip(a, b, p0):
        # compare the accumulated updates, not the weights (which are dominated by their initial values)
        ua, ub = pa.detach() - q * (1 - KW["lr"] * KW["weight_decay"]) ** 2, pb.detach() - q * (1 - KW["lr"] * KW["weight_decay"]) ** 2
        assert not torch.equal(pa, pb)
        assert float((ua - ub).norm() / ub.norm()) <= 2e-2
    assert nat.read_device_status() == 0
