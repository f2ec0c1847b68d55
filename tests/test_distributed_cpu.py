"""Host logic of the multi-rank paths on CPU: two gloo ranks, with the device kernels replaced by the oracle.

The package has no CPU compute path, so these tests inject one at the same seam the reference's own tests patch
(the module-level step functions and ``newton_schulz`` of ``muon_utils``): what is under test is the sharding,
ownership, collectives and bookkeeping around the kernels, not the kernels.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from emerging_optimizers_b200 import _native
from emerging_optimizers_b200.distributed import LayerParallelMuon, ns_cost, partition_by_cost
from emerging_optimizers_b200.distributed.layer_parallel import _plan_buckets
from emerging_optimizers_b200.orthogonalized_optimizers import Muon, muon_utils
from oracle import ns_oracle as orc


GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
WORLD = 2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_ns(x, steps, coefficient_type="quintic", custom_coefficient_sets=None, eps=1e-15, transpose=None,
            tp_group=None, use_syrk=False, normalize_in_double=False):  # fmt: skip
    """Oracle-backed stand-in for muon_utils.newton_schulz on CPU tensors (single device only)."""
    assert tp_group is None
    y = orc.newton_schulz(x.detach().numpy(), steps, coefficient_type, custom_coefficient_sets, eps, transpose,
                          torch.get_float32_matmul_precision(), normalize_in_double)  # fmt: skip
    return torch.from_numpy(np.ascontiguousarray(y))


def _cpu_normalize(x, eps, group, normalize_in_double, out_dtype):
    """muon_utils.py:132-146 of the reference with torch CPU ops (sum of squares, all-reduce, divide)."""
    xs = x.double() if normalize_in_double else x
    ss = (xs * xs).sum()
    if group is not None:
        dist.all_reduce(ss, op=dist.ReduceOp.SUM, group=group)
    norm = torch.sqrt(ss).to(x.dtype)
    if not normalize_in_double:
        norm.clamp_min_(eps)
    return (x / norm).to(out_dtype)


def _cpu_step(X, a, b, c, tp_group=None):
    """muon_utils.py:370-377 of the reference with torch CPU ops."""
    A = X @ X.mT
    if tp_group is not None:
        dist.all_reduce(A, op=dist.ReduceOp.SUM, group=tp_group)
    if c != 0.0:
        B = torch.addmm(A, A, A, alpha=c, beta=b)
        return torch.addmm(X, B, X, alpha=1.0, beta=a)
    return torch.addmm(X, A, X, alpha=b, beta=a)


def _patch_cpu_backend():
    muon_utils._normalize = _cpu_normalize
    for name in ("newton_schulz_step", "batched_newton_schulz_step", "newton_schulz_step_tsyrk",
                 "batched_newton_schulz_step_tsyrk"):  # fmt: skip
        setattr(muon_utils, name, _cpu_step)
    _native.require_cuda = lambda t, name="tensor": None


def _worker_tp(rank, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    torch.set_float32_matmul_precision("highest")
    _patch_cpu_backend()
    data = np.load(os.path.join(GOLDEN, "ns_tp.npz"))
    x = torch.from_numpy(data["x_full"])
    res = {}
    for pdim in (0, 1):
        src = x if pdim == 1 else x.mT.contiguous()
        shard = src.chunk(WORLD, dim=pdim)[rank].contiguous()
        for mode in ("distributed", "duplicated"):
            y = muon_utils.newton_schulz_tp(shard, 5, "quintic", dist.group.WORLD, partition_dim=pdim, tp_mode=mode)
            ref = torch.from_numpy(data[f"p{pdim}.{mode}.rank{rank}"])
            res[f"p{pdim}.{mode}"] = float((y - ref).norm() / ref.norm())
            assert tuple(y.shape) == tuple(shard.shape)
        # distributed_normalize_p2: every rank divides by the global norm
        z = muon_utils.distributed_normalize_p2(shard, 1e-15, dist.group.WORLD)
        res[f"p{pdim}.norm"] = float((z - shard / x.norm()).abs().max())
    # partition_dim=None must be the plain single-device call
    y = muon_utils.newton_schulz_tp(x, 5, "quintic", dist.group.WORLD)
    res["none"] = float((y - muon_utils.newton_schulz(x, 5, "quintic")).abs().max())
    out[rank] = res
    dist.destroy_process_group()


def test_newton_schulz_tp_two_ranks_matches_reference_golden():
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker_tp, args=(_free_port(), out), nprocs=WORLD, join=True)
        results = dict(out)
    assert sorted(results) == [0, 1]
    for rank, res in results.items():
        for key, err in res.items():
            assert err <= 2e-5, (rank, key, err)


SHAPES = [(32, 32), (8, 32), (48, 16), (16, 48), (24, 24), (8, 64), (40, 8)]
KW = dict(lr=0.02, momentum=0.95, weight_decay=0.1, nesterov=True, weight_decay_method="decoupled",
          num_ns_steps=5, scale_mode="shape_scaling", coefficient_type="simple", fp32_matmul_prec="medium")  # fmt: skip


def _make_params():
    g = torch.Generator().manual_seed(7)
    return [torch.nn.Parameter(torch.randn(*s, generator=g) * 0.02) for s in SHAPES]


def _grads(step):
    g = torch.Generator().manual_seed(100 + step)
    return [(torch.randn(*s, generator=g) * 1e-3).bfloat16().float() for s in SHAPES]


def _worker_lp(rank, port, out, kw, exchange="updates"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    muon_utils.newton_schulz = _cpu_ns
    params = _make_params()
    opt = LayerParallelMuon(params, bucket_numel=1024, exchange=exchange, **kw)
    for step in range(3):
        for p, g in zip(params, _grads(step)):
            p.grad = g.clone()
        opt.step()
    sd = opt.state_dict()
    full = opt.gathered_state_dict()
    full_momentum = {i: st["momentum_buffer"].numpy().copy() for i, st in full["state"].items()}  # owned entries alias the state
    # A fresh optimizer that loads the gathered checkpoint keeps exactly the entries it owns, and continues
    # identically.
    params2 = [torch.nn.Parameter(p.detach().clone()) for p in params]
    opt2 = LayerParallelMuon(params2, bucket_numel=1024, exchange=exchange, **kw)
    opt2.load_state_dict(full)
    for o, ps in ((opt, params), (opt2, params2)):
        for p, g in zip(ps, _grads(3)):
            p.grad = g.clone()
        o.step()
    out[rank] = {
        "params": [p.detach().numpy().copy() for p in params],
        "params_resumed": [p.detach().numpy().copy() for p in params2],
        "owned": opt.owned_indices(),
        "state_keys": sorted(sd["state"]),
        "full_momentum": full_momentum,
        "resumed_keys": sorted(i for i, p in enumerate(params2) if "momentum_buffer" in opt2.state.get(p, {})),
        "n_buckets": len(opt.buckets),
    }
    dist.destroy_process_group()


@pytest.mark.parametrize("method,exchange", [("decoupled", "updates"), ("l2", "updates"), ("decoupled", "parameters"), ("l2", "parameters"), ("decoupled", "mixed")])
def test_layer_parallel_muon_equals_single_process_bitwise(method, exchange, monkeypatch):
    kw = dict(KW, weight_decay_method=method)
    # single-process specification: this package's Muon with the same injected CPU orthogonalizer
    monkeypatch.setattr(muon_utils, "newton_schulz", _cpu_ns)
    ref_params = _make_params()
    ref = Muon(ref_params, **kw)
    for step in range(3):
        for p, g in zip(ref_params, _grads(step)):
            p.grad = g.clone()
        ref.step()
    ref_momentum = [ref.state[p]["momentum_buffer"].clone().numpy() for p in ref_params]
    for p, g in zip(ref_params, _grads(3)):
        p.grad = g.clone()
    ref.step()

    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker_lp, args=(_free_port(), out, kw, exchange), nprocs=WORLD, join=True)
        results = dict(out)
    owned_all = sorted(results[0]["owned"] + results[1]["owned"])
    assert owned_all == list(range(len(SHAPES)))  # every matrix has exactly one owner
    assert results[0]["state_keys"] == sorted(results[0]["owned"])  # momentum lives on the owner only
    assert results[0]["n_buckets"] > 1  # the small bucket size forces several exchanges
    for i in range(len(SHAPES)):
        assert np.array_equal(results[0]["params"][i], results[1]["params"][i]), i
        assert np.array_equal(results[0]["params"][i], ref_params[i].detach().numpy()), i
        # the gathered checkpoint holds every momentum buffer on every rank, equal to the single-process one
        for rank in range(WORLD):
            assert np.array_equal(results[rank]["full_momentum"][i], ref_momentum[i]), (rank, i)
            assert np.array_equal(results[rank]["params_resumed"][i], ref_params[i].detach().numpy()), (rank, i)
    for rank in range(WORLD):
        assert results[rank]["resumed_keys"] == sorted(results[rank]["owned"])


def test_partition_is_balanced_and_deterministic():
    layer = [(4096, 4096)] * 2 + [(1024, 4096)] * 2 + [(14336, 4096)] * 2 + [(4096, 14336)]
    shapes = layer * 32
    costs = [ns_cost(s) for s in shapes]
    assert ns_cost((14336, 4096)) == ns_cost((4096, 14336))
    for world in (1, 2, 4, 8):
        owners = partition_by_cost(costs, world)
        assert owners == partition_by_cost(costs, world)
        load = [sum(c for c, o in zip(costs, owners) if o == r) for r in range(world)]
        assert max(load) <= 1.02 * (sum(costs) / world)
    with pytest.raises(ValueError):
        partition_by_cost(costs, 0)
    assert partition_by_cost([], 4) == []


def test_bucket_plan_covers_every_matrix_once():
    numels = [100, 7, 64, 1000, 8, 8, 300]
    owners = [0, 1, 0, 1, 0, 0, 1]
    buckets = _plan_buckets(numels, owners, 2, bucket_numel=128)
    seen = sorted(i for b in buckets for r in range(2) for i, _ in b.per_rank[r])
    assert seen == list(range(len(numels)))
    for b in buckets:
        assert b.slot_numel % 8 == 0
        for r in range(2):
            end = 0
            for i, off in b.per_rank[r]:
                assert off >= end and off % 8 == 0
                end = off + numels[i]
            assert end <= b.slot_numel


def test_layer_parallel_rejects_non_2d():
    with pytest.raises(ValueError, match="Only 2D parameters are supported."):
        LayerParallelMuon([torch.nn.Parameter(torch.zeros(4))])
    with pytest.raises(ValueError, match="num_ns_steps must be at least 1"):
        LayerParallelMuon([torch.nn.Parameter(torch.zeros(4, 4))], num_ns_steps=0)


def test_layer_parallel_is_a_torch_optimizer_with_parameter_groups(monkeypatch):
    """Parameter groups with their own lr / weight decay, an LR scheduler, ``zero_grad`` and torch's own
    ``state_dict`` layout (``momentum_buffer`` per parameter, as the single-process class keeps it) all work, and a
    single-rank run equals Muon built from the same groups bit for bit."""
    monkeypatch.setattr(muon_utils, "newton_schulz", _cpu_ns)
    kw = dict(momentum=0.9, nesterov=True, num_ns_steps=5, coefficient_type="simple", scale_mode="shape_scaling")

    def groups(ps):
        return [{"params": ps[:3], "lr": 0.02, "weight_decay": 0.1}, {"params": ps[3:], "lr": 0.005, "weight_decay": 0.0}]

    a, b = _make_params(), _make_params()
    ref = Muon(groups(a), **kw)
    lp = LayerParallelMuon(groups(b), bucket_numel=1024, **kw)
    assert isinstance(lp, torch.optim.Optimizer)
    assert [g["lr"] for g in lp.param_groups] == [0.02, 0.005]
    sched = [torch.optim.lr_scheduler.StepLR(o, step_size=1, gamma=0.5) for o in (ref, lp)]
    for step in range(3):
        for ps in (a, b):
            for p, g in zip(ps, _grads(step)):
                p.grad = g.clone()
        ref.step()
        lp.step()
        for s in sched:
            s.step()
    assert lp.param_groups[0]["lr"] == pytest.approx(0.02 * 0.125)
    for pa, pb in zip(a, b):
        assert torch.equal(pa, pb)
        assert set(lp.state[pb]) == {"momentum_buffer"}
        assert torch.equal(lp.state[pb]["momentum_buffer"], ref.state[pa]["momentum_buffer"])
    sd = lp.state_dict()
    assert sorted(sd["state"]) == list(range(len(SHAPES))) and len(sd["param_groups"]) == 2
    lp.zero_grad()
    assert all(p.grad is None for p in b)
    with pytest.raises(ValueError, match="closure is not supported"):
        lp.step(lambda: 0.0)


def test_bucket_plan_by_shape_stacks_equal_shapes_and_ends_with_the_smallest():
    layer = [(4096, 4096)] * 2 + [(1024, 4096)] * 2 + [(14336, 4096)] * 2 + [(4096, 14336)]
    shapes = layer * 32
    numels = [a * b for a, b in shapes]
    world = 8
    owners = partition_by_cost([ns_cost(s) for s in shapes], world)
    buckets = _plan_buckets(numels, owners, world, 64 * 1024 * 1024, shapes)
    seen = sorted(i for b in buckets for r in range(world) for i, _ in b.per_rank[r])
    assert seen == list(range(len(shapes)))  # every matrix exactly once
    for b in buckets:
        for r in range(world):
            assert len({shapes[i] for i, _ in b.per_rank[r]}) <= 1  # one shape per rank and bucket: one batched run
    for r in range(world):
        sizes = [numels[b.per_rank[r][0][0]] for b in buckets if b.per_rank[r]]
        assert sizes == sorted(sizes, reverse=True)  # largest matrices first, smallest in the last buckets
        last = [b for b in buckets if b.per_rank[r]][-1]
        assert all(shapes[i] == (1024, 4096) for i, _ in last.per_rank[r])
