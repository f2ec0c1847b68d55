"""Shared by the CPU and GPU tests of the optimizers built on Newton-Schulz: rebuild a golden case (weights and
gradients from their seeds), run it on a device, and hand back what the golden file recorded."""

import json
import os

import numpy as np
import torch

import emerging_optimizers_b200.orthogonalized_optimizers as opt_pkg
import emerging_optimizers_b200.weight_update_hooks as hooks_pkg


GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

with open(os.path.join(GOLDEN, "consumer_cases.json")) as f:
    CASES = json.load(f)
SHAPES = [tuple(s) for s in CASES["shapes"]]
STEPS = CASES["steps"]
OPTIMIZER_CASES = sorted(CASES["optimizers"])


def golden():
    return np.load(os.path.join(GOLDEN, "consumers.npz"))


def randn(*shape, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32) * scale


def initial_weights(cls, kw):
    ws = []
    for i, s in enumerate(SHAPES):
        w = randn(*s, seed=400 + i, scale=0.05)
        if cls == "MuonHyperball":
            w = w * (kw["hyperball_radius"] / w.norm())
        ws.append(w)
    return ws


def run_case(name, precision, device):
    """Run the recorded steps; returns {"p<i>.after<step>" | "p<i>.<state key>": cpu tensor} and the initial
    weights."""
    cls, kw, hook = CASES["optimizers"][name]
    init = initial_weights(cls, kw)
    params = [torch.nn.Parameter(w.clone().to(device)) for w in init]
    extra = {} if hook is None else {"weight_update_hook": getattr(hooks_pkg, hook[0])(**hook[1])}
    if cls == "Muown":
        from emerging_optimizers_b200.contrib import Muown as opt_cls
    else:
        opt_cls = getattr(opt_pkg, cls)
    if "betas" in kw:
        kw = dict(kw, betas=tuple(kw["betas"]))
    opt = opt_cls(params, fp32_matmul_prec=precision, **kw, **extra)
    got = {}
    for step in range(STEPS):
        for i, p in enumerate(params):
            p.grad = randn(*p.shape, seed=450 + 10 * step + i, scale=1e-2).to(device)
        opt.step()
        if step in (0, STEPS - 1):
            for i, p in enumerate(params):
                got[f"p{i}.after{step}"] = p.detach().cpu().clone()
    for i, p in enumerate(params):
        for key, t in opt.state[p].items():
            if isinstance(t, torch.Tensor):
                got[f"p{i}.{key}"] = t.detach().cpu().clone()
    return got, init


def rel_fro(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-300))


def run_split_qkv(name, precision, device):
    """Two steps of SplitQkvMuon on a fused QKV weight and an ordinary weight; returns both weights (cpu) and
    their initial values."""
    cfg = CASES["split_qkv"]
    split, groups, per_head, head_dim = cfg["cases"][name]
    qkv0 = randn(groups * sum(split), cfg["hidden"], seed=600, scale=0.05)
    other0 = randn(24, 40, seed=601, scale=0.05)
    qkv, other = torch.nn.Parameter(qkv0.clone().to(device)), torch.nn.Parameter(other0.clone().to(device))
    qkv.is_qkv = True
    opt = opt_pkg.SplitQkvMuon(
        [qkv, other],
        qkv_split_shapes=split,
        num_query_groups=groups,
        per_head=per_head,
        head_dim=head_dim,
        fp32_matmul_prec=precision,
        **cfg["muon"],
    )
    for step in range(2):
        qkv.grad = randn(*qkv.shape, seed=610 + step, scale=1e-2).to(device)
        other.grad = randn(*other.shape, seed=620 + step, scale=1e-2).to(device)
        opt.step()
    return {"qkv": qkv.detach().cpu(), "other": other.detach().cpu()}, {"qkv": qkv0, "other": other0}
