"""Generate the golden vectors under tests/golden/ by running the reference implementation on CPU.

Run once, in a container that has the reference checkout (read-only) at the path given by $EO_REFERENCE:

    EO_REFERENCE=<reference checkout> python tests/golden/make_golden.py

(add ``TORCHDYNAMO_DISABLE=1`` where the container cannot build ``torch.compile`` kernels: the reference's Muown
decorates one elementwise helper with it, which then runs eagerly with the same arithmetic).

The reference is imported, never copied.  The outputs (small .npz / .json files next to this script) are
committed; the tests read only those files, so they also run where the reference checkout is absent.
"""

from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch
import torch.multiprocessing as mp


HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("EO_REFERENCE")
if not REF:
    raise SystemExit("set EO_REFERENCE to the root of the reference checkout")
sys.path.insert(0, REF)

from emerging_optimizers.orthogonalized_optimizers import muon_utils as ref_mu  # noqa: E402
from emerging_optimizers.orthogonalized_optimizers.muon import Muon as RefMuon  # noqa: E402
from emerging_optimizers.orthogonalized_optimizers.muon import get_muon_scale_factor as ref_scale  # noqa: E402


def randn(*shape: int, seed: int, scale: float = 1.0) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32) * scale


def run_ns(x: torch.Tensor, precision: str, **kw) -> np.ndarray:
    prev = torch.get_float32_matmul_precision()
    torch.set_float32_matmul_precision(precision)
    try:
        return ref_mu.newton_schulz(x, **kw).contiguous().numpy()
    finally:
        torch.set_float32_matmul_precision(prev)


NS_CASES = {
    # name: (shape, seed, input scale, kwargs)
    "simple_wide": ((24, 40), 10, 1.0, dict(steps=5, coefficient_type="simple")),
    "quintic_wide": ((24, 40), 11, 1.0, dict(steps=5, coefficient_type="quintic")),
    "quintic_tall": ((40, 24), 12, 1.0, dict(steps=5, coefficient_type="quintic")),
    "quintic_7steps": ((16, 32), 13, 1.0, dict(steps=7, coefficient_type="quintic")),
    "polar_express_9": ((24, 40), 14, 1.0, dict(steps=9, coefficient_type="polar_express")),
    "cans_6": ((24, 40), 15, 1.0, dict(steps=6, coefficient_type="cans")),
    "aol_4": ((24, 40), 16, 1.0, dict(steps=4, coefficient_type="aol")),
    "deepseekv4_10": ((24, 40), 17, 1.0, dict(steps=10, coefficient_type="deepseekv4")),
    "cubic5": ((24, 40), 18, 1.0, dict(steps=5, coefficient_type="cubic5")),
    "custom": (
        (24, 40),
        19,
        1.0,
        dict(steps=3, coefficient_type="custom", custom_coefficient_sets=[(3.0, -3.0, 1.0), (2.0, -1.5, 0.5)]),
    ),
    "steps0": ((8, 16), 20, 1.0, dict(steps=0, coefficient_type="simple")),
    "batched": ((3, 16, 24), 21, 1.0, dict(steps=5, coefficient_type="simple")),
    "batched_tall": ((2, 24, 16), 22, 1.0, dict(steps=5, coefficient_type="quintic")),
    "square": ((32, 32), 23, 1.0, dict(steps=5, coefficient_type="quintic")),
    "small_grad": ((24, 40), 24, 1e-3, dict(steps=5, coefficient_type="simple")),
    "tiny_double": ((8, 16), 25, 1e-25, dict(steps=3, coefficient_type="simple", normalize_in_double=True)),
    "force_no_transpose": ((40, 24), 26, 1.0, dict(steps=2, coefficient_type="simple", transpose=False)),
    "unaligned": ((13, 21), 27, 1.0, dict(steps=5, coefficient_type="quintic")),
}


def make_ns() -> None:
    for precision in ("highest", "medium"):
        out = {}
        for name, (shape, seed, scale, kw) in NS_CASES.items():
            x = randn(*shape, seed=seed, scale=scale)
            out[f"{name}.x"] = x.numpy()
            out[f"{name}.y"] = run_ns(x, precision, **kw)
        np.savez_compressed(os.path.join(HERE, f"ns_{precision}.npz"), **out)
    meta = {name: {"shape": list(shape), "kwargs": kw} for name, (shape, _, _, kw) in NS_CASES.items()}
    with open(os.path.join(HERE, "ns_cases.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)


def make_config1() -> None:
    """BASELINE config 1: 1024 x 4096 N(0,1) seed 0, five "simple" steps; a strided sample of the result, its
    singular-value band and a checksum of the input are stored."""
    x = randn(1024, 4096, seed=0)
    rec = {"x_sum": np.float64(x.double().sum().item()), "x_sumsq": np.float64((x.double() ** 2).sum().item())}
    for precision in ("highest", "medium"):
        y = torch.from_numpy(run_ns(x, precision, steps=5, coefficient_type="simple"))
        sv = torch.linalg.svdvals(y.double())
        rec[f"{precision}.sample"] = y[::16, ::16].contiguous().numpy()
        rec[f"{precision}.sv_min"] = np.float64(sv.min().item())
        rec[f"{precision}.sv_max"] = np.float64(sv.max().item())
        rec[f"{precision}.fro"] = np.float64(y.double().norm().item())
    np.savez_compressed(os.path.join(HERE, "config1.npz"), **rec)


MUON_CASES = {
    "config3_like": dict(
        lr=0.02, momentum=0.95, weight_decay=0.1, nesterov=True, weight_decay_method="decoupled",
        num_ns_steps=5, scale_mode="shape_scaling", coefficient_type="simple", fp32_matmul_prec="medium",
    ),
    "defaults_highest": dict(fp32_matmul_prec="highest"),
    "l2_unit_rms": dict(
        lr=0.01, weight_decay=0.05, weight_decay_method="l2", scale_mode="unit_rms_norm", extra_scale_factor=0.2,
        fp32_matmul_prec="highest", coefficient_type="polar_express", num_ns_steps=6,
    ),
}  # fmt: skip
MUON_SHAPES = [(32, 32), (8, 32), (48, 16), (16, 48)]


def make_muon() -> None:
    out = {}
    for name, kw in MUON_CASES.items():
        params = [torch.nn.Parameter(randn(*s, seed=100 + i, scale=0.02)) for i, s in enumerate(MUON_SHAPES)]
        opt = RefMuon(params, **kw)
        for i, p in enumerate(params):
            out[f"{name}.p{i}.init"] = p.detach().clone().numpy()
        for step in range(2):
            for i, p in enumerate(params):
                g = randn(*p.shape, seed=200 + 10 * step + i, scale=1e-3).bfloat16().float()
                out[f"{name}.p{i}.grad{step}"] = g.numpy()
                p.grad = g.clone()
            opt.step()
            for i, p in enumerate(params):
                out[f"{name}.p{i}.after{step}"] = p.detach().clone().numpy()
                out[f"{name}.p{i}.mom{step}"] = opt.state[p]["momentum_buffer"].clone().numpy()
    np.savez_compressed(os.path.join(HERE, "muon_steps.npz"), **out)
    with open(os.path.join(HERE, "muon_cases.json"), "w") as f:
        json.dump({"cases": MUON_CASES, "shapes": MUON_SHAPES}, f, indent=1, sort_keys=True)


def make_tables() -> None:
    sched = {}
    for name, sets in ref_mu._COEFFICIENT_SETS.items():
        mode = "repeat_last" if name in ("polar_express", "cans", "deepseekv4") else "cycle"
        sched[name] = {"mode": mode, "steps12": [list(t) for t in ref_mu.get_coefficient_iterator(12, sets, mode)]}
    scales = {
        f"{mode}:{m}x{n}": ref_scale(m, n, mode)
        for mode in ("shape_scaling", "spectral", "unit_rms_norm")
        for (m, n) in [(4096, 4096), (1024, 4096), (14336, 4096), (4096, 14336), (128, 8192)]
    }
    with open(os.path.join(HERE, "tables.json"), "w") as f:
        json.dump({"schedules": sched, "scale_factors": scales}, f, indent=1, sort_keys=True)


def _tp_worker(rank: int, world: int, port: int, x_full: torch.Tensor, results: dict) -> None:
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    group = torch.distributed.group.WORLD
    torch.set_float32_matmul_precision("highest")
    for pdim in (0, 1):
        for mode in ("distributed", "duplicated"):
            src = x_full if pdim == 1 else x_full.mT.contiguous()
            shard = src.chunk(world, dim=pdim)[rank].contiguous()
            y = ref_mu.newton_schulz_tp(shard, 5, "quintic", group, partition_dim=pdim, tp_mode=mode)
            results[f"p{pdim}.{mode}.rank{rank}"] = y.contiguous().numpy()
    torch.distributed.destroy_process_group()


def make_tp() -> None:
    world = 2
    x_full = randn(16, 48, seed=300)
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_tp_worker, args=(world, 29731, x_full, results), nprocs=world, join=True)
        out = {k: v for k, v in results.items()}
    out["x_full"] = x_full.numpy()
    np.savez_compressed(os.path.join(HERE, "ns_tp.npz"), **out)


CONSUMER_SHAPES = [(32, 48), (48, 32)]
CONSUMER_STEPS = 3
# name: (optimizer class, constructor kwargs, weight-update hook (class name, kwargs) or None)
CONSUMER_CASES = {
    "scion": ("Scion", dict(lr=0.05, momentum=0.9, num_ns_steps=5, spectral_radius=1.5), None),
    "spel": ("Spel", dict(lr=0.05, momentum=0.9, weight_decay=0.1, nesterov=True, num_ns_steps=5), None),
    "polargrad": (
        "PolarGrad",
        dict(lr=0.05, momentum=0.9, weight_decay=0.01, extra_scale_factor=0.5, coefficient_type="polar_express",
             num_ns_steps=6),
        None,
    ),
    "adamuon": (
        "AdaptiveMuon",
        dict(lr=0.02, momentum=0.9, weight_decay=0.05, nesterov=True, moment2_method="adamuon"),
        None,
    ),
    "normuon": (
        "AdaptiveMuon",
        dict(lr=0.02, momentum=0.9, weight_decay=0.05, moment2_method="normuon", scale_mode="shape_scaling"),
        None,
    ),
    "namo": (
        "AdaptiveMuon",
        dict(lr=0.02, momentum=0.9, weight_decay=0.05, nesterov=True, moment2_method="namo", extra_scale_factor=0.3),
        None,
    ),
    "hyperball": ("MuonHyperball", dict(lr=0.05, momentum=0.9, hyperball_radius=2.0), None),
    "muon_radial_brake": (
        "Muon",
        dict(lr=0.05, momentum=0.9, weight_decay=0.0),
        ("RadialBrakeHook", dict(outward_scale=0.25, inward_scale=0.75)),
    ),
    "muon_relative_update": ("Muon", dict(lr=0.05, momentum=0.9), ("RelativeUpdateHook", dict())),
    "mop": ("MOP", dict(lr=0.05, momentum=0.9, nesterov=True, extra_scale_factor=0.5), None),
    "muown": (
        "Muown",
        dict(lr=0.05, momentum=0.9, weight_decay=0.05, betas=(0.9, 0.95), extra_scale_factor=0.2),
        None,
    ),
}  # fmt: skip

SPECTRAL_CASES = {
    # name: (function, shape, seed, kwargs)
    "clip_wide": ("spectral_clip", (32, 48), 500, dict(sigma_min=0.5, sigma_max=1.5)),
    "clip_tall": ("spectral_clip", (48, 32), 501, dict(sigma_min=0.5, sigma_max=1.5)),
    "clip_default": ("spectral_clip", (40, 40), 502, dict()),
    "hardcap_wide": ("spectral_hardcap", (32, 48), 503, dict(beta=1.0)),
    "hardcap_tall": ("spectral_hardcap", (48, 32), 504, dict(beta=0.8)),
    "clipped_wd": ("spectral_clipped_weight_decay", (32, 48), 505, dict(beta=1.0, c=0.25)),
}
ONE_SIDED_CASES = {
    "left": ((16, 64), 510, dict(side="left")),
    "left_centered": ((16, 64), 511, dict(side="left", center_rows=True, alpha=0.5)),
    "right": ((64, 16), 512, dict(side="right", extra_scale_factor=0.2)),
    "right_centered": ((64, 16), 513, dict(side="right", center_rows=True)),
}


QKV_HIDDEN = 48
QKV_CASES = {
    # name: (rows of q, k, v in one query group; query groups; per-head; head_dim)
    "stacked": ((32, 16, 16), 1, False, None),
    "interleaved": ((16, 8, 8), 2, False, None),
    "per_head": ((16, 8, 8), 2, True, 8),
}
QKV_MUON = dict(lr=0.05, momentum=0.9, weight_decay=0.01, nesterov=True, scale_mode="shape_scaling")


def qkv_row_sets(split, groups, per_head, head_dim):
    """Row indices of every logical matrix inside a fused QKV weight laid out [q_0; k_0; v_0; q_1; ...]."""
    per_group = sum(split)
    sets = []
    offset = 0
    for rows in split:
        block = [g * per_group + offset + r for g in range(groups) for r in range(rows)]
        if per_head:
            sets += [block[i : i + head_dim] for i in range(0, len(block), head_dim)]
        else:
            sets.append(block)
        offset += rows
    return sets


def make_split_qkv(out: dict) -> None:
    """Fused-QKV Muon the way the docstring of the reference's base class sketches it: a subclass of the
    reference's Muon that runs ``scaled_orthogonalize_fn`` on every logical matrix of a tagged parameter."""

    class RefSplitQkvMuon(RefMuon):
        def __init__(self, params, row_sets, **kw):
            super().__init__(params, **kw)
            self.row_sets = row_sets

        def orthogonalize(self, p, grad, **kwargs):
            if not getattr(p, "is_qkv", False):
                return self.scaled_orthogonalize_fn(grad)
            res = torch.empty_like(grad)
            for rows in self.row_sets:
                idx = torch.tensor(rows)
                res[idx] = self.scaled_orthogonalize_fn(grad[idx])
            return res

    for name, (split, groups, per_head, head_dim) in QKV_CASES.items():
        for precision in ("highest", "medium"):
            qkv = torch.nn.Parameter(randn(groups * sum(split), QKV_HIDDEN, seed=600, scale=0.05))
            qkv.is_qkv = True
            other = torch.nn.Parameter(randn(24, 40, seed=601, scale=0.05))
            opt = RefSplitQkvMuon(
                [qkv, other], qkv_row_sets(split, groups, per_head, head_dim), fp32_matmul_prec=precision, **QKV_MUON
            )
            for step in range(2):
                qkv.grad = randn(*qkv.shape, seed=610 + step, scale=1e-2)
                other.grad = randn(*other.shape, seed=620 + step, scale=1e-2)
                opt.step()
            out[f"split_qkv.{name}.{precision}.qkv"] = qkv.detach().clone().numpy()
            out[f"split_qkv.{name}.{precision}.other"] = other.detach().clone().numpy()


def make_consumers() -> None:
    """Optimizers and utilities built on Newton-Schulz: three steps of each optimizer on three small matrices, at
    "highest" and at "medium" precision; the spectral clipping functions; the one-sided polar updates."""
    import emerging_optimizers.orthogonalized_optimizers as ref_opt
    import emerging_optimizers.weight_update_hooks as ref_hooks
    from emerging_optimizers.orthogonalized_optimizers import polargrad as ref_pg
    from emerging_optimizers.orthogonalized_optimizers import spectral_clipping_utils as ref_sc

    out = {}
    for name, (cls, kw, hook) in CONSUMER_CASES.items():
        for precision in ("highest", "medium"):
            key = f"{name}.{precision}"
            params = []
            for i, s in enumerate(CONSUMER_SHAPES):
                w = randn(*s, seed=400 + i, scale=0.05)
                if cls == "MuonHyperball":
                    w = w * (kw["hyperball_radius"] / w.norm())
                params.append(torch.nn.Parameter(w))
            extra = {} if hook is None else {"weight_update_hook": getattr(ref_hooks, hook[0])(**hook[1])}
            if cls == "Muown":
                from emerging_optimizers.contrib.muown import Muown as ref_cls
            else:
                ref_cls = getattr(ref_opt, cls)
            opt = ref_cls(params, fp32_matmul_prec=precision, **kw, **extra)
            # Initial weights and gradients are regenerated from their seeds by the tests, not stored.
            for step in range(CONSUMER_STEPS):
                for i, p in enumerate(params):
                    p.grad = randn(*p.shape, seed=450 + 10 * step + i, scale=1e-2)
                opt.step()
                if step in (0, CONSUMER_STEPS - 1):
                    for i, p in enumerate(params):
                        out[f"{key}.p{i}.after{step}"] = p.detach().clone().numpy()
            for i, p in enumerate(params):
                for buf, t in opt.state[p].items():
                    if isinstance(t, torch.Tensor):  # Muown also keeps an integer step count
                        out[f"{key}.p{i}.{buf}"] = t.clone().numpy()

    torch.set_float32_matmul_precision("highest")
    for name, (fn, shape, seed, kw) in SPECTRAL_CASES.items():
        x = randn(*shape, seed=seed, scale=0.2)
        out[f"spectral.{name}"] = getattr(ref_sc, fn)(x, **kw).contiguous().numpy()
    for name, (shape, seed, kw) in ONE_SIDED_CASES.items():
        x = randn(*shape, seed=seed)
        out[f"one_sided.{name}"] = ref_pg.one_sided_polargrad_orth_fn(x, **kw).contiguous().numpy()

    make_split_qkv(out)
    np.savez_compressed(os.path.join(HERE, "consumers.npz"), **out)
    with open(os.path.join(HERE, "consumer_cases.json"), "w") as f:
        json.dump(
            {
                "shapes": CONSUMER_SHAPES,
                "steps": CONSUMER_STEPS,
                "optimizers": CONSUMER_CASES,
                "spectral": SPECTRAL_CASES,
                "one_sided": ONE_SIDED_CASES,
                "split_qkv": {"hidden": QKV_HIDDEN, "cases": QKV_CASES, "muon": QKV_MUON},
            },
            f,
            indent=1,
            sort_keys=True,
        )


if __name__ == "__main__":
    torch.manual_seed(0)
    if sys.argv[1:] == ["consumers"]:
        make_consumers()
        raise SystemExit(0)
    make_tables()
    make_ns()
    make_config1()
    make_muon()
    make_tp()
    make_consumers()
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))
