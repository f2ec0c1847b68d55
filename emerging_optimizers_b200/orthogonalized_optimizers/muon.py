"""Muon: momentum orthogonalized by Newton-Schulz, on the sm_100a kernels.

Constructor signature, defaults, read-only properties, registry name and scale-factor modes follow
``emerging_optimizers/orthogonalized_optimizers/muon.py:34-216`` of the reference.
"""

from __future__ import annotations

from typing import Literal

import torch
from absl import logging
from torch.optim.optimizer import ParamsT

from emerging_optimizers_b200 import registry, triton_kernels
from emerging_optimizers_b200.mixin import WeightDecayT
from emerging_optimizers_b200 import _native
from emerging_optimizers_b200.orthogonalized_optimizers import _fused_step, muon_utils
from emerging_optimizers_b200.orthogonalized_optimizers.muon_utils import NSCoeffT
from emerging_optimizers_b200.orthogonalized_optimizers.orthogonalized_optimizer import (
    OrthogonalizedOptimizer,
    _args_doc,
)
from emerging_optimizers_b200.utils import FP32MatmulPrecT
from emerging_optimizers_b200.weight_update_hooks import NoOpWeightUpdateHook, WeightUpdateHook
from emerging_optimizers_b200.weight_update_hooks.base import HookStateT


__all__ = ["Muon", "get_muon_scale_factor"]

MuonScaleT = Literal["shape_scaling", "spectral", "unit_rms_norm"]

# Compute capabilities on which the SYRK kernel of this package runs.
_SYRK_SM = ((10, 0), (10, 3))

# Set to False to force the per-parameter step even where the grouped fused step applies.
FUSED_STEP = True

# The driver functions as defined by this package: the fused step only takes over while nobody has replaced them.
_NS_FUNCTIONS = {
    name: getattr(muon_utils, name)
    for name in (
        "newton_schulz",
        "newton_schulz_step",
        "batched_newton_schulz_step",
        "newton_schulz_step_tsyrk",
        "batched_newton_schulz_step_tsyrk",
    )
}

# parameter shrink p <- p + f * p applied before the update, per weight-decay method ("l2" acts on the gradient)
_SHRINK = {
    "decoupled": lambda lr, wd: -wd * lr,
    "independent": lambda lr, wd: -wd,
    "palm": lambda lr, wd: -(wd * lr * lr),
    "l2": lambda lr, wd: 0.0,
}


def _read_only(name: str) -> property:
    def getter(self):  # type: ignore[no-untyped-def]
        return getattr(self, "_" + name)

    def setter(self, _value):  # type: ignore[no-untyped-def]
        raise AttributeError(f"Cannot set `{name}` post-initialization.")

    return property(getter, setter)


@registry.register_optimizer("muon")
class Muon(OrthogonalizedOptimizer[HookStateT]):
    """MomentUm Orthogonalized by Newton-schulz.

    EMA momentum (optionally Nesterov), then every 2-D update is replaced by an approximation of its nearest
    semi-orthogonal matrix computed by Newton-Schulz iteration on tensor cores, scaled, and applied with decoupled
    weight decay.  Use it for hidden 2-D weights only; embeddings, the output layer and 1-D parameters belong to a
    standard optimizer.

    Args:
        {_args_doc}
        coefficient_type: Newton-Schulz schedule, one of "simple", "quintic", "polar_express", "cans", "aol",
            "deepseekv4", "cubic5", "custom".
        num_ns_steps: number of Newton-Schulz iterations (at least 1).
        scale_mode: update scale, see :func:`get_muon_scale_factor`.
        extra_scale_factor: extra multiplier of the update (0.2 roughly matches AdamW's update RMS).
        use_syrk: use the lower-triangular SYRK kernel for the symmetric products of the iteration.
    """

    def __init__(
        self,
        params: ParamsT,
        lr: float = 3e-4,
        momentum: float = 0.95,
        weight_decay: float = 0.01,
        *,
        nesterov: bool = False,
        weight_decay_method: WeightDecayT = "decoupled",
        fp32_matmul_prec: FP32MatmulPrecT = "medium",
        coefficient_type: NSCoeffT = "quintic",
        num_ns_steps: int = 5,
        scale_mode: MuonScaleT = "spectral",
        extra_scale_factor: float = 1.0,
        use_syrk: bool = False,
        weight_update_hook: WeightUpdateHook[HookStateT] | None = None,
    ) -> None:
        if num_ns_steps < 1:
            raise ValueError(f"num_ns_steps must be at least 1, got {num_ns_steps}")

        if use_syrk:
            sm = torch.cuda.get_device_capability() if torch.cuda.is_available() else (0, 0)
            if not triton_kernels.HAS_TRITON_340:
                logging.error("libeo_b200.so is required for use_syrk to be True. Setting use_syrk to False.")
                use_syrk = False
            elif sm not in _SYRK_SM:
                logging.error("The SYRK kernel does not run on SM %s. Setting use_syrk to False.", sm)
                use_syrk = False

        self._num_ns_steps = num_ns_steps
        self._coefficient_type = coefficient_type
        self._scale_mode = scale_mode
        self._extra_scale_factor = extra_scale_factor
        self._use_syrk = use_syrk

        def scaled_orthogonalize_fn(grad: torch.Tensor) -> torch.Tensor:
            orth = muon_utils.newton_schulz(
                grad, steps=num_ns_steps, coefficient_type=coefficient_type, use_syrk=use_syrk
            )
            # Scale from the size of one matrix, so a 3-D stack of per-head blocks is scaled per block.
            scale = get_muon_scale_factor(grad.size(-2), grad.size(-1), mode=scale_mode)
            return orth * scale * extra_scale_factor

        super().__init__(
            params,
            lr,
            momentum,
            nesterov=nesterov,
            weight_decay=weight_decay,
            weight_decay_method=weight_decay_method,
            fp32_matmul_prec=fp32_matmul_prec,
            scaled_orthogonalize_fn=scaled_orthogonalize_fn,
            weight_update_hook=weight_update_hook,
        )
        self._muon_closure = scaled_orthogonalize_fn

    def _fused_step_applies(self) -> bool:
        """The grouped fused step computes exactly what the per-parameter step computes, but bypasses the
        override points; it is used only while none of them is customised and the bf16 path is selected."""
        cls, base = type(self), OrthogonalizedOptimizer
        return (
            FUSED_STEP
            and self.fp32_matmul_prec == "medium"
            and self.weight_decay_method in _SHRINK
            and self._coefficient_type in muon_utils._COEFFICIENT_SETS
            and cls.orthogonalize is base.orthogonalize
            and cls._step_param is base._step_param
            and cls._momentum_update is base._momentum_update
            and cls._init_group is base._init_group
            and cls._apply_weight_decay_inplace is base._apply_weight_decay_inplace
            and cls.pre_weight_update_fn_inplace is base.pre_weight_update_fn_inplace
            and cls.post_weight_update_fn_inplace is base.post_weight_update_fn_inplace
            and type(self._weight_update_hook) is NoOpWeightUpdateHook
            and self.scaled_orthogonalize_fn is self._muon_closure
            and all(getattr(muon_utils, name) is fn for name, fn in _NS_FUNCTIONS.items())
        )

    @torch.no_grad()
    def step(self, closure=None):  # type: ignore[no-untyped-def]
        """One optimization step.

        Parameters that the fused kernels can take (2-D contiguous fp32 CUDA tensors, bf16 path, no customised
        hook or override) are processed as groups of equally shaped matrices: fused momentum / normalise kernels,
        one batched Newton-Schulz run per group, fused weight update.  Everything else takes the per-parameter
        path of the base class.  Both paths compute the same update.  One visible difference: with
        ``weight_decay_method="l2"`` the per-parameter path adds ``weight_decay * p`` into ``p.grad`` in place (as the
        reference does), while the fused kernels form ``g + weight_decay * p`` on the fly and leave ``p.grad`` as the
        caller set it.
        """
        if closure is not None:
            raise ValueError("closure is not supported")
        if not self._fused_step_applies():
            return super().step()

        for group in self.param_groups:
            self._init_group(group)
            lr, wd, mu = group["lr"], group["weight_decay"], group["momentum"]
            fused = []
            for p in group["params"]:
                if p.grad is None:
                    continue
                if _fused_step.eligible(p, p.grad) and self.state[p]["momentum_buffer"].is_contiguous():
                    fused.append(p)
                else:
                    self._step_param(group, p)
            if not fused:
                continue
            l2 = wd if self.weight_decay_method == "l2" else 0.0
            updates = _fused_step.orthogonalized_updates(
                [p.data for p in fused],
                [p.grad for p in fused],
                [self.state[p]["momentum_buffer"] for p in fused],
                momentum=mu,
                nesterov=self.nesterov,
                l2_weight_decay=l2,
                steps=self._num_ns_steps,
                coefficient_type=self._coefficient_type,
                use_syrk=self._use_syrk,
            )
            shrink = _SHRINK[self.weight_decay_method](lr, wd) if wd != 0.0 else 0.0
            by_device: dict = {}
            for p, u in zip(fused, updates):
                by_device.setdefault(p.device, []).append((p, u))
            for pairs in by_device.values():
                scales = [get_muon_scale_factor(p.size(-2), p.size(-1), mode=self._scale_mode) for p, _ in pairs]
                _native.muon_apply_batch(
                    [p.data for p, _ in pairs], [u for _, u in pairs], scales, shrink, self._extra_scale_factor, lr
                )
        return None

    num_ns_steps = _read_only("num_ns_steps")
    coefficient_type = _read_only("coefficient_type")
    scale_mode = _read_only("scale_mode")
    extra_scale_factor = _read_only("extra_scale_factor")
    use_syrk = _read_only("use_syrk")


Muon.__doc__ = Muon.__doc__.format(_args_doc=_args_doc)  # type: ignore[union-attr]


def get_muon_scale_factor(size_out: int, size_in: int, mode: MuonScaleT = "spectral") -> float:
    """Scale applied to the orthogonalized update of a ``size_out x size_in`` weight.

    - "shape_scaling": ``sqrt(max(1, size_out / size_in))`` (Keller Jordan's Muon write-up)
    - "spectral": ``sqrt(max(size_out, size_in))`` (Jordan / Kimi, arXiv:2502.16982; lets AdamW learning rates
      transfer)
    - "unit_rms_norm": ``sqrt(size_out / size_in)`` (Scion, arXiv:2502.07529)
    """
    if mode == "shape_scaling":
        return max(1, size_out / size_in) ** 0.5
    if mode == "spectral":
        return max(size_out, size_in) ** 0.5
    if mode == "unit_rms_norm":
        return (size_out / size_in) ** 0.5
    raise ValueError(f"Invalid mode for Muon update scale factor: {mode}")
