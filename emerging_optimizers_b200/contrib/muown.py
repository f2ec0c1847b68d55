"""Muown: Muon on a weight-normalised parameterisation (a magnitude per row times a direction).

Same constructor surface, state keys and arithmetic as ``emerging_optimizers/contrib/muown.py:60-210`` of the
reference (Lion et al., arXiv:2605.10797): every 2-D weight is kept as ``W = g * v / ||v||_row``; the direction ``v``
takes a Muon step (momentum, Newton-Schulz on this package's kernels, scale) with the direction part of the
gradient, the per-row magnitude ``g`` takes a bias-corrected Adam step with the magnitude part, decoupled weight
decay acts on ``g`` only, and the weight is rebuilt from both.  Only the elementwise algebra lives here; the
orthogonalization is Muon's closure, so it runs on the same tensor-core path as every other caller.
"""

from __future__ import annotations

from typing import Callable

import torch
from torch.optim.optimizer import ParamsT

from emerging_optimizers_b200 import utils
from emerging_optimizers_b200.orthogonalized_optimizers.muon import Muon, MuonScaleT
from emerging_optimizers_b200.orthogonalized_optimizers.muon_utils import NSCoeffT
from emerging_optimizers_b200.utils import FP32MatmulPrecT


__all__ = ["Muown"]

_ROW_NORM_FLOOR = 1e-12  # keeps W / g finite for an all-zero row


def _split_gradient(weight, grad, g, v_norm):
    """Direction ``v`` rebuilt from the weight, and the gradient split into its magnitude and direction parts."""
    u = weight / g  # unit rows
    grad_g = (grad * u).sum(dim=1, keepdim=True)
    grad_v = (g / v_norm) * (grad - u * grad_g)
    return u * v_norm, grad_g, grad_v


def _adam_direction(grad, m, v, betas, eps, step):
    """Bias-corrected Adam update (no Nesterov); ``m`` and ``v`` are advanced in place."""
    b1, b2 = betas
    m.lerp_(grad, 1 - b1)
    v.lerp_(grad.square(), 1 - b2)
    return (m / (1.0 - b1**step)) / ((v / (1.0 - b2**step)).sqrt() + eps)


class Muown(Muon):
    """Muon with row-norm control.

    Args:
        params: parameters or parameter groups (2-D tensors only).
        lr: learning rate of both the direction and the magnitude update.
        momentum: EMA coefficient of the direction's momentum buffer.
        weight_decay: decoupled weight decay, applied to the magnitudes.
        betas: Adam coefficients of the magnitude update.
        adam_eps: Adam epsilon of the magnitude update.
        fp32_matmul_prec, coefficient_type, num_ns_steps, scale_mode, extra_scale_factor, use_syrk: as for
            :class:`~emerging_optimizers_b200.orthogonalized_optimizers.Muon`.
    """

    def __init__(
        self,
        params: ParamsT,
        lr: float = 3e-4,
        momentum: float = 0.95,
        weight_decay: float = 0.0,
        *,
        betas: tuple[float, float] = (0.9, 0.95),
        adam_eps: float = 1e-8,
        fp32_matmul_prec: FP32MatmulPrecT = "medium",
        coefficient_type: NSCoeffT = "quintic",
        num_ns_steps: int = 5,
        scale_mode: MuonScaleT = "spectral",
        extra_scale_factor: float = 1.0,
        use_syrk: bool = False,
    ) -> None:
        self.betas = betas
        self.adam_eps = adam_eps
        super().__init__(
            params, lr, momentum, weight_decay, nesterov=False, weight_decay_method="decoupled",
            fp32_matmul_prec=fp32_matmul_prec, coefficient_type=coefficient_type, num_ns_steps=num_ns_steps,
            scale_mode=scale_mode, extra_scale_factor=extra_scale_factor, use_syrk=use_syrk,
        )  # fmt: skip

    @torch.no_grad()
    def _init_group(self, group: dict, skip_non_grad_params: bool = True) -> None:
        for p in group["params"]:
            if skip_non_grad_params and p.grad is None:
                continue
            if p.dim() != 2:
                raise TypeError("Muown is only supported for 2D parameters")
            state = self.state[p]
            if len(state) == 0:
                # magnitude and direction norm both start at the weight's row norms: the first step equals Muon's
                rows = p.norm(dim=1, keepdim=True).to(torch.float32).clamp_min(_ROW_NORM_FLOOR)
                state["step"] = 0
                state["g"] = rows.clone()
                state["v_norm"] = rows.clone()
                state["momentum_buffer"] = torch.zeros_like(p, dtype=torch.float32)
                state["m_g"] = torch.zeros_like(rows)
                state["v_g"] = torch.zeros_like(rows)

    @torch.no_grad()
    def step(self, closure: Callable[[], float] | None = None) -> None:  # type: ignore[override]
        if closure is not None:
            raise ValueError("closure is not supported")
        for group in self.param_groups:
            self._init_group(group)
            lr, momentum, weight_decay = group["lr"], group["momentum"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                g = state["g"]
                v, grad_g, grad_v = _split_gradient(p.to(torch.float32), p.grad.to(torch.float32), g, state["v_norm"])

                state["momentum_buffer"].lerp_(grad_v, 1 - momentum)
                with utils.fp32_matmul_precision(self.fp32_matmul_prec):
                    direction = self.scaled_orthogonalize_fn(state["momentum_buffer"])
                v_new = v.add(direction, alpha=-lr)

                g.add_(_adam_direction(grad_g, state["m_g"], state["v_g"], self.betas, self.adam_eps, state["step"] + 1),
                       alpha=-lr)  # fmt: skip
                self._apply_weight_decay_inplace(g, grad_g, lr, weight_decay)

                v_norm_new = v_new.norm(dim=1, keepdim=True)
                p.copy_(g * (v_new / v_norm_new))
                state["v_norm"] = v_norm_new
                state["step"] += 1
        return None
