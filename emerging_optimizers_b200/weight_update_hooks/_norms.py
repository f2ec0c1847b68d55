"""Frobenius-norm helpers shared by the weight-update hooks.

All norms are accumulated in fp32 whatever the tensor's dtype, and a norm below the hook's ``eps`` counts as an
exact zero: such a tensor has no usable direction, so anything derived from it is mapped to zero instead of being
divided by a tiny number.  Everything stays on the tensor's device (no host synchronisation).
"""

import math

import torch


def check_eps(eps: float, *, finite: bool = True) -> None:
    if finite:
        if not math.isfinite(eps) or eps <= 0.0:
            raise ValueError(f"eps must be finite and positive, got {eps}")
    elif eps <= 0.0:
        raise ValueError(f"eps must be positive, got {eps}")


def fro_norm(t: torch.Tensor) -> torch.Tensor:
    """0-d fp32 Frobenius norm of ``t``."""
    return torch.linalg.vector_norm(t, dtype=torch.float32)


def fro_norm_or_zero(t: torch.Tensor, eps: float) -> torch.Tensor:
    """Frobenius norm, flushed to exactly zero below ``eps``."""
    n = fro_norm(t)
    return torch.where(n < eps, torch.zeros_like(n), n)


def guarded_ratio(num: torch.Tensor, den: torch.Tensor, eps: float, dead: torch.Tensor) -> torch.Tensor:
    """``num / den`` with the denominator clamped at ``eps``; exactly zero wherever ``dead`` is set."""
    return torch.where(dead, torch.zeros_like(den), num / den.clamp_min(eps))


def scale_inplace(t: torch.Tensor, scale: torch.Tensor) -> None:
    """``t *= scale`` with the 0-d ``scale`` cast to the tensor's dtype first."""
    t.mul_(scale.to(dtype=t.dtype))
