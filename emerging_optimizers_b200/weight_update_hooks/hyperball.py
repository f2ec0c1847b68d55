"""Hook that keeps update and weight on a sphere of fixed Frobenius radius.

Behaviour of ``emerging_optimizers/weight_update_hooks/hyperball.py:23-63`` of the reference: before the update the
*update* is rescaled to norm ``radius``; after the update the *weight* is projected back to norm ``radius``.
"""

import math

import torch

from emerging_optimizers_b200.weight_update_hooks import _norms


__all__ = ["HyperballHook"]


class HyperballHook:
    """``update <- radius * update / |update|`` before, ``p <- radius * p / |p|`` after the weight update.

    A tensor whose norm is below ``eps`` becomes exactly zero.

    Args:
        radius: target Frobenius norm; finite and at least ``eps``.
        eps: threshold of a numerical zero; finite and positive.
    """

    def __init__(self, radius: float, eps: float = 1e-15) -> None:
        _norms.check_eps(eps)
        if not math.isfinite(radius) or radius < eps:
            raise ValueError(f"radius must be finite and at least eps={eps}, got {radius}")
        self.radius = radius
        self.eps = eps

    def _project(self, t: torch.Tensor) -> None:
        n = _norms.fro_norm(t)
        target = torch.as_tensor(self.radius, device=t.device, dtype=torch.float32)
        _norms.scale_inplace(t, _norms.guarded_ratio(target, n, self.eps, n < self.eps))

    def pre_weight_update_inplace(self, p: torch.Tensor, update: torch.Tensor) -> None:
        self._project(update)
        return None

    def post_weight_update_inplace(self, p: torch.Tensor, pre_update_state: None) -> None:
        self._project(p)
