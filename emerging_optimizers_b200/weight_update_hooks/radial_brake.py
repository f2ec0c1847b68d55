"""Hook that damps the change of a weight's Frobenius norm caused by an update.

Behaviour of ``emerging_optimizers/weight_update_hooks/radial_brake.py:23-89`` of the reference: after
``w = w_prev + dw`` the weight is rescaled so that ``|w_braked| = |w_prev| + s * (|w| - |w_prev|)``, where ``s`` is
``outward_scale`` if the norm grew and ``inward_scale`` if it shrank.
"""

import torch

from emerging_optimizers_b200.weight_update_hooks import _norms


__all__ = ["RadialBrakeHook"]


class RadialBrakeHook:
    """Keep only a fraction of the radial (norm) change of each update; the direction is untouched.

    Args:
        outward_scale: fraction of a norm increase that is kept, in [0, 1].
        inward_scale: fraction of a norm decrease that is kept, in [0, 1].
        eps: norms and norm changes smaller than this count as zero; finite and positive.
    """

    def __init__(self, outward_scale: float = 0.5, inward_scale: float = 1.0, eps: float = 1e-15) -> None:
        for name, value in (("outward_scale", outward_scale), ("inward_scale", inward_scale)):
            if not 0.0 <= value <= 1.0:
                raise ValueError(f"{name} must be in [0, 1], got {value}")
        _norms.check_eps(eps)
        self.outward_scale = outward_scale
        self.inward_scale = inward_scale
        self.eps = eps

    def pre_weight_update_inplace(self, p: torch.Tensor, update: torch.Tensor) -> torch.Tensor:
        """Returns the norm of the weight before the update (the hook's state)."""
        return _norms.fro_norm_or_zero(p, self.eps)

    def post_weight_update_inplace(self, p: torch.Tensor, pre_update_state: torch.Tensor) -> None:
        before = pre_update_state
        after = _norms.fro_norm_or_zero(p, self.eps)
        delta = after - before
        kept = torch.zeros_like(delta)
        kept = torch.where(delta >= self.eps, kept + self.outward_scale, kept)
        kept = torch.where(delta <= -self.eps, kept + self.inward_scale, kept)
        target = before + kept * delta
        _norms.scale_inplace(p, _norms.guarded_ratio(target, after, self.eps, after < self.eps))
