"""Hook that gives the update the Frobenius norm of the weight it is applied to.

Behaviour of ``emerging_optimizers/weight_update_hooks/relative_update.py:22-60`` of the reference: the learning
rate then is the relative size of the step.  The weight itself is not projected afterwards.
"""

import torch

from emerging_optimizers_b200.weight_update_hooks import _norms


__all__ = ["RelativeUpdateHook"]


class RelativeUpdateHook:
    """``update <- |p| / |update| * update`` before the weight update; nothing after it.

    If either norm is below ``eps`` the update becomes exactly zero.
    """

    def __init__(self, eps: float = 1e-15) -> None:
        _norms.check_eps(eps, finite=False)
        self.eps = eps

    def pre_weight_update_inplace(self, p: torch.Tensor, update: torch.Tensor) -> None:
        w, u = _norms.fro_norm(p), _norms.fro_norm(update)
        _norms.scale_inplace(update, _norms.guarded_ratio(w, u, self.eps, (w < self.eps) | (u < self.eps)))
        return None

    def post_weight_update_inplace(self, p: torch.Tensor, pre_update_state: None) -> None:
        return None
