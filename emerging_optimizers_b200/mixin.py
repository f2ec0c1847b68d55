"""Weight-decay variants applied at the top of the optimizer step.

Same four methods and argument meaning as ``emerging_optimizers/mixin.py:21-56`` of the reference.
"""

from typing import Literal

import torch


WeightDecayT = Literal["decoupled", "independent", "l2", "palm"]

_PARAM_SHRINK = {
    # method -> factor f such that p <- p + f(lr, wd) * p
    "decoupled": lambda lr, wd: -wd * lr,
    "independent": lambda lr, wd: -wd,
    "palm": lambda lr, wd: -(wd * lr * lr),
}


class WeightDecayMixin:
    """Adds ``_apply_weight_decay_inplace`` to an optimizer.

    - "decoupled": shrink the parameter by ``lr * weight_decay``
    - "independent": shrink the parameter by ``weight_decay`` (not tied to the learning rate)
    - "l2": add ``weight_decay * p`` to the gradient
    - "palm": shrink the parameter by ``lr^2 * weight_decay``

    The method is read from ``self.weight_decay_method`` and defaults to "l2" when the attribute is absent.
    """

    def _apply_weight_decay_inplace(self, p: torch.Tensor, grad: torch.Tensor, lr: float, weight_decay: float) -> None:
        if weight_decay == 0.0:
            return
        method = getattr(self, "weight_decay_method", "l2")
        if method in _PARAM_SHRINK:
            p.add_(p, alpha=_PARAM_SHRINK[method](lr, weight_decay))
        elif method == "l2":
            grad.add_(p, alpha=weight_decay)
        else:
            raise ValueError(f"Invalid weight decay method: {method}")
