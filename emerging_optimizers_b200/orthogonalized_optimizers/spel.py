"""Spel: spectral steepest descent on the Stiefel manifold.

Same constructor, registry name and arithmetic as ``emerging_optimizers/orthogonalized_optimizers/spel.py:33-129``
of the reference (arXiv:2601.21487): ``x <- msign(x - lr * msign(momentum))``.
"""

import torch
from torch.optim.optimizer import ParamsT

from emerging_optimizers_b200 import registry, utils
from emerging_optimizers_b200.mixin import WeightDecayT
from emerging_optimizers_b200.orthogonalized_optimizers import _consumers
from emerging_optimizers_b200.orthogonalized_optimizers.muon_utils import NSCoeffT
from emerging_optimizers_b200.orthogonalized_optimizers.orthogonalized_optimizer import (
    OrthogonalizedOptimizer,
    _args_doc,
)
from emerging_optimizers_b200.utils import FP32MatmulPrecT


__all__ = ["Spel"]


@registry.register_optimizer("spel")
class Spel(OrthogonalizedOptimizer):
    """Two Newton-Schulz runs per parameter and step: one on the momentum (the descent direction, unscaled) and
    one on the updated weight, which retracts it to (the neighbourhood of) the set of semi-orthogonal matrices.

    Weight decay still matters: ``(1 - lr * wd) x - lr * msign(m)`` is re-orthogonalized as a whole, so the decay
    sets how much the old weight counts against the new direction.  For hidden 2-D weights only.

    Args:
        {_args_doc}
        coefficient_type: Newton-Schulz schedule name, used for both runs.
        num_ns_steps: iterations of each of the two runs (at least 1).
    """

    def __init__(
        self,
        params: ParamsT,
        lr: float = 3e-4,
        momentum: float = 0.95,
        weight_decay: float = 0.1,
        *,
        nesterov: bool = False,
        weight_decay_method: WeightDecayT = "decoupled",
        fp32_matmul_prec: FP32MatmulPrecT = "medium",
        coefficient_type: NSCoeffT = "quintic",
        num_ns_steps: int = 5,
    ) -> None:
        _consumers.check_steps(num_ns_steps)

        def polar_factor(x: torch.Tensor) -> torch.Tensor:
            return _consumers.msign(x, num_ns_steps, coefficient_type)

        super().__init__(
            params,
            lr,
            momentum,
            weight_decay,
            nesterov=nesterov,
            weight_decay_method=weight_decay_method,
            fp32_matmul_prec=fp32_matmul_prec,
            scaled_orthogonalize_fn=polar_factor,
        )

    def post_weight_update_fn_inplace(self, p: torch.Tensor) -> None:
        """The outer ``msign``: overwrite the freshly updated weight with its polar factor."""
        with utils.fp32_matmul_precision(self.fp32_matmul_prec):
            retracted = self.scaled_orthogonalize_fn(p)
        p.copy_(retracted)


Spel.__doc__ = Spel.__doc__.format(_args_doc=_args_doc)  # type: ignore[union-attr]
