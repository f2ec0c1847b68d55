"""Scion: stochastic conditional descent with operator norms, spectral-norm LMO for hidden 2-D weights.

Same constructor, registry name and arithmetic as ``emerging_optimizers/orthogonalized_optimizers/scion.py:31-106``
of the reference (arXiv:2502.07529).
"""

import torch
from absl import logging
from torch.optim.optimizer import ParamsT

from emerging_optimizers_b200 import registry
from emerging_optimizers_b200.orthogonalized_optimizers import _consumers
from emerging_optimizers_b200.orthogonalized_optimizers.muon import get_muon_scale_factor
from emerging_optimizers_b200.orthogonalized_optimizers.muon_utils import NSCoeffT
from emerging_optimizers_b200.orthogonalized_optimizers.orthogonalized_optimizer import OrthogonalizedOptimizer
from emerging_optimizers_b200.utils import FP32MatmulPrecT


__all__ = ["Scion"]


@registry.register_optimizer("scion")
class Scion(OrthogonalizedOptimizer):
    """Frank-Wolfe view of weight decay: ``p <- (1 - lr) p - lr * radius * sqrt(out/in) * msign(m)``.

    The base class is configured with decoupled weight decay of strength 1 (the ``(1 - lr) p`` term), no Nesterov
    momentum, and an update that is the Newton-Schulz polar factor of the momentum scaled to unit RMS->RMS operator
    norm times ``spectral_radius``.  For hidden 2-D weights only; other layers need the LMO of their own norm.

    Args:
        params: iterable of parameters or of dicts defining parameter groups.
        lr: step size of the conditional-gradient step.
        momentum: EMA coefficient of the momentum buffer.
        fp32_matmul_prec: fp32 matmul precision while orthogonalizing ("medium" selects the bf16 kernels).
        coefficient_type: Newton-Schulz schedule name.
        num_ns_steps: number of Newton-Schulz iterations (at least 1).
        spectral_radius: radius of the spectral-norm ball the LMO is scaled to.
    """

    def __init__(
        self,
        params: ParamsT,
        lr: float = 3e-4,
        momentum: float = 0.95,
        *,
        fp32_matmul_prec: FP32MatmulPrecT = "medium",
        coefficient_type: NSCoeffT = "quintic",
        num_ns_steps: int = 5,
        spectral_radius: float = 1.0,
    ) -> None:
        _consumers.check_steps(num_ns_steps)
        logging.info("Scion fixes weight_decay=1 (decoupled) and nesterov=False.")

        def lmo(momentum_buf: torch.Tensor) -> torch.Tensor:
            rows, cols = momentum_buf.size(-2), momentum_buf.size(-1)
            direction = _consumers.msign(momentum_buf, num_ns_steps, coefficient_type)
            return direction * get_muon_scale_factor(rows, cols, mode="unit_rms_norm") * spectral_radius

        super().__init__(
            params,
            lr,
            momentum,
            1,
            nesterov=False,
            weight_decay_method="decoupled",
            fp32_matmul_prec=fp32_matmul_prec,
            scaled_orthogonalize_fn=lmo,
        )
