"""MOP: momentum orthogonalized by an exact polar decomposition (SVD), the non-iterative sibling of Muon.

Same constructor, registry name and arithmetic as ``emerging_optimizers/orthogonalized_optimizers/mop.py:30-107``
of the reference.  Nothing here runs on the Newton-Schulz kernels: the polar factor comes from the library SVD.  The
class exists so that code written against the reference's ``orthogonalized_optimizers`` package finds it.
"""

from typing import Literal

import torch
from torch.optim.optimizer import ParamsT

from emerging_optimizers_b200 import registry
from emerging_optimizers_b200.mixin import WeightDecayT
from emerging_optimizers_b200.orthogonalized_optimizers import muon
from emerging_optimizers_b200.orthogonalized_optimizers.orthogonalized_optimizer import (
    OrthogonalizedOptimizer,
    _args_doc,
)
from emerging_optimizers_b200.utils import FP32MatmulPrecT


__all__ = ["MOP"]


def polar_via_svd(A: torch.Tensor, return_p: bool = False) -> tuple[torch.Tensor, torch.Tensor | None, torch.Tensor]:
    """Polar decomposition ``A = U P`` from the thin SVD ``A = W diag(s) V^H``: ``U = W V^H``, ``P = V diag(s) V^H``.

    Args:
        A: matrix (or batch of matrices) to decompose.
        return_p: also form the positive-semidefinite factor (MOP itself does not need it).

    Returns:
        ``(U, P or None, s)`` with ``s`` the singular values.
    """
    W, s, Vh = torch.linalg.svd(A, full_matrices=False)
    U = W @ Vh
    if not return_p:
        return U, None, s
    return U, Vh.mH @ torch.diag(s) @ Vh, s


@registry.register_optimizer("mop")
class MOP(OrthogonalizedOptimizer):
    """Momentum orthogonalized by polar decomposition.  Experimental, as in the reference.

    Args:
        {_args_doc}
        scale_mode: one of Muon's scale modes, or "nuclear_norm" (default): multiply the polar factor by the sum of
            the singular values of the momentum (arXiv:2505.21799).
        extra_scale_factor: extra multiplier of the update.
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
        fp32_matmul_prec: FP32MatmulPrecT = "highest",
        scale_mode: muon.MuonScaleT | Literal["nuclear_norm"] = "nuclear_norm",
        extra_scale_factor: float = 1.0,
    ) -> None:
        def exact_polar_update(m: torch.Tensor) -> torch.Tensor:
            u, _, s = polar_via_svd(m)
            if scale_mode == "nuclear_norm":
                scale: float | torch.Tensor = s.sum()
            else:
                scale = muon.get_muon_scale_factor(m.size(-2), m.size(-1), mode=scale_mode)
            return u * scale * extra_scale_factor

        super().__init__(
            params,
            lr,
            momentum,
            weight_decay,
            nesterov=nesterov,
            weight_decay_method=weight_decay_method,
            fp32_matmul_prec=fp32_matmul_prec,
            scaled_orthogonalize_fn=exact_polar_update,
        )


MOP.__doc__ = MOP.__doc__.format(_args_doc=_args_doc)  # type: ignore[union-attr]
