"""PolarGrad: steepest descent w.r.t. the spectral norm, the polar factor scaled by the nuclear norm.

Same public names, signatures and arithmetic as
``emerging_optimizers/orthogonalized_optimizers/polargrad.py:34-204`` of the reference (arXiv:2505.21799).
"""

from typing import Literal

import torch
from absl import logging
from torch.optim.optimizer import ParamsT

from emerging_optimizers_b200 import registry
from emerging_optimizers_b200.mixin import WeightDecayT
from emerging_optimizers_b200.orthogonalized_optimizers import _consumers, muon_utils
from emerging_optimizers_b200.orthogonalized_optimizers.muon_utils import NSCoeffT
from emerging_optimizers_b200.orthogonalized_optimizers.orthogonalized_optimizer import (
    OrthogonalizedOptimizer,
    _args_doc,
)
from emerging_optimizers_b200.utils import FP32MatmulPrecT


__all__ = ["PolarGrad", "left_polargrad_orth_fn", "one_sided_polargrad_orth_fn", "right_polargrad_orth_fn"]


@registry.register_optimizer("polargrad")
class PolarGrad(OrthogonalizedOptimizer):
    """Update ``= <U, M> * U * extra_scale_factor`` with ``U`` the Newton-Schulz polar factor of the momentum
    ``M``; ``<U, M>`` estimates the nuclear norm of ``M``.  Decoupled weight decay by default, fp32 products by
    default ("highest").  For hidden 2-D weights only.

    Args:
        {_args_doc}
        coefficient_type: Newton-Schulz schedule name.
        num_ns_steps: number of Newton-Schulz iterations; 0 is accepted (the update then is the normalised
            momentum times its inner product with the momentum).
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
        coefficient_type: NSCoeffT = "quintic",
        num_ns_steps: int = 5,
        extra_scale_factor: float = 1.0,
    ) -> None:
        _consumers.check_steps(num_ns_steps, minimum=0)

        def polar_times_nuclear(m: torch.Tensor) -> torch.Tensor:
            # The reference leaves use_syrk at the driver's default here (polargrad.py:91-95).
            u = muon_utils.newton_schulz(m, steps=num_ns_steps, coefficient_type=coefficient_type)
            nuclear = (u * m).sum()
            return u * nuclear * extra_scale_factor

        super().__init__(
            params,
            lr,
            momentum,
            nesterov=nesterov,
            weight_decay=weight_decay,
            weight_decay_method=weight_decay_method,
            fp32_matmul_prec=fp32_matmul_prec,
            scaled_orthogonalize_fn=polar_times_nuclear,
        )


PolarGrad.__doc__ = PolarGrad.__doc__.format(_args_doc=_args_doc)  # type: ignore[union-attr]


def _eigh_descending(sym: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Eigen-decomposition of a symmetric matrix, eigenvalues descending; retried in fp64 if the fp32 solver fails
    (the policy of ``emerging_optimizers/utils/eig.py:29-66`` of the reference)."""
    try:
        w, v = torch.linalg.eigh(sym)
    except (torch.linalg.LinAlgError, RuntimeError) as err:
        logging.warning("Falling back to double precision: %s", err)
        w, v = torch.linalg.eigh(sym.to(torch.float64))
        w, v = w.to(sym.dtype), v.to(sym.dtype)
    return w.flip(-1), v.flip(-1)


def one_sided_polargrad_orth_fn(
    grad: torch.Tensor,
    *,
    side: Literal["left", "right"],
    alpha: float = 1.0,
    center_rows: bool = False,
    eps: float = 1e-15,
    extra_scale_factor: float = 1.0,
) -> torch.Tensor:
    r"""Exact one-sided polar orthogonalization through an eigen-decomposition of the (small) Gram matrix.

    ``side="left"``: :math:`u = (G G^\top)^{-1/2} G` (wide matrices, e.g. a router weight);
    ``side="right"``: :math:`u = G (G^\top G)^{-1/2}` (tall matrices, e.g. an embedding).  The update is
    :math:`\lVert G\rVert_*^{\alpha}\, u` times ``extra_scale_factor``.

    Args:
        grad: matrix to orthogonalize (any float dtype; the work is done in fp32).
        side: which Gram matrix to invert.
        alpha: exponent of the nuclear norm.
        center_rows: subtract the mean over rows (``dim=0``) from input and output.
        eps: floor of the Gram eigenvalues.
        extra_scale_factor: extra multiplier.

    Returns:
        The update, shaped and typed like ``grad``.

    Raises:
        ValueError: ``side`` is neither "left" nor "right".
    """
    if side not in ("left", "right"):
        raise ValueError(f"side must be 'left' or 'right', got {side!r}")
    left = side == "left"

    g = grad.to(torch.float32)
    if center_rows:
        g = g - g.mean(dim=0, keepdim=True)
    gram = g @ g.mT if left else g.mT @ g

    lam, vec = _eigh_descending(gram)
    lam.clamp_min_(eps)
    # Directions whose eigenvalue is within round-off of zero carry no information: drop them from the inverse.
    negligible = lam.amax() * gram.shape[-1] * torch.finfo(g.dtype).eps
    inv_sqrt = torch.where(lam > negligible, lam.rsqrt(), torch.zeros_like(lam))
    root_inv = (vec * inv_sqrt.unsqueeze(-2)) @ vec.mT

    u = root_inv @ g if left else g @ root_inv
    out = u * lam.sqrt().sum().pow(alpha) * extra_scale_factor
    if center_rows:
        out = out - out.mean(dim=0, keepdim=True)
    return out.to(grad.dtype)


def right_polargrad_orth_fn(
    grad: torch.Tensor,
    *,
    alpha: float = 1.0,
    center_rows: bool = False,
    eps: float = 1e-15,
    extra_scale_factor: float = 1.0,
) -> torch.Tensor:
    """:func:`one_sided_polargrad_orth_fn` with ``side="right"`` (tall matrices)."""
    return one_sided_polargrad_orth_fn(
        grad, side="right", alpha=alpha, center_rows=center_rows, eps=eps, extra_scale_factor=extra_scale_factor
    )


def left_polargrad_orth_fn(
    grad: torch.Tensor,
    *,
    alpha: float = 1.0,
    center_rows: bool = False,
    eps: float = 1e-15,
    extra_scale_factor: float = 1.0,
) -> torch.Tensor:
    """:func:`one_sided_polargrad_orth_fn` with ``side="left"`` (wide matrices)."""
    return one_sided_polargrad_orth_fn(
        grad, side="left", alpha=alpha, center_rows=center_rows, eps=eps, extra_scale_factor=extra_scale_factor
    )
