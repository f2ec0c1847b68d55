"""Clipping of singular values without an SVD, through matrix sign functions computed by Newton-Schulz.

Same functions and arithmetic as
``emerging_optimizers/orthogonalized_optimizers/spectral_clipping_utils.py:23-98`` of the reference (after
https://leloykun.github.io/ponder/spectral-clipping/).  Every matrix sign is an 8-step "polar_express" run of
:func:`~emerging_optimizers_b200.orthogonalized_optimizers.muon_utils.newton_schulz`, at the ambient fp32 matmul
precision.
"""

import torch

from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils


__all__ = ["spectral_hardcap", "spectral_clip"]


def _msign(x: torch.Tensor) -> torch.Tensor:
    return muon_utils.newton_schulz(x, steps=8, coefficient_type="polar_express")


def _wide(x: torch.Tensor) -> tuple[torch.Tensor, bool]:
    """The matrix in the orientation with no more rows than columns, and whether that took a transpose."""
    tall = x.shape[0] > x.shape[1]
    return (x.T if tall else x), tall


def spectral_clip(X: torch.Tensor, sigma_min: float = -1.0, sigma_max: float = 1.0) -> torch.Tensor:
    r"""Clip the singular values of ``X`` to ``[sigma_min, sigma_max]``, keeping its singular vectors.

    Scalar clipping is :math:`\tfrac12\,(lo + hi + (lo - x)\,\mathrm{sign}(lo - x) - (hi - x)\,\mathrm{sign}(hi -
    x))`; applied to singular values it becomes, with :math:`O = \mathrm{msign}(X)`,
    :math:`\tfrac12\,[(lo + hi)\,O + \sum_{s} \pm\,\mathrm{msign}(sI - O X^\top)\,(sO - X)]`.

    Args:
        X: 2-D fp32 tensor.
        sigma_min: lower bound of the singular values.
        sigma_max: upper bound of the singular values.

    Returns:
        The clipped matrix, shaped like ``X``.
    """
    X, tall = _wide(X)
    O = _msign(X)
    eye = torch.eye(X.shape[0], device=X.device, dtype=X.dtype)
    acc = (sigma_min + sigma_max) * O
    for bound, weight in ((sigma_min, 1), (sigma_max, -1)):
        left = torch.addmm(bound * eye, O, X.T, beta=1.0, alpha=-1.0)
        right = torch.add(bound * O, X, alpha=-1)
        acc = torch.addmm(acc, _msign(left), right, alpha=weight)
    acc = acc * 0.5
    return acc.T if tall else acc


def spectral_hardcap(X: torch.Tensor, beta: float = 1.0) -> torch.Tensor:
    r"""Cap the singular values of ``X`` at ``beta`` from above (:math:`\min(\sigma, \beta)`), no lower bound.

    With :math:`O = \mathrm{msign}(X)` and :math:`D = \beta O - X`:
    :math:`\tfrac12\,[\beta O + X - D\,\mathrm{msign}(D)^\top O]`.

    Args:
        X: 2-D fp32 tensor.
        beta: upper bound of the singular values.

    Returns:
        The capped matrix, shaped like ``X``.
    """
    X, tall = _wide(X)
    O = _msign(X)
    D = torch.add(beta * O, X, alpha=-1)
    acc = torch.add(beta * O, X)
    acc = torch.addmm(acc, D, torch.mm(_msign(D).T, O), alpha=-1)
    acc = acc * 0.5
    return acc.T if tall else acc


def spectral_clipped_weight_decay(X: torch.Tensor, beta: float = 1.0, c: float = 0.5) -> torch.Tensor:
    """Spectral analogue of decoupled weight decay: ``(1 - c) X + c * spectral_hardcap(X, beta)``.

    Args:
        X: 2-D fp32 tensor.
        beta: upper bound of the singular values in the hard-capped term.
        c: mixing weight of the hard-capped term.
    """
    return torch.add((1 - c) * X, spectral_hardcap(X, beta), alpha=c)
