"""CPU restatement of the reference's Newton-Schulz driver with torch CPU operators.  TEST INFRASTRUCTURE ONLY.

``ns_oracle.py`` models the bf16 path with fp32 numpy matmuls on bf16-rounded operands, which is the right
arithmetic but not the speed of the reference on a CPU: there the iterate is a ``torch.bfloat16`` tensor and every
product is a bf16 ``torch.matmul`` / ``torch.addmm`` (oneDNN / MKL kernels, all cores).  This file restates the same
driver with exactly those operators, so that the timed CPU baseline of ``bench.py`` measures what the reference's
own CPU path costs.  Used by ``bench.py`` (``cpu_baseline`` and ``--impl reference``) and checked against the
reference-generated golden vectors by ``tests/test_oracle_golden.py``; nothing in the shipped package imports it.

Follows emerging_optimizers/orthogonalized_optimizers/muon_utils.py:149-274 (driver) and :348-378 / :381-411 (step).
"""

from __future__ import annotations

import torch

from oracle import ns_oracle


def newton_schulz_step(X: torch.Tensor, a: float, b: float, c: float) -> torch.Tensor:
    """muon_utils.py:370-377 (2-D) and :403-410 (batched): the three products in X's dtype."""
    A = X @ X.mT
    if c != 0.0:
        B = torch.baddbmm(A, A, A, alpha=c, beta=b) if X.ndim == 3 else torch.addmm(A, A, A, alpha=c, beta=b)
        return torch.baddbmm(X, B, X, alpha=1.0, beta=a) if X.ndim == 3 else torch.addmm(X, B, X, alpha=1.0, beta=a)
    return torch.baddbmm(X, A, X, alpha=b, beta=a) if X.ndim == 3 else torch.addmm(X, A, X, alpha=b, beta=a)


def newton_schulz(
    x: torch.Tensor, steps: int, coefficient_type: str = "quintic", precision: str = "medium", eps: float = 1e-15
) -> torch.Tensor:
    """muon_utils.py:199-274 for a CPU tensor: wide transpose, Frobenius normalisation, bf16 cast under "medium",
    ``steps`` iterations, fp32 result in the input's orientation."""
    if x.ndim < 2 or x.ndim > 3:
        raise TypeError(f"Input tensor x must be 2d or 3d (batched 2d), got {x.ndim}d")
    if x.dtype != torch.float32:
        raise TypeError(f"Input tensor x must be in float32, got {x.dtype}")
    transpose = x.size(-2) > x.size(-1)
    if transpose:
        x = x.mT
    X = x / x.norm(dim=(-2, -1), keepdim=True).clamp_min(eps)
    if precision == "medium":
        X = X.to(torch.bfloat16)
    for a, b, c in ns_oracle.coefficient_schedule(steps, coefficient_type):
        X = newton_schulz_step(X, a, b, c)
    X = X.to(torch.float32)
    return X.mT if transpose else X
