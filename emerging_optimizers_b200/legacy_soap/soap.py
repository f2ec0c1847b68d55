"""Kronecker factor statistics ``L <- lerp(L, G G^T)``, ``R <- lerp(R, G^T G)`` on the fp32-accurate SYRK kernel.

Same signature and effect as ``update_kronecker_factors`` of
``emerging_optimizers/legacy_soap/soap.py:296-325`` of the reference, which forms both outer products with library
GEMMs.  Here each is one launch of the lower-triangular tensor-core kernel on the three-plane bf16 split of the
gradient (half the products of a general GEMM, fp32 round-off accuracy), with the exponential moving average done
in the kernel epilogue: ``beta * L + (1 - beta) * G G^T``.  Nothing else of the SOAP / Shampoo optimizers is
provided by this package.
"""

import torch

from emerging_optimizers_b200 import _native


__all__ = ["update_kronecker_factors"]


@torch.no_grad()
def update_kronecker_factors(
    kronecker_factor_list: list[torch.Tensor], grad: torch.Tensor, shampoo_beta: float
) -> None:
    """Update the left and right preconditioner statistics of a 2-D gradient in place.

    Args:
        kronecker_factor_list: ``[L, R]``, fp32 CUDA matrices of shape ``(m, m)`` and ``(n, n)`` for an ``(m, n)``
            gradient; both stay exactly symmetric.
        grad: fp32 CUDA gradient.
        shampoo_beta: weight of the old statistics.
    """
    if grad.dim() != 2 or grad.dtype != torch.float32:
        raise TypeError(f"grad must be a 2-D float32 tensor, got {tuple(grad.shape)} {grad.dtype}")
    _native.require_cuda(grad, "grad")
    g = grad if _native.is_matrix_layout(grad) else grad.contiguous()
    planes = _native.Split3(g)
    for factor, operand in zip(kronecker_factor_list, (planes, planes.mT)):
        side = operand.size(-2)
        if factor.shape != (side, side) or factor.dtype != torch.float32:
            raise ValueError(f"Kronecker factor must be a float32 {side} x {side} matrix, got {tuple(factor.shape)}")
        old = factor if factor.is_contiguous() else factor.contiguous()
        new = torch.empty_like(old)
        _native.syrk(operand, old, new, alpha=1.0 - shampoo_beta, beta=shampoo_beta)
        factor.copy_(new)
