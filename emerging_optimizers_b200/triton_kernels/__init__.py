"""bf16 extended SYRK entry points, ``D = alpha * A @ A^T + beta * C``.

The module keeps the reference's name and function signatures (``emerging_optimizers/triton_kernels``:
``syrk.py:335-337, 411-418``, ``batched_syrk.py:237, 266-273``) so callers need no change, but nothing here is
Triton: every function launches the hand-written sm_100a kernel behind ``eo_syrk`` in ``libeo_b200.so``.  That
kernel computes only tiles touching the lower triangle (tcgen05 MMA, fp32 accumulation in tensor memory), applies
``alpha`` / ``beta * C`` in fp32, rounds to bf16 once and writes each element and its mirror image exactly once.

Argument checks raise the same exception types and messages as the reference functions.
"""

from __future__ import annotations

import os

import torch

from emerging_optimizers_b200 import _native


__all__ = ["tsyrk_ex", "tsyrk_ex_small_matrix", "batched_tsyrk_ex", "can_use_batched_tsyrk", "HAS_TRITON_340"]

# Kept under the reference's name: callers test it before using the SYRK path.  Here it states whether the native
# library has been built.
HAS_TRITON_340: bool = os.path.exists(_native.library_path())


def _check_2d_operands(a: torch.Tensor, c: torch.Tensor | None, beta: float) -> None:
    if a.dtype != torch.bfloat16:
        raise TypeError("Input tensor must be bfloat16")
    if a.dim() != 2:
        raise TypeError("Input tensor must be 2D")
    if not (a.is_contiguous() or a.T.is_contiguous()):
        raise TypeError("invalid input tensor layout. a or a.T must be contiguous.")
    n = a.size(0)
    if c is None:
        if beta != 0.0:
            raise RuntimeError("if c is provided, c must be of shape (N, N)")
    else:
        if tuple(c.shape) != (n, n):
            raise RuntimeError("if c is provided, c must be of shape (N, N)")
        if not (c.is_contiguous() or c.T.is_contiguous()):
            raise RuntimeError("if c is provided, c or c.T must be contiguous")


def _check_out(out: torch.Tensor, shape: tuple[int, ...], like: torch.Tensor) -> None:
    if tuple(out.shape) != shape or out.dtype != like.dtype or out.device != like.device:
        raise RuntimeError("out must be same shape/device/dtype as output")
    if not out.is_contiguous():
        raise RuntimeError("out must be contiguous")


def _check_tma_alignment(n: int, k: int) -> None:
    if n % 8 != 0 or k % 8 != 0:
        raise RuntimeError(f"N and K must be multiples of 8 for bf16 TMA alignment, got N={n}, K={k}")


def tsyrk_ex(
    a: torch.Tensor, c: torch.Tensor = None, alpha: float = 1.0, beta: float = 0.0, skip_upper_triangle: bool = False
) -> torch.Tensor:
    """bf16 SYRK of one matrix (cuBLAS-style name: 't' for bf16).

    Args:
        a: ``(N, K)`` bfloat16, ``a`` or ``a.T`` contiguous.
        c: ``None`` or a symmetric ``(N, N)`` bfloat16 tensor (required when ``beta != 0``).
        alpha: scale of the product.
        beta: scale of ``c``.
        skip_upper_triangle: leave the strict upper triangle of the result unwritten.

    Returns:
        A new contiguous ``(N, N)`` bfloat16 tensor.
    """
    return tsyrk_ex_small_matrix(a, c, alpha, beta, skip_upper_triangle)


def tsyrk_ex_small_matrix(
    a: torch.Tensor,
    c: torch.Tensor = None,
    alpha: float = 1.0,
    beta: float = 0.0,
    skip_upper_triangle: bool = False,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Same operation as :func:`tsyrk_ex` with an optional preallocated ``out``.

    The reference keeps a second Triton kernel for small matrices; here one kernel serves every size (its tile
    scheduler is triangular for all of them), so the two functions differ only in the ``out`` argument.
    """
    _check_2d_operands(a, c, beta)
    n, k = a.shape
    if out is None:
        out = torch.empty((n, n), device=a.device, dtype=a.dtype)
    else:
        _check_out(out, (n, n), a)
    _check_tma_alignment(n, k)
    _native.syrk(a, c if beta != 0.0 else None, out, alpha=alpha, beta=beta, skip_upper=skip_upper_triangle)
    return out


def can_use_batched_tsyrk(a: torch.Tensor, c: torch.Tensor | None = None) -> bool:
    """True when :func:`batched_tsyrk_ex` accepts these operands (lets callers choose without catching errors)."""
    if not HAS_TRITON_340 or not a.is_cuda or a.dtype != torch.bfloat16 or a.dim() != 3:
        return False
    if not (a.is_contiguous() or a.mT.is_contiguous()):
        return False
    batch, n, k = a.shape
    if n % 8 != 0 or k % 8 != 0:
        return False
    if c is not None:
        if tuple(c.shape) != (batch, n, n) or c.dtype != a.dtype:
            return False
        if not (c.is_contiguous() or c.mT.is_contiguous()):
            return False
    return True


def batched_tsyrk_ex(
    a: torch.Tensor,
    c: torch.Tensor | None = None,
    alpha: float = 1.0,
    beta: float = 0.0,
    skip_upper_triangle: bool = False,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """Batched bf16 SYRK: ``d[b] = alpha * a[b] @ a[b].mT + beta * c[b]``; stands in for ``torch.baddbmm``.

    Args:
        a: ``(B, N, K)`` bfloat16 with ``a`` or ``a.mT`` contiguous; ``N`` and ``K`` multiples of 8.
        c: ``None`` or ``(B, N, N)`` with every ``c[b]`` symmetric.
        alpha, beta: scales of the product and of ``c``.
        skip_upper_triangle: leave the strict upper triangle of each result unwritten.
        out: optional contiguous ``(B, N, N)`` bfloat16 result tensor.

    Returns:
        ``(B, N, N)`` bfloat16.
    """
    if not HAS_TRITON_340:
        raise RuntimeError("libeo_b200.so has not been built; the batched SYRK kernel is unavailable.")
    if a.dtype != torch.bfloat16:
        raise TypeError("Input tensor must be bfloat16")
    if a.dim() != 3:
        raise TypeError("Input tensor must be 3D of shape (B, N, K)")
    if not (a.is_contiguous() or a.mT.is_contiguous()):
        raise TypeError("invalid input tensor layout. a or a.mT must be contiguous.")
    batch, n, k = a.shape
    _check_tma_alignment(n, k)
    if c is None:
        if beta != 0.0:
            raise RuntimeError("if c is provided, c must be of shape (B, N, N)")
    else:
        if tuple(c.shape) != (batch, n, n):
            raise RuntimeError("if c is provided, c must be of shape (B, N, N)")
        if not (c.is_contiguous() or c.mT.is_contiguous()):
            raise RuntimeError("if c is provided, c or c.mT must be contiguous")
    if out is None:
        out = torch.empty((batch, n, n), device=a.device, dtype=a.dtype)
    else:
        _check_out(out, (batch, n, n), a)
    _native.syrk(a, c if beta != 0.0 else None, out, alpha=alpha, beta=beta, skip_upper=skip_upper_triangle)
    return out
