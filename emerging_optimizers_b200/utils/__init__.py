"""Precision switch and process-group helpers used by the orthogonalization path.

Same public names and behaviour as ``emerging_optimizers/utils/__init__.py:25-54`` of the reference.
"""

from __future__ import annotations

from typing import Literal

import torch


__all__ = ["fp32_matmul_precision", "FP32MatmulPrecT", "get_pg_size", "get_pg_rank"]

FP32MatmulPrecT = Literal["highest", "high", "medium"]


class fp32_matmul_precision:  # noqa: N801 - used as ``with fp32_matmul_precision("medium"):``
    """Switch ``torch.set_float32_matmul_precision`` for the duration of a ``with`` block.

    The Newton-Schulz driver reads this ambient setting to choose its arithmetic, exactly as the reference does
    (``muon_utils.py:245`` there): "medium" selects the bf16 tensor-core kernels, "high" / "highest" the
    fp32-accurate split-bf16 products.  The previous value comes back on exit, also when the block raises.
    """

    def __init__(self, precision: FP32MatmulPrecT = "highest") -> None:
        self.precision = precision
        self._outer: str | None = None

    def __enter__(self) -> None:
        self._outer = torch.get_float32_matmul_precision()
        torch.set_float32_matmul_precision(self.precision)

    def __exit__(self, exc_type, exc, tb) -> bool:
        torch.set_float32_matmul_precision(self._outer)
        return False


def _group_or_none(group: "torch.distributed.ProcessGroup | None"):
    """``group`` if it can be queried (torch.distributed initialised and a group given), else ``None``."""
    if group is not None and torch.distributed.is_available() and torch.distributed.is_initialized():
        return group
    return None


def get_pg_size(group: "torch.distributed.ProcessGroup | None" = None) -> int:
    """Number of ranks in ``group``; 1 for a single process."""
    g = _group_or_none(group)
    return 1 if g is None else g.size()


def get_pg_rank(group: "torch.distributed.ProcessGroup | None" = None) -> int:
    """This process's rank in ``group``; 0 for a single process."""
    g = _group_or_none(group)
    return 0 if g is None else g.rank()
