"""Precision switch and process-group helpers used by the orthogonalization path.

Mirrors ``emerging_optimizers/utils/__init__.py:25-54`` of the reference (names and behaviour).
"""

from contextlib import contextmanager
from typing import Generator, Literal

import torch


__all__ = ["fp32_matmul_precision", "FP32MatmulPrecT", "get_pg_size", "get_pg_rank"]

FP32MatmulPrecT = Literal["highest", "high", "medium"]


@contextmanager
def fp32_matmul_precision(precision: FP32MatmulPrecT = "highest") -> Generator[None, None, None]:
    """Set ``torch.set_float32_matmul_precision`` inside the block and put the old value back after it.

    The Newton-Schulz driver reads this ambient setting to choose between the bf16 kernels ("medium") and the
    fp32-accurate ones, exactly as the reference does (``muon_utils.py:245``).
    """
    saved = torch.get_float32_matmul_precision()
    torch.set_float32_matmul_precision(precision)
    try:
        yield
    finally:
        torch.set_float32_matmul_precision(saved)


def get_pg_size(group: "torch.distributed.ProcessGroup | None" = None) -> int:
    """World size of ``group``; 1 when torch.distributed is not initialised or no group is given."""
    if group is None or not torch.distributed.is_initialized():
        return 1
    return group.size()


def get_pg_rank(group: "torch.distributed.ProcessGroup | None" = None) -> int:
    """Rank inside ``group``; 0 when torch.distributed is not initialised or no group is given."""
    if group is None or not torch.distributed.is_initialized():
        return 0
    return group.rank()
