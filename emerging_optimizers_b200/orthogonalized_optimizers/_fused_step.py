"""Grouped, fused execution of the Muon update for many parameter matrices at once.

The per-parameter loop of the optimizer step (``orthogonalized_optimizer.py:164-212`` in the reference) issues,
for every matrix, a handful of elementwise passes and fifteen small GEMM launches.  For a model-sized parameter set
that is hundreds of launches on matrices too small to fill 148 SMs (k/v projections, per-head blocks).  This module
restructures the same arithmetic:

1. per matrix, two fused elementwise kernels: momentum update + sum of squares, then normalise + bf16 cast, the
   latter writing straight into a slot of a stacked ``(B, rows, cols)`` bf16 buffer (no fp32 temporary);
2. per group of equally shaped matrices, one *batched* Newton-Schulz run: every product of every iteration is a
   single launch of the tensor-core kernel over the whole stack (the grouped launcher for split-QKV / per-head /
   k-v sized matrices);
3. the result stays bf16 (the bf16 path's result is bf16-valued anyway) and is consumed by the fused
   ``p <- (p + shrink p) - lr ((u scale) extra)`` kernel, locally or after an all-gather.
"""

from __future__ import annotations

from typing import Sequence

import torch

from emerging_optimizers_b200 import _native
from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils


# Upper bound on the bf16 bytes of one stacked batch (keeps A, B and the two iterates of a batch near 3 GiB).
MAX_BATCH_BYTES = 1 << 30


def eligible(p: torch.Tensor, g: torch.Tensor | None) -> bool:
    """True if the fused kernels can take this parameter: 2-D fp32 CUDA, contiguous, gradient likewise."""
    return (
        g is not None
        and p.is_cuda
        and p.ndim == 2
        and p.dtype == torch.float32
        and g.dtype == torch.float32
        and p.is_contiguous()
        and g.is_contiguous()
        and p.data_ptr() % 16 == 0
        and g.data_ptr() % 16 == 0
    )


def plan_batches(shapes: Sequence[tuple[int, int]], max_batch_bytes: int = MAX_BATCH_BYTES) -> list[list[int]]:
    """Group indices of equally shaped matrices, in order of first appearance, into batches of bounded size."""
    by_shape: dict[tuple[int, int], list[int]] = {}
    for i, s in enumerate(shapes):
        by_shape.setdefault(tuple(s), []).append(i)
    batches: list[list[int]] = []
    for shape, idx in by_shape.items():
        per = max(1, max_batch_bytes // max(1, 2 * shape[0] * shape[1]))
        for k in range(0, len(idx), per):
            batches.append(idx[k : k + per])
    return batches


def orthogonalized_updates(
    params: Sequence[torch.Tensor],
    grads: Sequence[torch.Tensor],
    momenta: Sequence[torch.Tensor],
    *,
    momentum: float,
    nesterov: bool,
    l2_weight_decay: float,
    steps: int,
    coefficient_type: str,
    use_syrk: bool,
    eps: float = 1e-15,
    max_batch_bytes: int = MAX_BATCH_BYTES,
) -> list[torch.Tensor]:
    """Momentum update (in place on ``momenta``) and bf16 Newton-Schulz for every matrix; returns, per matrix, the
    unscaled orthogonalized update as a contiguous bf16 tensor of the parameter's shape.

    All tensors must satisfy :func:`eligible`.  The arithmetic per matrix is that of
    ``newton_schulz(lerp(...), steps, coefficient_type, use_syrk=use_syrk)`` at "medium" precision.
    """
    if coefficient_type in muon_utils._COEFFICIENT_SETS:
        sets = muon_utils._COEFFICIENT_SETS[coefficient_type]
    else:
        raise ValueError(f"Invalid coefficient type: {coefficient_type}")
    if coefficient_type == "cubic5" and steps != len(sets):
        raise ValueError(f"cubic5 is a fixed {len(sets)}-step schedule; got steps={steps}.")
    mode = "repeat_last" if coefficient_type in muon_utils._REPEAT_LAST_TYPES else "cycle"
    schedule = list(muon_utils.get_coefficient_iterator(steps, sets, mode=mode))

    out: list[torch.Tensor | None] = [None] * len(params)
    syrk_ok = use_syrk
    for batch in plan_batches([tuple(p.shape) for p in params], max_batch_bytes):
        rows, cols = params[batch[0]].shape
        dev = params[batch[0]].device
        stack = torch.empty((len(batch), rows, cols), dtype=torch.bfloat16, device=dev)
        for slot, i in enumerate(batch):
            ss = _native.muon_momentum(grads[i], momenta[i], params[i], momentum, nesterov, l2_weight_decay)
            _native.muon_normalize(
                grads[i], momenta[i], params[i], momentum, nesterov, l2_weight_decay, ss, eps, stack[slot]
            )
        # Iterate on the wide orientation; a tall matrix is used through its transposed view (no copy).
        X = stack.mT if rows > cols else stack
        syrk = syrk_ok and rows % 8 == 0 and cols % 8 == 0
        for a, b, c in schedule:
            X = muon_utils._ns_step(X, a, b, c, None, use_syrk=syrk)
        X = X.mT if rows > cols else X
        if not X.is_contiguous():
            X = X.contiguous()
        for slot, i in enumerate(batch):
            out[i] = X[slot]
    return out  # type: ignore[return-value]
