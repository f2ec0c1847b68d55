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

# Batches (groups of equally shaped matrices) are issued round-robin on this many CUDA streams.  Every product of a
# batch is a persistent launch whose last wave leaves SMs idle (a k/v-sized group of a sharded model has fewer tiles
# than the GPU has SMs); with a second, independent chain of launches in flight those SMs pick up the other chain's
# CTAs, and the tile scheduler of the kernels shares the machine between the two.  Results do not depend on it.
# 1 issues everything on the caller's stream.
NS_STREAMS = 2

_side_streams: dict[tuple, list] = {}


def _streams(device: torch.device, n: int) -> list:
    key = (device.index, n)
    if key not in _side_streams:
        _side_streams[key] = [torch.cuda.Stream(device=device) for _ in range(n)]
    return _side_streams[key]


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


def plan_batches(
    shapes: Sequence[tuple[int, int]], max_batch_bytes: int = MAX_BATCH_BYTES, devices: Sequence | None = None
) -> list[list[int]]:
    """Group indices of equally shaped matrices (on the same device), in order of first appearance, into batches of
    bounded size."""
    by_shape: dict[tuple, list[int]] = {}
    for i, s in enumerate(shapes):
        key = (tuple(s), None if devices is None else devices[i])
        by_shape.setdefault(key, []).append(i)
    batches: list[list[int]] = []
    for (shape, _), idx in by_shape.items():
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
    batches = plan_batches([tuple(p.shape) for p in params], max_batch_bytes, [p.device for p in params])

    def run(batch: list[int]) -> None:
        rows, cols = params[batch[0]].shape
        dev = params[batch[0]].device
        # Row stride padded to 16 bytes so that TMA can address shapes like 40 x 24 too.
        ld = (cols + 7) // 8 * 8
        slot = (rows * ld + 7) // 8 * 8
        gs, ms, ps = [grads[i] for i in batch], [momenta[i] for i in batch], [params[i] for i in batch]
        stack = torch.empty((len(batch), slot), dtype=torch.bfloat16, device=dev)
        # Large matrices skip the normalisation pass (muon_utils.FOLD_NORMALIZATION_MIN_NUMEL): the momentum kernel
        # writes the un-normalised bf16 update in its one pass and the iteration divides in its first two epilogues.
        defer = ld == cols and muon_utils._defer_normalization(rows, cols, len(schedule))
        scales = torch.empty((len(batch), 2), dtype=torch.float32, device=dev) if defer else None
        if ld == cols:
            _native.muon_prepare_batch(gs, ms, ps, momentum, nesterov, l2_weight_decay, eps, stack, scales)
            X = stack[:, : rows * cols].unflatten(1, (rows, cols))
        else:
            dense = torch.empty((len(batch), (rows * cols + 7) // 8 * 8), dtype=torch.bfloat16, device=dev)
            _native.muon_prepare_batch(gs, ms, ps, momentum, nesterov, l2_weight_decay, eps, dense)
            X = stack[:, : rows * ld].unflatten(1, (rows, ld))[:, :, :cols]
            X.copy_(dense[:, : rows * cols].unflatten(1, (rows, cols)))
        if schedule:
            X = _native.newton_schulz_bf16(X, schedule, use_syrk, scales=scales)
        elif not X.is_contiguous():
            X = X.contiguous()
        for k, i in enumerate(batch):
            out[i] = X[k]

    one_device = len({p.device for p in params}) == 1
    if NS_STREAMS <= 1 or len(batches) < 2 or not one_device or not params[0].is_cuda:
        for batch in batches:
            run(batch)
        return out  # type: ignore[return-value]

    dev = params[0].device
    cur = torch.cuda.current_stream(dev)
    streams = _streams(dev, min(NS_STREAMS, len(batches)))
    fork = torch.cuda.Event()
    fork.record(cur)
    for s in streams:
        s.wait_event(fork)
    for k, batch in enumerate(batches):
        with torch.cuda.stream(streams[k % len(streams)]):
            run(batch)
    for s in streams:
        cur.wait_stream(s)
    for t in out:
        t.record_stream(cur)  # allocated on a side stream, consumed on the caller's
    return out  # type: ignore[return-value]
