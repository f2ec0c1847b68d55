"""Muon for fused QKV projection weights: every logical matrix inside the fused parameter is orthogonalized on
its own.

The reference leaves this to the user: the docstring of its base class
(``emerging_optimizers/orthogonalized_optimizers/orthogonalized_optimizer.py:64-87``) sketches a subclass that
overrides ``orthogonalize``, splits the momentum of a parameter tagged ``is_qkv`` along dim 0, runs
``scaled_orthogonalize_fn`` per piece and concatenates.  This module is that subclass for :class:`Muon`, extended to
the two layouts and the two granularities met in practice:

- layout: ``[Q; K; V]`` stacked once (``num_query_groups=1``), or interleaved per query group as Megatron-Core
  stores it, ``[q_0; k_0; v_0; q_1; k_1; v_1; ...]`` with ``q_g`` holding the query heads of group ``g``;
- granularity: Q, K and V as three whole matrices, or every head as its own ``head_dim x hidden`` matrix
  (``per_head=True``).

Equally shaped pieces are stacked and go through ONE batched Newton-Schulz call, which is where the grouped
small-matrix kernel runs (all iterations of up to hundreds of 128-row heads in a single launch), instead of one call
per piece.
"""

from __future__ import annotations

from typing import Any, Sequence

import torch

from emerging_optimizers_b200.orthogonalized_optimizers.muon import Muon


__all__ = ["SplitQkvMuon"]


class SplitQkvMuon(Muon):
    """:class:`Muon` that orthogonalizes the pieces of fused QKV parameters separately.

    A parameter is treated as fused QKV if it carries a truthy attribute ``is_qkv`` or its parameter group has a
    truthy entry ``is_qkv``; every other parameter takes Muon's normal path.

    Args:
        params: as for Muon.
        *args: positional arguments of Muon.
        qkv_split_shapes: rows of the q, k and v block inside ONE query group, e.g. ``(q_heads_per_group *
            head_dim, head_dim, head_dim)``; with ``num_query_groups=1`` simply the rows of Q, K and V.
        num_query_groups: how many times the ``[q; k; v]`` pattern repeats along dim 0.
        per_head: orthogonalize every ``head_dim``-row block on its own instead of whole Q / K / V.
        head_dim: rows of one head; required with ``per_head``.
        **kwargs: keyword arguments of Muon.

    Raises:
        ValueError: inconsistent split arguments, or (at step time) a fused parameter whose dim 0 is not
            ``num_query_groups * sum(qkv_split_shapes)``.
    """

    def __init__(
        self,
        params: Any,
        *args: Any,
        qkv_split_shapes: Sequence[int],
        num_query_groups: int = 1,
        per_head: bool = False,
        head_dim: int | None = None,
        **kwargs: Any,
    ) -> None:
        split = tuple(int(s) for s in qkv_split_shapes)
        if len(split) != 3 or min(split) <= 0:
            raise ValueError(f"qkv_split_shapes must be three positive row counts, got {tuple(qkv_split_shapes)}")
        if num_query_groups < 1:
            raise ValueError(f"num_query_groups must be at least 1, got {num_query_groups}")
        if per_head:
            if head_dim is None or head_dim <= 0 or any(s % head_dim for s in split):
                raise ValueError(
                    f"per_head needs a head_dim that divides every entry of qkv_split_shapes={split}, got {head_dim}"
                )
        super().__init__(params, *args, **kwargs)
        self.qkv_split_shapes = split
        self.num_query_groups = num_query_groups
        self.per_head = per_head
        self.head_dim = head_dim

    def orthogonalize(self, p: torch.Tensor, grad: torch.Tensor, **kwargs: Any) -> torch.Tensor:
        if not (getattr(p, "is_qkv", False) or kwargs.get("is_qkv", False)):
            return super().orthogonalize(p, grad, **kwargs)
        if grad.ndim != 2:
            raise ValueError("Only 2D parameters are supported.")
        groups, per_group = self.num_query_groups, sum(self.qkv_split_shapes)
        if grad.size(0) != groups * per_group:
            raise ValueError(
                f"fused QKV parameter has {grad.size(0)} rows, expected num_query_groups * sum(qkv_split_shapes) = "
                f"{groups} * {per_group}"
            )
        hidden = grad.size(1)
        blocks = grad.view(groups, per_group, hidden).split(self.qkv_split_shapes, dim=1)  # q, k, v: (G, rows, hidden)

        if self.per_head:
            pieces = [b.reshape(-1, self.head_dim, hidden) for b in blocks]  # (heads, head_dim, hidden)
        else:
            pieces = [b.reshape(1, -1, hidden) for b in blocks]  # (1, G * rows, hidden)

        # One batched call per distinct piece shape (q, k and v heads all share one; whole K and V usually do).
        results: list[torch.Tensor | None] = [None] * len(pieces)
        by_shape: dict[tuple[int, int], list[int]] = {}
        for i, piece in enumerate(pieces):
            by_shape.setdefault((piece.size(1), piece.size(2)), []).append(i)
        for idxs in by_shape.values():
            stack = torch.cat([pieces[i] for i in idxs], dim=0)
            out = self.scaled_orthogonalize_fn(stack if stack.size(0) > 1 else stack[0])
            out = out.reshape(stack.shape)
            start = 0
            for i in idxs:
                n = pieces[i].size(0)
                results[i] = out[start : start + n]
                start += n

        merged = [
            r.reshape(groups, rows, hidden)  # type: ignore[union-attr]
            for r, rows in zip(results, self.qkv_split_shapes)
        ]
        return torch.cat(merged, dim=1).reshape(groups * per_group, hidden)
