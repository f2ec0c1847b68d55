"""Structural contract for code that wraps ``p.add_(update, alpha=-lr)``.

Same protocol as ``emerging_optimizers/weight_update_hooks/base.py:26-59`` of the reference: the optimizer calls
``pre_weight_update_inplace(p, update)`` right before the update and hands its return value to
``post_weight_update_inplace(p, state)`` right after it.
"""

from typing import Protocol, TypeVar

import torch


__all__ = ["NoOpWeightUpdateHook", "WeightUpdateHook", "HookStateT"]

HookStateT = TypeVar("HookStateT", bound="torch.Tensor | None")


class WeightUpdateHook(Protocol[HookStateT]):
    def pre_weight_update_inplace(self, p: torch.Tensor, update: torch.Tensor) -> HookStateT:
        """Runs immediately before the weight update; may change ``p`` or ``update`` in place."""

    def post_weight_update_inplace(self, p: torch.Tensor, pre_update_state: HookStateT) -> None:
        """Runs after the weight update and the optimizer's own post-update function."""


class NoOpWeightUpdateHook:
    """Default: leave the update alone."""

    def pre_weight_update_inplace(self, p: torch.Tensor, update: torch.Tensor) -> None:
        return None

    def post_weight_update_inplace(self, p: torch.Tensor, pre_update_state: None) -> None:
        return None
