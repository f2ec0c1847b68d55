"""Hooks called around the final in-place weight update (protocol and the no-op default only)."""

from emerging_optimizers_b200.weight_update_hooks.base import HookStateT, NoOpWeightUpdateHook, WeightUpdateHook


__all__ = ["HookStateT", "NoOpWeightUpdateHook", "WeightUpdateHook"]
