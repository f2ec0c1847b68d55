"""Hooks called around the final in-place weight update: the protocol, the no-op default and three norm-control
hooks (fixed radius, relative step size, radial brake)."""

from emerging_optimizers_b200.weight_update_hooks.base import HookStateT, NoOpWeightUpdateHook, WeightUpdateHook
from emerging_optimizers_b200.weight_update_hooks.hyperball import HyperballHook
from emerging_optimizers_b200.weight_update_hooks.radial_brake import RadialBrakeHook
from emerging_optimizers_b200.weight_update_hooks.relative_update import RelativeUpdateHook


__all__ = [
    "HookStateT",
    "HyperballHook",
    "NoOpWeightUpdateHook",
    "RadialBrakeHook",
    "RelativeUpdateHook",
    "WeightUpdateHook",
]
