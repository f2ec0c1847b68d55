"""MuonHyperball: Muon whose weights stay on a sphere of fixed Frobenius radius.

Same constructor contract and checks as ``emerging_optimizers/orthogonalized_optimizers/muon_hyperball.py:27-95``
of the reference: ``W <- R * normalize(W - lr * R * normalize(update))``.
"""

from typing import Any

import torch

from emerging_optimizers_b200 import registry
from emerging_optimizers_b200.orthogonalized_optimizers import muon
from emerging_optimizers_b200.weight_update_hooks import HyperballHook


__all__ = ["MuonHyperball"]


@registry.register_optimizer("muon_hyperball")
class MuonHyperball(muon.Muon[None]):
    """Muon with a :class:`HyperballHook` installed: the update is rescaled to norm ``hyperball_radius`` before it
    is applied, and the weight is projected back to that norm afterwards.  Experimental.

    Args:
        *args: positional arguments of :class:`~emerging_optimizers_b200.orthogonalized_optimizers.muon.Muon`.
        hyperball_radius: the fixed Frobenius norm; every parameter must already have it (rtol 1e-5).
        hyperball_eps: threshold of a numerical zero in the normalisations.
        **kwargs: keyword arguments of Muon, except ``weight_update_hook``.

    Raises:
        KeyError: ``weight_update_hook`` was passed.
        ValueError: a parameter has (almost) zero norm, or a norm different from ``hyperball_radius``.
    """

    def __init__(self, *args: Any, hyperball_radius: float, hyperball_eps: float = 1e-15, **kwargs: Any) -> None:
        if "weight_update_hook" in kwargs:
            raise KeyError(
                "MuonHyperball does not accept a 'weight_update_hook' argument; "
                "it manages its own HyperballHook internally."
            )
        super().__init__(
            *args, weight_update_hook=HyperballHook(radius=hyperball_radius, eps=hyperball_eps), **kwargs
        )
        self._check_radii(hyperball_radius, hyperball_eps)

    @torch.no_grad()
    def _check_radii(self, radius: float, eps: float) -> None:
        params = [p for group in self.param_groups for p in group["params"]]
        if not params:
            return
        # One host read per device instead of one (or two) per parameter.
        per_device: dict[torch.device, list[torch.Tensor]] = {}
        for p in params:
            per_device.setdefault(p.device, []).append(torch.linalg.vector_norm(p, dtype=torch.float32))
        norms = [n for group in per_device.values() for n in torch.stack(group).tolist()]
        radius = float(torch.tensor(radius, dtype=torch.float32))
        for norm in norms:
            if norm < eps:
                raise ValueError(
                    "MuonHyperball requires all parameters to have non-zero norm. "
                    "Found parameter with almost zero norm."
                )
            if not abs(norm - radius) <= 1e-5 * abs(radius):
                raise ValueError(
                    f"hyperball_radius={radius} was specified but a parameter "
                    f"has Frobenius norm {norm}. Rescale your model parameters to the "
                    f"desired radius before constructing the optimizer."
                )
