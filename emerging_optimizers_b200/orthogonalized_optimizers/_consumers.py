"""What the optimizers built on top of Newton-Schulz share: the call into the driver.

The reference's Scion, Spel and AdaptiveMuon pass ``use_syrk=False`` to ``muon_utils.newton_schulz``
(``scion.py:91-93``, ``spel.py:96-101``, ``adaptive_muon.py:98-103``).  They do the same here unless
:data:`USE_SYRK` is switched on, in which case the symmetric products of their iterations run on the
lower-triangular kernel (bf16 path only; the driver itself falls back for shapes the kernel cannot address).
"""

import torch

from emerging_optimizers_b200.orthogonalized_optimizers import muon_utils


# Process-wide switch; off by default so that the optimizers compute exactly what the reference's compute.
USE_SYRK = False


def check_steps(num_ns_steps: int, minimum: int = 1) -> None:
    if num_ns_steps < minimum:
        if minimum == 1:
            raise ValueError(f"num_ns_steps must be at least 1, got {num_ns_steps}")
        raise ValueError(f"num_ns_steps must be positive, got {num_ns_steps}")


def msign(x: torch.Tensor, steps: int, coefficient_type: str) -> torch.Tensor:
    """Approximate matrix sign (polar factor) of ``x``: the driver is looked up at call time."""
    return muon_utils.newton_schulz(x, steps=steps, coefficient_type=coefficient_type, use_syrk=USE_SYRK)
