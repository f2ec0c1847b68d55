"""Orthogonalized optimizers on the sm_100a Newton-Schulz kernels: ``OrthogonalizedOptimizer``, ``Muon`` and the
``muon_utils`` driver functions."""

from emerging_optimizers_b200.orthogonalized_optimizers.muon import *  # noqa: F401,F403
from emerging_optimizers_b200.orthogonalized_optimizers.orthogonalized_optimizer import *  # noqa: F401,F403
