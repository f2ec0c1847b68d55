"""Orthogonalized optimizers on the sm_100a Newton-Schulz kernels: the ``OrthogonalizedOptimizer`` base, ``Muon``
and the optimizers derived from them (``AdaptiveMuon``, ``MuonHyperball``, ``PolarGrad``, ``Scion``, ``Spel``,
``SplitQkvMuon``), ``MOP`` (exact polar factor from a library SVD), the ``muon_utils`` driver functions and the
``spectral_clipping_utils`` functions."""

from emerging_optimizers_b200.orthogonalized_optimizers.adaptive_muon import *  # noqa: F401,F403
from emerging_optimizers_b200.orthogonalized_optimizers.mop import *  # noqa: F401,F403
from emerging_optimizers_b200.orthogonalized_optimizers.muon import *  # noqa: F401,F403
from emerging_optimizers_b200.orthogonalized_optimizers.muon_hyperball import *  # noqa: F401,F403
from emerging_optimizers_b200.orthogonalized_optimizers.orthogonalized_optimizer import *  # noqa: F401,F403
from emerging_optimizers_b200.orthogonalized_optimizers.polargrad import *  # noqa: F401,F403
from emerging_optimizers_b200.orthogonalized_optimizers.scion import *  # noqa: F401,F403
from emerging_optimizers_b200.orthogonalized_optimizers.spectral_clipping_utils import *  # noqa: F401,F403
from emerging_optimizers_b200.orthogonalized_optimizers.spel import *  # noqa: F401,F403
from emerging_optimizers_b200.orthogonalized_optimizers.split_qkv import *  # noqa: F401,F403
