"""B200-native (sm_100a) Newton-Schulz / Muon orthogonalization path.

Mirrors the module layout of the reference package for the hot path only:
``emerging_optimizers_b200.orthogonalized_optimizers`` (``muon_utils``, ``Muon``, ``OrthogonalizedOptimizer``),
``emerging_optimizers_b200.triton_kernels`` (the SYRK entry points, now backed by hand-written CUDA) and the small
helpers they need.  All dense math runs in ``libeo_b200.so``; there is no CPU or PyTorch fallback.
"""

__version__ = "0.1.0"
