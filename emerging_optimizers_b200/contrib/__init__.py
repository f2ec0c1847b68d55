"""Optimizers outside the core package that reuse its Newton-Schulz path."""

from emerging_optimizers_b200.contrib.muown import Muown


__all__ = ["Muown"]
