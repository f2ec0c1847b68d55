"""The one piece of the SOAP / Shampoo family that is a symmetric rank-k product: the Kronecker factor update."""

from emerging_optimizers_b200.legacy_soap.soap import update_kronecker_factors


__all__ = ["update_kronecker_factors"]
