"""Multi-GPU partitioning of the orthogonalization work inside one NVSwitch box."""

from emerging_optimizers_b200.distributed.layer_parallel import LayerParallelMuon, ns_cost, partition_by_cost


__all__ = ["LayerParallelMuon", "ns_cost", "partition_by_cost"]
