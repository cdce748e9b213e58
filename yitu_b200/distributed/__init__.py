"""Row-partitioned multi-GPU SpMM: one process per GPU, destination rows split into contiguous edge-balanced
ranges, source features sharded the same way, halo rows fetched over NVLink.

This reworks the role of YiTu_GNN/distributed (feature-dimension sharding with per-rank reduces,
communication.py:230-264, over DistDGL partitions) for graphs that fit the GPUs of one NVSwitch box."""
from .partition import HaloPlan, RowShard, allgather_columns, partition_bounds, split_local_halo
from .runtime import PartitionedAggregate, PartitionedSpmm, SharedBuffer

__all__ = ["HaloPlan", "RowShard", "allgather_columns", "partition_bounds", "split_local_halo", "PartitionedSpmm",
           "PartitionedAggregate", "SharedBuffer"]
