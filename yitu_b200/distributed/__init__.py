"""Row-partitioned multi-GPU SpMM: one process per GPU, destination rows split into contiguous edge-balanced
ranges, source features sharded the same way, halo rows pushed by their owners (or fetched by their readers) over
NVLink.

This reworks the role of YiTu_GNN/distributed (feature-dimension sharding with per-rank reduces,
communication.py:230-264, over DistDGL partitions) for graphs that fit the GPUs of one NVSwitch box."""
from .partition import (HaloPlan, PushSchedule, RowShard, allgather_columns, exchange_need_lists, owner_edge_counts,
                        partition_bounds, source_passes)
from .runtime import PartitionedAggregate, PartitionedSpmm, SharedBuffer

__all__ = ["HaloPlan", "PushSchedule", "RowShard", "allgather_columns", "exchange_need_lists", "owner_edge_counts",
           "partition_bounds", "source_passes", "PartitionedSpmm", "PartitionedAggregate", "SharedBuffer"]
