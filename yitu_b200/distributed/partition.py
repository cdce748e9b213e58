"""Partition bookkeeping (integer work, device-agnostic torch): row ranges, per-rank shards, halo lists and
column renumbering.  Runs on CUDA tensors in production and on CPU tensors in the gloo tests."""
import torch

from .. import ops


def partition_bounds(indptr, n_parts, row_cost=0):
    """Edge-balanced contiguous row ranges: bounds[p] = min{ r : indptr[r] >= ceil(p*nnz/P) } as a Python list.

    The reference's own range partition balances node counts (YiTu_GNN/mmap/partition.py:12-22); balancing
    edges balances the gather work instead.  row_cost > 0 balances edges + row_cost * rows (a destination row costs
    about as much as row_cost edges: its output write and per-row latency), which evens out both the aggregation
    time and the size of the feature shards on skewed graphs."""
    if row_cost:
        indptr = indptr.long() + int(row_cost) * torch.arange(indptr.numel(), dtype=torch.int64, device=indptr.device)
    if indptr.is_cuda:
        g = ops.PreparedGraph(indptr, torch.empty(0, dtype=torch.int32, device=indptr.device), 0)
        return ops.partition_rows(g, n_parts).tolist()
    return ops.partition_rows_host(indptr, n_parts).tolist()


class RowShard:
    """Rows [bounds[rank], bounds[rank+1]) of a CSR: row pointers rebased to 0 (the convention of
    YiTu_GNN/mmap/partition.py:197), column ids still global."""

    def __init__(self, indptr, indices, values, bounds, rank):
        self.rank, self.bounds = rank, list(bounds)
        self.row_begin, self.row_end = bounds[rank], bounds[rank + 1]
        e0, e1 = int(indptr[self.row_begin]), int(indptr[self.row_end])
        self.edge_begin, self.edge_end = e0, e1
        self.indptr = (indptr[self.row_begin:self.row_end + 1] - e0).contiguous()
        self.indices = indices[e0:e1].contiguous()
        self.values = None if values is None else values[e0:e1].contiguous()
        self.n_local = self.row_end - self.row_begin
        self.nnz = e1 - e0


class HaloPlan:
    """Which remote source rows a shard needs, and its column ids renumbered for the buffer
    [own rows | halo rows]: own source id s -> s - row_begin, remote id -> n_local + position in halo_ids.

    With row_bounds (K+1 row offsets inside the shard) the halo list is ordered by the first row block that uses a
    row, ascending ids within a block: halo_ids[chunk_offsets[b]:chunk_offsets[b+1]] are the rows block b needs in
    addition to those of the blocks before it, so block b can be aggregated as soon as chunks 0..b have arrived."""

    def __init__(self, shard, row_bounds=None):
        lo, hi = shard.row_begin, shard.row_end
        cols = shard.indices
        own = (cols >= lo) & (cols < hi)
        halo_sorted = torch.unique(cols[~own])  # sorted ascending, int32
        self.n_halo = halo_sorted.numel()
        pos = torch.searchsorted(halo_sorted, cols)
        bounds_t = torch.tensor(shard.bounds, dtype=halo_sorted.dtype, device=cols.device)
        # halo rows [owner_offsets[p], owner_offsets[p+1]) of the id-sorted list live on rank p
        self.owner_offsets = torch.searchsorted(halo_sorted, bounds_t).tolist()
        self.chunk_offsets = [0, self.n_halo]
        self.row_bounds = None
        if row_bounds is not None and len(row_bounds) > 2 and self.n_halo > 0:
            k = len(row_bounds) - 1
            edge_bounds = shard.indptr.long()[torch.tensor(row_bounds, device=cols.device)]
            edge_ids = torch.arange(cols.numel(), device=cols.device)
            block_of_edge = torch.searchsorted(edge_bounds, edge_ids, right=True) - 1
            del edge_ids
            first = torch.full((self.n_halo,), k, dtype=torch.int64, device=cols.device)
            first.scatter_reduce_(0, pos[~own], block_of_edge[~own], reduce="amin")
            del block_of_edge
            first_sorted, perm = torch.sort(first, stable=True)  # new position j holds old position perm[j]
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(self.n_halo, device=cols.device)
            self.halo_ids = halo_sorted[perm].contiguous()
            pos = inv[pos.clamp(max=self.n_halo - 1)]
            counts = torch.bincount(first_sorted, minlength=k + 1)[:k]
            self.chunk_offsets = [0] + torch.cumsum(counts, 0).tolist()
            self.row_bounds = list(row_bounds)
        else:
            self.halo_ids = halo_sorted
        self.local_indices = torch.where(own, cols - lo, pos.to(cols.dtype) + shard.n_local).to(torch.int32)
        self.own_mask = own


def split_local_halo(shard, plan):
    """Split a shard's CSR by source into (own-source part, halo-source part) so the first can run while the
    halo is still in flight.  Returns two (indptr, indices, values) triples; the halo part's column ids index
    the halo buffer alone (0 .. n_halo)."""
    own = plan.own_mask
    csum = torch.zeros(own.numel() + 1, dtype=torch.int64, device=own.device)
    torch.cumsum(own, 0, out=csum[1:])
    ip = shard.indptr.long()
    ip_own = csum[ip]
    ip_halo = ip - ip_own
    dt = shard.indptr.dtype
    li = plan.local_indices
    vals = shard.values
    part_own = (ip_own.to(dt), li[own].contiguous(), None if vals is None else vals[own].contiguous())
    part_halo = (ip_halo.to(dt), (li[~own] - shard.n_local).contiguous(),
                 None if vals is None else vals[~own].contiguous())
    return part_own, part_halo


def allgather_columns(indices, bounds, max_rows):
    """Column ids for a replicated buffer made of P slots of max_rows rows (an all-gather of padded shards):
    global id s owned by rank p -> p*max_rows + (s - bounds[p])."""
    b = torch.tensor(bounds, dtype=indices.dtype, device=indices.device)
    owner = torch.searchsorted(b, indices, right=True) - 1
    return (owner * max_rows + (indices - b[owner])).to(torch.int32)
