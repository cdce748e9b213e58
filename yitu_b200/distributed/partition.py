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
    halo_ids is sorted, hence grouped by owner: rows [owner_offsets[p], owner_offsets[p+1]) of the halo part
    belong to rank p, in ascending id order — the layout both the reader-side gather and the owner-side push fill."""

    def __init__(self, shard):
        lo, hi = shard.row_begin, shard.row_end
        cols = shard.indices
        own = (cols >= lo) & (cols < hi)
        self.halo_ids = torch.unique(cols[~own])  # sorted ascending, int32
        self.n_halo = self.halo_ids.numel()
        pos = torch.searchsorted(self.halo_ids, cols)
        bounds_t = torch.tensor(shard.bounds, dtype=self.halo_ids.dtype, device=cols.device)
        self.owner_offsets = torch.searchsorted(self.halo_ids, bounds_t).tolist()
        self.local_indices = torch.where(own, cols - lo, pos.to(cols.dtype) + shard.n_local).to(torch.int32)


def allgather_columns(indices, bounds, max_rows):
    """Column ids for a replicated buffer made of P slots of max_rows rows (an all-gather of padded shards):
    global id s owned by rank p -> p*max_rows + (s - bounds[p])."""
    b = torch.tensor(bounds, dtype=indices.dtype, device=indices.device)
    owner = torch.searchsorted(b, indices, right=True) - 1
    return (owner * max_rows + (indices - b[owner])).to(torch.int32)


# ---------------------------------------------------------------------------------------------------------
# Owner-side push with source-group passes: who sends what to whom, in which order the shards become usable,
# and how a rank cuts its edges into aggregation passes that can start before the last byte has arrived.
# ---------------------------------------------------------------------------------------------------------
def owner_edge_counts(shard, world):
    """Edges of the shard per owner of their source row: a list of `world` ints."""
    b = torch.tensor(shard.bounds, dtype=shard.indices.dtype, device=shard.indices.device)
    owner = torch.searchsorted(b, shard.indices, right=True) - 1
    return torch.bincount(owner, minlength=world)[:world].tolist()


class PushSchedule:
    """When each owner's rows are with its readers, and how each rank cuts its aggregation into passes.

    Every owner pushes the rows its peers need from the first moment of a step, at the speed of its own NVLink
    egress, so owner p has delivered after about egress_rows[p] * row_bytes / bandwidth; readers learn of it through
    per-(reader, owner) flags, so each reader plans for itself.  A rank aggregates in PASSES: its owners sorted by
    delivery time are cut into at most `max_passes` consecutive groups; pass 0 also takes the edges whose sources the
    rank owns (usable at once); a pass starts when its last owner has delivered and accumulates into the output of
    the passes before it.  More passes start earlier but pay the per-row cost of a pass again.

    One rank may be served FIRST (`priority`): every owner sends that rank's rows before anything else, and the
    rank aggregates them in a single pass as soon as they are in (the edges whose sources it owns itself in a pass
    of their own while it waits, with `priority_own_first`).  This is for the rank whose aggregation is the longest
    (the shard with by far the most destination rows on a skewed graph): it cannot afford to wait for the slowest
    owner, and a second pass over its many rows costs more than it gains.

    Cuts and the priority rank are chosen by exhaustive search over a cost model of a pass (`pass_ms`: the cost
    of an edge grows from 0.05 ns on long rows to 0.17 ns where a row holds an edge or less) and of a push
    (690 GB/s out of one GPU), fitted to B200 measurements of the 128-feature workload; the model only has to rank
    the alternatives.

    need_rows[q][p]   rows that rank q needs from owner p          (every rank holds the same matrix)
    block_edges[q][p] edges of rank q whose source row owner p holds
    rows[q]           destination rows of rank q
    """

    PRIORITY = -2

    def __init__(self, need_rows, block_edges, rows, d, max_passes=3, egress_gbs=690.0, sync_ms=0.03,
                 priority="auto", priority_own_first="auto"):
        import itertools
        P = len(rows)
        self.world, self.d = P, int(d)
        scale = d / 128.0
        row_ms = 4.0 * d / (egress_gbs * 1e9) * 1e3  # one feature row over one link direction
        need = [[0 if p == q else int(need_rows[q][p]) for p in range(P)] for q in range(P)]
        self.egress_rows = [sum(need[q][p] for q in range(P)) for p in range(P)]
        total_edges = [sum(int(e) for e in block_edges[q]) for q in range(P)]

        def pass_ms(edges, n_rows, first):
            """Aggregation pass over `edges` edges spread over n_rows destination rows, fitted to the edge-stream and
            warp-per-row kernels on B200 at 128 features: 0.05 ns per edge of a long row, up to 0.17 ns where rows hold
            an edge or less (short rows are cold gathers), plus writing (first pass) or visiting the rows."""
            if edges <= 0:
                return 0.0
            per_edge = 0.05 + 0.12 * (n_rows / float(edges)) ** 0.7
            return (edges * per_edge * scale + n_rows * (0.09 * scale if first else 0.047)) * 1e-6

        def plan_reader(q, push_ms):
            """Best cuts for reader q: (finish time, [(owners, time the pass may start)])."""
            owners = sorted((p for p in range(P) if p != q and block_edges[q][p] > 0), key=lambda p: (push_ms[p], p))
            idle = [p for p in range(P) if p != q and block_edges[q][p] <= 0]  # nothing to gather from them
            best_q = None
            n = len(owners)
            for k in range(1, min(max_passes, max(n, 1)) + 1):
                for cut in itertools.combinations(range(1, n), k - 1) if n else [()]:
                    groups = [owners[a:b] for a, b in zip((0,) + cut, cut + (n,))] if n else [[]]
                    # own sources: a pass of their own when that is worth it, else part of the first group
                    for own_alone in ((False, True) if n and block_edges[q][q] > 0 and k < max_passes else (False,)):
                        t, plan = 0.0, []
                        if own_alone:
                            t = pass_ms(int(block_edges[q][q]), rows[q], True)
                            plan.append(([q], 0.0))
                        for gi, grp in enumerate(groups):
                            edges = sum(int(block_edges[q][p]) for p in grp)
                            members = list(grp)
                            if gi == 0 and not own_alone:
                                edges += int(block_edges[q][q])
                                members = [q] + members
                            start = max([push_ms[p] + sync_ms for p in grp] + [0.0])
                            t = max(t, start) + pass_ms(edges, rows[q], not plan)
                            plan.append((members, start))
                        if best_q is None or t < best_q[0] - 1e-9:
                            best_q = (t, plan)
            t, plan = best_q
            plan[0] = (plan[0][0] + idle, plan[0][1])
            return t, plan

        if priority == "auto":
            heavy = max(range(P), key=lambda q: pass_ms(total_edges[q], rows[q], True))
            prio_options = [None, heavy] if P > 2 else [None]
        else:
            prio_options = [priority]
        best = None
        for prio in prio_options:
            if prio is None:
                first_ms, prio_ready = [0.0] * P, 0.0
            else:
                first_ms = [need[prio][p] * row_ms for p in range(P)]
                prio_ready = max(max(first_ms), sum(need[prio]) * row_ms) + sync_ms  # slowest sender or its own ingress
            push_ms = [first_ms[p] + (self.egress_rows[p] - (need[prio][p] if prio is not None else 0)) * row_ms
                       for p in range(P)]
            worst, plans = 0.0, []
            for q in range(P):
                if q == prio:
                    # one pass as soon as its rows are in - or the edges whose sources it owns while it waits, then
                    # everything else in one pass; whichever the model ends earlier
                    t, plan = prio_ready + pass_ms(total_edges[q], rows[q], True), [(list(range(P)), prio_ready)]
                    own = int(block_edges[q][q])
                    if priority_own_first and 0 < own < total_edges[q]:
                        t2 = max(prio_ready, pass_ms(own, rows[q], True)) + pass_ms(total_edges[q] - own, rows[q], False)
                        if priority_own_first is True or t2 < t:
                            t, plan = t2, [([q], 0.0), ([p for p in range(P) if p != q], prio_ready)]
                else:
                    t, plan = plan_reader(q, push_ms)
                plans.append(plan)
                worst = max(worst, t)
            if best is None or worst < best[0] - 1e-6:  # ties: no priority rank
                best = (worst, plans, prio, push_ms)
        self.model_ms, plans, self.priority, self.push_ms = best
        # passes[q]: list of (owners whose edges the pass takes, PRIORITY for the priority rank's passes, else
        # the pass number)
        self.passes = [[(owners, self.PRIORITY if q == self.priority else j) for j, (owners, _) in enumerate(plan)]
                       for q, plan in enumerate(plans)]
        self._starts = [[round(t, 3) for _, t in plan] for plan in plans]

    def describe(self):
        return {"priority_rank": self.priority,
                "push_ms_model": [round(t, 3) for t in self.push_ms],
                "passes_per_rank": [[{"owners": o, "may_start_ms_model": t} for (o, _), t in zip(ps, ts)]
                                    for ps, ts in zip(self.passes, self._starts)],
                "step_ms_model": round(self.model_ms, 3)}


def source_passes(shard, plan, passes):
    """Cut a shard's edges into the aggregation passes of a PushSchedule.  `passes` is this rank's list of
    (owners, tag).  Returns [(indptr, local_indices, values, tag)] with every row present in every
    pass (empty where the pass holds none of its edges); the column ids index the buffer [own rows | halo rows]."""
    cols = shard.indices
    b = torch.tensor(shard.bounds, dtype=cols.dtype, device=cols.device)
    owner = torch.searchsorted(b, cols, right=True) - 1
    pass_of_owner = torch.full((len(shard.bounds) - 1,), -1, dtype=torch.int64, device=cols.device)
    for j, (owners, _) in enumerate(passes):
        pass_of_owner[torch.tensor(owners, dtype=torch.int64, device=cols.device)] = j
    pass_of_edge = pass_of_owner[owner]
    del owner
    ip = shard.indptr.long()
    out = []
    for j, (_, wait) in enumerate(passes):
        if len(passes) == 1:
            out.append((shard.indptr, plan.local_indices, shard.values, wait))
            break
        m = pass_of_edge == j
        csum = torch.zeros(m.numel() + 1, dtype=torch.int64, device=m.device)
        torch.cumsum(m, 0, out=csum[1:])
        out.append((csum[ip].to(shard.indptr.dtype), plan.local_indices[m].contiguous(),
                    None if shard.values is None else shard.values[m].contiguous(), wait))
    return out


def exchange_need_lists(plan, rank, world, group=None):
    """Tell every owner which of its rows this rank needs.  Returns (need_rows, recv_ids, recv_counts):
    need_rows[q][p] = rows rank q needs from owner p (the same matrix on every rank), recv_ids = the global ids
    the peers need from THIS rank, concatenated by requesting rank, recv_counts[q] = how many of them rank q asked for."""
    import torch.distributed as dist
    off = plan.owner_offsets
    send_counts = [off[p + 1] - off[p] for p in range(world)]
    dev = plan.halo_ids.device
    mine = torch.tensor(send_counts, dtype=torch.int64, device=dev)
    rows = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(rows, mine, group=group)
    need_rows = [r.tolist() for r in rows]
    recv_counts = [need_rows[q][rank] for q in range(world)]
    recv = torch.empty(sum(recv_counts), dtype=plan.halo_ids.dtype, device=dev)
    dist.all_to_all_single(recv, plan.halo_ids.contiguous(), output_split_sizes=recv_counts,
                           input_split_sizes=send_counts, group=group)
    return need_rows, recv, recv_counts
