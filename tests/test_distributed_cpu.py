"""Row partition and halo bookkeeping on CPU ranks over gloo (world_size 2, 3 and 4): bounds, shards, halo lists and
renumbered columns are bit-exact against the CPU checker, the partitioned aggregation assembled from
[own rows | halo rows] (and from the all-gather layout) equals the single-graph result, and the owner-side push
(request lists, slot layout, schedule, aggregation passes) is consistent across ranks."""
import os
import socket
import sys
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, errors):
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from oracle import oracle as O
        from yitu_b200 import graphs
        from yitu_b200.distributed import (HaloPlan, PushSchedule, RowShard, allgather_columns, exchange_need_lists,
                                           owner_edge_counts, partition_bounds, source_passes)

        n, d = 3000, 12
        src, dst = graphs.rmat_edges(4, n, n, 40000)
        indptr, indices = graphs.csr_by_destination(src, dst, n, n, ptr_dtype=torch.int64)
        deg = (indptr[1:] - indptr[:-1]).clamp(min=1)
        values = torch.repeat_interleave(1.0 / deg.float(), indptr[1:] - indptr[:-1])
        x = graphs.randn_features(7, n, d)

        bounds = partition_bounds(indptr, world)
        assert bounds == O.partition_rows(indptr.numpy(), world).tolist()
        gathered = [None] * world
        dist.all_gather_object(gathered, bounds)
        assert all(b == bounds for b in gathered), "every rank must derive the same partition"

        shard = RowShard(indptr, indices, values, bounds, rank)
        lo, hi = bounds[rank], bounds[rank + 1]
        assert shard.indptr[0] == 0 and shard.indptr.dtype == torch.int64
        assert torch.equal(shard.indptr, indptr[lo:hi + 1] - indptr[lo])
        nnz_parts = [None] * world
        dist.all_gather_object(nnz_parts, shard.nnz)
        assert sum(nnz_parts) == indices.numel()
        assert max(nnz_parts) - min(nnz_parts) <= int(deg.max()), "edge-balanced up to one row"

        plan = HaloPlan(shard)
        halo = plan.halo_ids.numpy()
        cols = shard.indices.numpy()
        expect_halo = np.unique(cols[(cols < lo) | (cols >= hi)])
        assert np.array_equal(halo, expect_halo)
        li = plan.local_indices.numpy()
        rebuilt = np.where(li < shard.n_local, li + lo, halo[np.maximum(li - shard.n_local, 0)])
        assert np.array_equal(rebuilt, cols), "renumbered columns must map back to the global ids"
        for p in range(world):
            seg = halo[plan.owner_offsets[p]:plan.owner_offsets[p + 1]]
            assert np.all((seg >= bounds[p]) & (seg < bounds[p + 1]))
        assert plan.owner_offsets[rank] == plan.owner_offsets[rank + 1], "no halo rows from oneself"

        # halo exchange emulated with a gloo all-gather of padded shards, then the aggregation by the CPU checker
        max_rows = max(bounds[p + 1] - bounds[p] for p in range(world))
        mine = torch.zeros(max_rows, d)
        mine[:shard.n_local] = x[lo:hi]
        rep = torch.empty(world * max_rows, d)
        dist.all_gather_into_tensor(rep, mine)
        ag_cols = allgather_columns(shard.indices, bounds, max_rows)
        assert torch.equal(rep[ag_cols.long()], x[shard.indices.long()])
        b = np.asarray(bounds)
        owner = np.searchsorted(b, halo, side="right") - 1
        x_halo = rep[torch.from_numpy(owner * max_rows + (halo - b[owner])).long()]
        xbuf = torch.cat([x[lo:hi], x_halo]).numpy()
        ref = O.spmm(indptr.numpy(), indices.numpy(), x.numpy(), wmode=O.W_EDGE, values=values.numpy())[lo:hi]
        got = O.spmm(shard.indptr.numpy(), li, xbuf, wmode=O.W_EDGE, values=shard.values.numpy())
        assert np.array_equal(got, ref), "partitioned aggregation must equal the single-graph rows"

        # owner-side push: the request lists that reach every owner, the slot layout, the schedule and the passes
        need_rows, recv_ids, recv_counts = exchange_need_lists(plan, rank, world)
        assert need_rows[rank] == [plan.owner_offsets[p + 1] - plan.owner_offsets[p] for p in range(world)]
        assert all(need_rows[q][q] == 0 for q in range(world))
        assert recv_ids.numel() == sum(recv_counts) and recv_counts[rank] == 0
        assert recv_ids.numel() == 0 or (int(recv_ids.min()) >= lo and int(recv_ids.max()) < hi), "only rows this rank owns"
        # the push itself, emulated by an all-to-all of the requested rows: what arrives, in arrival order
        # (by owner, ascending ids within an owner), must be exactly the halo part of the reader's buffer
        sent = x[recv_ids.long()].contiguous()
        got_rows = torch.empty(plan.n_halo, d)
        dist.all_to_all_single(got_rows, sent, output_split_sizes=need_rows[rank], input_split_sizes=recv_counts)
        assert torch.equal(got_rows, x[plan.halo_ids.long()]), "pushed rows must land in the slots the columns point to"
        mine = torch.tensor(owner_edge_counts(shard, world), dtype=torch.int64)
        assert int(mine.sum()) == shard.nnz
        blocks = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(blocks, mine)
        rows_per_rank = [bounds[p + 1] - bounds[p] for p in range(world)]
        for max_passes, prio in ((3, "auto"), (1, None), (2, world - 1), (4, None)):
            sched = PushSchedule(need_rows, [b_.tolist() for b_ in blocks], rows_per_rank, d, max_passes=max_passes,
                                 priority=prio)
            seen = [None] * world
            dist.all_gather_object(seen, sched.describe())
            assert all(s_ == seen[0] for s_ in seen), "every rank must derive the same schedule"
            my = sched.passes[rank]
            assert 1 <= len(my) <= max_passes
            assert sorted(p for owners, _ in my for p in owners) == list(range(world)), "each owner in exactly one pass"
            assert rank in my[0][0], "own sources belong to the first pass"
            if prio == world - 1 and rank == prio:
                # its own sources while it waits for its delivery, then every other owner in one pass
                forced = PushSchedule(need_rows, [b_.tolist() for b_ in blocks], rows_per_rank, d, max_passes=max_passes,
                                      priority=prio, priority_own_first=True)
                assert forced.passes[rank] == [([rank], PushSchedule.PRIORITY),
                                               ([p for p in range(world) if p != rank], PushSchedule.PRIORITY)]
                assert my in (forced.passes[rank], [(list(range(world)), PushSchedule.PRIORITY)])
                single = PushSchedule(need_rows, [b_.tolist() for b_ in blocks], rows_per_rank, d, max_passes=max_passes,
                                      priority=prio, priority_own_first=False)
                assert single.passes[rank] == [(list(range(world)), PushSchedule.PRIORITY)]
            elif sched.priority is None:
                # owners are taken in the order of their modelled delivery: a later pass never holds an earlier owner
                order = [max(sched.push_ms[p] for p in owners if p != rank) for owners, _ in my if set(owners) - {rank}]
                assert order == sorted(order)
            total = np.zeros_like(ref, dtype=np.float64)
            nnz_sum = 0
            for ip_j, li_j, v_j, _ in source_passes(shard, plan, my):
                assert ip_j.numel() == shard.n_local + 1 and int(ip_j[-1]) == li_j.numel() == v_j.numel()
                nnz_sum += li_j.numel()
                total += O.spmm(ip_j.numpy(), li_j.numpy(), xbuf, wmode=O.W_EDGE, values=v_j.numpy())
            assert nnz_sum == shard.nnz
            assert np.abs(total - ref).max() <= 1e-5 * np.abs(ref).max(), "the passes together give the whole aggregation"
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errors.put("rank %d:\n%s" % (rank, traceback.format_exc()))
        raise


@pytest.mark.parametrize("world", [2, 3, 4])
def test_partition_and_halo_plan_over_gloo(world):
    ctx = mp.get_context("spawn")
    errors = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, errors)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    msgs = []
    while not errors.empty():
        msgs.append(errors.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            msgs.append("a rank did not finish")
    assert not msgs and all(p.exitcode == 0 for p in procs), "\n".join(msgs)
