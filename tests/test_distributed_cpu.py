"""Row partition and halo bookkeeping on CPU ranks over gloo (world_size 2 and 3): bounds, shards, halo lists and
renumbered columns are bit-exact against the CPU checker, and the partitioned aggregation assembled from
[own rows | halo rows] (and from the all-gather layout) equals the single-graph result."""
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
        from yitu_b200.distributed import HaloPlan, RowShard, allgather_columns, partition_bounds, split_local_halo

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

        # halo list ordered by the first row block that needs a row
        rb = [0, shard.n_local // 3, (2 * shard.n_local) // 3, shard.n_local]
        plan_b = HaloPlan(shard, rb)
        assert sorted(plan_b.halo_ids.tolist()) == halo.tolist() and plan_b.chunk_offsets[-1] == plan_b.n_halo
        lib_ = plan_b.local_indices.numpy()
        hb = plan_b.halo_ids.numpy()
        assert np.array_equal(np.where(lib_ < shard.n_local, lib_ + lo, hb[np.maximum(lib_ - shard.n_local, 0)]), cols)
        ipn = shard.indptr.numpy()
        for b in range(3):
            used = lib_[ipn[rb[b]]:ipn[rb[b + 1]]]
            used = used[used >= shard.n_local] - shard.n_local
            assert used.size == 0 or used.max() < plan_b.chunk_offsets[b + 1], "block b may only use chunks 0..b"
            seg = hb[plan_b.chunk_offsets[b]:plan_b.chunk_offsets[b + 1]]
            assert np.all(np.diff(seg) > 0), "ascending ids inside a chunk"
        xbuf_b = torch.cat([x[lo:hi], x[torch.from_numpy(hb).long()]]).numpy()
        got_b = O.spmm(shard.indptr.numpy(), lib_, xbuf_b, wmode=O.W_EDGE, values=shard.values.numpy())
        assert np.array_equal(got_b, ref)

        (ipo, ixo, vo), (iph, ixh, vh) = split_local_halo(shard, plan)
        assert int(ipo[-1]) + int(iph[-1]) == shard.nnz
        assert ixo.numel() == 0 or int(ixo.max()) < shard.n_local
        assert ixh.numel() == 0 or int(ixh.max()) < plan.n_halo
        part = O.spmm(ipo.numpy(), ixo.numpy(), xbuf[:shard.n_local], wmode=O.W_EDGE, values=vo.numpy()).astype(np.float64)
        part += O.spmm(iph.numpy(), ixh.numpy(), xbuf[shard.n_local:], wmode=O.W_EDGE, values=vh.numpy())
        assert np.abs(part - ref).max() <= 1e-5 * np.abs(ref).max()
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errors.put("rank %d:\n%s" % (rank, traceback.format_exc()))
        raise


@pytest.mark.parametrize("world", [2, 3])
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
