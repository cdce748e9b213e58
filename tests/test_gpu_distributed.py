"""Row-partitioned SpMM.  On 2 GPUs (one process per GPU, NCCL + CUDA-IPC peer mappings; skipped on a single-GPU
box): every exchange mode must give the rows the single-GPU SpMM gives.  On one GPU: the owner-side push and the
aggregation passes of its schedule with four ranks emulated in one process (every "peer" buffer lives on the same
GPU and the kernels run one after another on one stream - nothing waits on anything)."""
import os
import socket
import sys
import traceback

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
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
        import torch.distributed as dist
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from yitu_b200 import graphs, ops
        from yitu_b200.distributed import PartitionedSpmm, RowShard, partition_bounds
        n, d = 1 << 16, 128
        src, dst = graphs.rmat_edges(4, n, n, 1 << 20, device=dev)
        indptr, indices = graphs.csr_by_destination(src, dst, n, n, ptr_dtype=torch.int64)
        deg = (indptr[1:] - indptr[:-1]).clamp(min=1)
        values = torch.repeat_interleave(1.0 / deg.float(), indptr[1:] - indptr[:-1])
        x = graphs.randn_features(7, n, d, device=dev)
        ref = ops.spmm(ops.PreparedGraph(indptr, indices, n), x, mode=ops.W_EDGE, edge_values=values)
        bounds = partition_bounds(indptr, world)
        shard = RowShard(indptr, indices, values, bounds, rank)
        lo, hi = shard.row_begin, shard.row_end
        for mode, kw in (("push", {}), ("push", dict(max_passes=1, priority=None)), ("push", dict(priority=1)),
                         ("peer", {}), ("allgather", {})):
            r = PartitionedSpmm(shard, d, dev, mode=mode, **kw)
            for step in range(3):  # new features every step: a stale halo row would show
                xs = x * float(step + 1)
                r.x_local.copy_(xs[lo:hi])
                out = r.step(fence=True)
                torch.cuda.synchronize(dev)
                err = float((out - ref[lo:hi] * float(step + 1)).abs().max())
                assert err <= 1e-5 * float(ref.abs().max()) * (step + 1), "%s %s step %d: max err %g" % (mode, kw, step, err)
                if mode in ("peer", "push"):
                    assert r.plan.n_halo > 0
                    assert torch.equal(r.x_halo, xs[r.plan.halo_ids.long()]), "halo rows must be the owners' rows"
            if mode == "push":
                assert sum(g.nnz for g, _, _ in r._passes) == shard.nnz
                r.check()  # no wait for a delivery ran out
            r.close()
        # differentiable form: forward over this rank's rows of A, backward over the same rows of A^T
        from yitu_b200.distributed import PartitionedAggregate
        whole = ops.PreparedGraph(indptr, indices, n)
        w_out = graphs.randn_features(9, n, d, device=dev)
        ref_grad = ops.spmm(whole.t_prepared(), w_out, mode=ops.W_EDGE, edge_values=values, edge_perm=whole.transpose()[2])
        agg = PartitionedAggregate(indptr, indices, values, d, dev)
        assert (agg.row_begin, agg.row_end) == (lo, hi)
        xl = x[lo:hi].clone().requires_grad_()
        for _ in range(2):  # twice: the shared shards are overwritten between steps
            xl.grad = None
            y = agg(xl)
            (y * w_out[lo:hi]).sum().backward()
        torch.cuda.synchronize(dev)
        assert float((y - ref[lo:hi]).abs().max()) <= 1e-5 * float(ref.abs().max())
        assert float((xl.grad - ref_grad[lo:hi]).abs().max()) <= 1e-5 * float(ref_grad.abs().max())
        dist.barrier()
        agg.close()
        dist.destroy_process_group()
    except Exception:
        errors.put("rank %d:\n%s" % (rank, traceback.format_exc()))
        raise


def test_partitioned_spmm_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    errors = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, errors)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    msgs = []
    while not errors.empty():
        msgs.append(errors.get())
    for p in procs:
        if p.is_alive():
            p.terminate()
            msgs.append("a rank did not finish")
    assert not msgs and all(p.exitcode == 0 for p in procs), "\n".join(msgs)


def test_push_exchange_and_passes_with_four_ranks_emulated_on_one_gpu():
    """yitu_halo_push_f32 and the aggregation passes of a PushSchedule without a second GPU: four ranks' buffers live
    on this GPU, every owner's push runs as an ordinary kernel on the current stream (its "peer" pointers are local),
    then every rank aggregates pass by pass.  Checks the slot layout bit for bit and the result against the
    whole-graph SpMM."""
    import ctypes as C
    sys.path.insert(0, ROOT)
    from yitu_b200 import graphs, ops
    from yitu_b200._lib import check, lib
    from yitu_b200.distributed import HaloPlan, PushSchedule, RowShard, owner_edge_counts, partition_bounds, source_passes
    dev = torch.device("cuda", 0)
    world, n, d = 4, 1 << 15, 128
    src, dst = graphs.rmat_edges(4, n, n, 1 << 19, device=dev)
    indptr, indices = graphs.csr_by_destination(src, dst, n, n, ptr_dtype=torch.int64)
    deg = (indptr[1:] - indptr[:-1]).clamp(min=1)
    values = torch.repeat_interleave(1.0 / deg.float(), indptr[1:] - indptr[:-1])
    x = graphs.randn_features(7, n, d, device=dev)
    ref = ops.spmm(ops.PreparedGraph(indptr, indices, n), x, mode=ops.W_EDGE, edge_values=values)
    bounds = partition_bounds(indptr, world)
    shards = [RowShard(indptr, indices, values, bounds, r) for r in range(world)]
    plans = [HaloPlan(s) for s in shards]
    bufs = [torch.full((s.n_local + p.n_halo, d), float("nan"), device=dev) for s, p in zip(shards, plans)]
    for r, s in enumerate(shards):
        bufs[r][:s.n_local] = x[s.row_begin:s.row_end]
    need = [[plans[q].owner_offsets[p + 1] - plans[q].owner_offsets[p] for p in range(world)] for q in range(world)]
    st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    counter = torch.zeros(1, dtype=torch.int64, device=dev)
    for p in range(world):  # owner p pushes to every reader q
        dests = [q for q in range(world) if q != p and need[q][p] > 0]
        ids = torch.cat([plans[q].halo_ids[plans[q].owner_offsets[p]:plans[q].owner_offsets[p + 1]] for q in dests])
        ids = (ids - shards[p].row_begin).to(torch.int32).contiguous()
        begin = [0]
        for q in dests:
            begin.append(begin[-1] + need[q][p])
        dst_ptrs = [bufs[q].data_ptr() + 4 * d * (shards[q].n_local + plans[q].owner_offsets[p]) for q in dests]
        check(lib().yitu_halo_push_f32(len(dests), (C.c_void_p * len(dests))(*dst_ptrs),
                                       (C.c_int64 * (len(dests) + 1))(*begin), C.c_void_p(ids.data_ptr()),
                                       C.c_void_p(bufs[p].data_ptr()), d, C.c_void_p(counter.data_ptr()), 0 if p % 2 else 3, st))
    torch.cuda.synchronize(dev)
    for q in range(world):
        assert torch.equal(bufs[q][shards[q].n_local:], x[plans[q].halo_ids.long()]), "rank %d: halo slots" % q
    blocks = [owner_edge_counts(s, world) for s in shards]
    rows = [s.n_local for s in shards]
    for kw in (dict(), dict(max_passes=1, priority=None), dict(max_passes=4, priority=world - 1)):
        sched = PushSchedule(need, blocks, rows, d, **kw)
        for q, s in enumerate(shards):
            out = torch.full((s.n_local, d), float("nan"), device=dev)
            passes = source_passes(s, plans[q], sched.passes[q])
            assert sum(li.numel() for _, li, _, _ in passes) == s.nnz
            for j, (ip, li, vals, _) in enumerate(passes):
                g = ops.PreparedGraph(ip, li, s.n_local + plans[q].n_halo)
                ops.spmm(g, bufs[q], mode=ops.W_EDGE, edge_values=vals, out=out, accumulate=j > 0)
            err = float((out - ref[s.row_begin:s.row_end]).abs().max())
            assert err <= 1e-5 * float(ref.abs().max()), "rank %d %s: max err %g" % (q, kw, err)


def test_delivery_flags_signal_then_wait_and_bounded_timeout():
    """The flag kernels on one GPU, one stream, in an order in which nothing waits for a later launch: a signal
    followed by a wait for the value just stored returns at once; a wait for a value that nothing stores gives up
    after its time limit, records which flag was missing, and leaves the stream and the context usable."""
    import ctypes as C
    import time
    sys.path.insert(0, ROOT)
    from yitu_b200._lib import check, lib
    dev = torch.device("cuda", 0)
    flags = torch.zeros(32, dtype=torch.int64, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    st = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    targets = (C.c_void_p * 3)(*[flags.data_ptr() + 8 * i for i in (0, 2, 5)])
    check(lib().yitu_flags_signal(3, targets, 7, st))
    check(lib().yitu_flags_wait(C.c_void_p(flags.data_ptr()), 0b100101, 7, 1_000_000_000, C.c_void_p(err.data_ptr()), st))
    check(lib().yitu_flags_wait(C.c_void_p(flags.data_ptr()), 0b000101, 3, 1_000_000_000, C.c_void_p(err.data_ptr()), st))
    torch.cuda.synchronize(dev)
    assert flags.tolist()[:6] == [7, 0, 7, 0, 0, 7] and int(err) == 0
    t0 = time.perf_counter()
    check(lib().yitu_flags_wait(C.c_void_p(flags.data_ptr()), 0b1000, 7, 5_000_000, C.c_void_p(err.data_ptr()), st))  # 5 ms
    torch.cuda.synchronize(dev)
    assert time.perf_counter() - t0 < 1.0, "the wait must give up after its limit"
    assert int(err) == 1 + 3, "flag 3 was the missing one"
    assert float(torch.ones(4, device=dev).sum()) == 4.0  # the context is alive
    with pytest.raises(RuntimeError):  # an unbounded wait is refused
        check(lib().yitu_flags_wait(C.c_void_p(flags.data_ptr()), 1, 8, 0, C.c_void_p(err.data_ptr()), st))


def test_partitioned_aggregate_single_gpu_autograd():
    """World size 1: the differentiable partitioned aggregation degenerates to the local SpMM and its transpose."""
    sys.path.insert(0, ROOT)
    from yitu_b200 import graphs, ops
    from yitu_b200.distributed import PartitionedAggregate
    dev = torch.device("cuda", 0)
    n, d = 1 << 14, 64
    src, dst = graphs.rmat_edges(5, n, n, 1 << 18, device=dev)
    indptr, indices = graphs.csr_by_destination(src, dst, n, n)
    values = torch.rand(indices.numel(), device=dev)
    whole = ops.PreparedGraph(indptr, indices, n)
    x = graphs.randn_features(1, n, d, device=dev).requires_grad_()
    w_out = graphs.randn_features(2, n, d, device=dev)
    for vals in (values, None):
        mode = ops.W_EDGE if vals is not None else ops.W_NONE
        agg = PartitionedAggregate(indptr, indices, vals, d, dev)
        x.grad = None
        y = agg(x)
        (y * w_out).sum().backward()
        ref = ops.spmm(whole, x.detach(), mode=mode, edge_values=vals)
        ref_grad = ops.spmm(whole.t_prepared(), w_out, mode=mode, edge_values=vals,
                            edge_perm=whole.transpose()[2] if vals is not None else None)
        assert float((y.detach() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
        assert float((x.grad - ref_grad).abs().max()) <= 1e-5 * float(ref_grad.abs().max())
        agg.close()
