"""Row-partitioned SpMM on 2 GPUs (one process per GPU, NCCL + CUDA-IPC peer loads): every halo mode must give
the rows the single-GPU SpMM gives.  Skipped on a single-GPU box."""
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
        for mode, overlap, blocks in (("peer", False, 1), ("peer", True, 1), ("peer", False, 4), ("allgather", False, 1)):
            r = PartitionedSpmm(shard, d, dev, mode=mode, overlap=overlap, row_blocks=blocks)
            r.x_local.copy_(x[lo:hi])
            for _ in range(2):
                out = r.step()
            torch.cuda.synchronize(dev)
            err = float((out - ref[lo:hi]).abs().max())
            assert err <= 1e-5 * float(ref.abs().max()), "%s overlap=%s blocks=%d: max err %g" % (mode, overlap, blocks, err)
            if mode == "peer":
                assert r.plan.n_halo > 0
                assert torch.equal(r.x_halo, x[r.plan.halo_ids.long()]), "halo rows must be the owners' rows"
            dist.barrier()
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
