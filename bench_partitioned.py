"""bench.py's leg for the row-partitioned SpMM (R-MAT N=2^24, 2^29 sampled edges, int64 row pointers, fp32
weights 1/in-degree, 128 features), one process per GPU.  Strong scaling: the graph is fixed, each rank
aggregates its edge-balanced row range.  Every rank builds the same graph from the same seed on its own GPU
(integer generator, bit-identical everywhere) and keeps its shard."""
import json
import os
import time

import torch
import torch.distributed as dist

METRIC = "aggregation_gedge_feat_per_s"
UNIT = "Gedge*feat/s"
NVLINK_PEER_GBS = 770.0  # measured peer-copy bandwidth per direction on this pool


def _reference_leg(args, device, n, e, d):
    """CPU restatement on all host cores, on the rows of partition 0 of 16 (bounded sample)."""
    from oracle import oracle as O
    from yitu_b200 import graphs
    from yitu_b200.distributed.partition import RowShard, partition_bounds
    indptr, indices, values = graphs.spmm_partitioned(device=device, n=n, e=e)
    bounds = partition_bounds(indptr, 16)
    sh = RowShard(indptr, indices, values, bounds, 8)
    x = graphs.randn_features(1, n, d, device=device).cpu().numpy()
    ip, ix, vals = sh.indptr.cpu().numpy(), sh.indices.cpu().numpy(), sh.values.cpu().numpy()
    O.build()
    cores = O.set_threads(len(os.sched_getaffinity(0)))  # torchrun exports OMP_NUM_THREADS=1
    best = None
    for _ in range(max(1, args.steps + args.warmup)):
        t0 = time.perf_counter()
        O.spmm(ip, ix, x, wmode=O.W_EDGE, values=vals)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    value = sh.nnz * d / best / 1e9
    base = {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "seconds": round(best, 3),
            "sample": "partition 8 of 16 (%d rows, %d of %d edges), forward SpMM, full feature matrix; best of %d" % (
                sh.n_local, sh.nnz, indices.numel(), max(1, args.steps + args.warmup))}
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": best * 1e3, "higher_is_better": True,
                      "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "partitioned_spmm_rmat_n%d_e%d_d%d" % (n, e, d),
                                 "note": "CPU restatement of the reference kernels; the reference has no CPU "
                                         "implementation of this path"},
                      "cpu_baseline": base,
                      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))


def _time_steps(runner, steps, world, events=None):
    """Device time of `steps` steps bracketed by barrier + synchronize, max over ranks (ms per step)."""
    dev = runner.device
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        runner.step(events)
    b.record()
    torch.cuda.synchronize(dev)
    ms = torch.tensor([a.elapsed_time(b) / steps], device=dev)
    if world > 1:
        dist.barrier()
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms)


def run(args):
    import bench  # the repo-root script: clock sampler and peak numbers
    from yitu_b200 import graphs, ops
    from yitu_b200.distributed.partition import RowShard, partition_bounds
    from yitu_b200.distributed.runtime import PartitionedSpmm

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n, e, d = (1 << 24) >> args.scale, (1 << 29) >> args.scale, 128
    if args.impl == "reference" and rank != 0:
        return  # the CPU arm runs on rank 0 alone
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    if args.impl == "reference":
        if rank == 0:
            _reference_leg(args, dev, n, e, d)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    indptr, indices, values = graphs.spmm_partitioned(device=dev, n=n, e=e)
    nnz = indices.numel()
    bounds = partition_bounds(indptr, world, row_cost=args.row_cost)
    shard = RowShard(indptr, indices, values, bounds, rank)
    if rank != 0:
        del indptr, indices, values
    torch.cuda.empty_cache()
    x_shard = graphs.randn_features(1, shard.n_local, d, device=dev, row_begin=shard.row_begin)

    candidates = [("local", False, 1)] if world == 1 else [("peer", False, 1), ("peer", True, 1), ("allgather", False, 1)]
    runners, trial = {}, {}
    for mode, overlap, blocks in candidates:
        r = PartitionedSpmm(shard, d, dev, mode=mode, overlap=overlap, row_blocks=blocks)
        r.x_local.copy_(x_shard)
        key = mode + ("+overlap" if overlap else "") + ("+rowblocks%d" % blocks if blocks > 1 else "")
        runners[key] = r
        for _ in range(3):
            r.step()
        trial[key] = _time_steps(r, 3, world)
    best = min(trial, key=trial.get)
    runner = runners[best]
    for k, r in runners.items():
        if k != best:
            r.close()
    warm = max(3, args.warmup)
    for _ in range(warm):
        runner.step()
    sampler = bench.ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    events = []
    ms_step = _time_steps(runner, args.steps, world, events)
    clocks = sampler.stop() if rank == 0 else None
    value = nnz * d / (ms_step * 1e-3) / 1e9

    spmm_ms = [a.elapsed_time(b) for tag, a, b in events if tag == "spmm"]
    fetch_ms = [a.elapsed_time(b) for tag, a, b in events if tag == "fetch"]
    # this library's kernels per step on this rank: one gather per fetch, one SpMM (+ one hub reduction when the
    # graph it ran on has split rows) per aggregation
    n_fetch = len(fetch_ms) / args.steps
    n_spmm = len(spmm_ms) / args.steps
    has_hub = 1 if runner.graph.plan() is not None else 0  # (row-block runs: counted from the whole-shard graph)
    launches_per_step = n_fetch + n_spmm * (1 + has_hub)
    k_ms = sum(spmm_ms) / args.steps  # SpMM time per step on this rank (one or two launches)
    k_bytes = shard.nnz * (4 * d + 8) + (shard.n_local + 1) * 8 + 4 * shard.n_local * d
    by_owner = [0.0] * world  # bytes this rank pulls from each owner per step
    if getattr(runner, "plan", None) is not None and world > 1:
        off = runner.plan.owner_offsets
        by_owner = [float((off[p + 1] - off[p]) * d * 4) for p in range(world)]
    stats = torch.tensor([k_ms, sum(fetch_ms) / args.steps if fetch_ms else 0.0, float(runner.halo_bytes),
                          float(shard.nnz), float(shard.n_local)] + by_owner, device=dev, dtype=torch.float64)
    all_stats = [torch.zeros_like(stats) for _ in range(world)]
    if world > 1:
        dist.all_gather(all_stats, stats)
    else:
        all_stats = [stats]

    # end to end: pinned host shard in, result shard back to pinned host memory, every step
    h_x = x_shard.cpu().pin_memory()
    h_out = torch.empty(shard.n_local, d).pin_memory()

    class E2E:
        device = dev

        def step(self, events=None):
            runner.x_local.copy_(h_x, non_blocking=True)
            h_out.copy_(runner.step(), non_blocking=True)

    e2e_runner = E2E()
    for _ in range(2):
        e2e_runner.step()
    e2e_ms = _time_steps(e2e_runner, max(2, min(args.steps, 5)), world)
    bytes_io = torch.tensor([h_x.numel() * 4.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(bytes_io)

    # the same aggregation on one GPU, for the speed-up (rank 0 only, outside the timed region)
    single = None
    if world > 1 and rank == 0 and not args.no_single:
        sh1 = RowShard(indptr, indices, values, [0, n], 0)
        r1 = PartitionedSpmm(sh1, d, dev, mode="local")
        r1.x_local.copy_(graphs.randn_features(1, n, d, device=dev))
        for _ in range(3):
            r1.step()
        single = nnz * d / (_time_steps(r1, max(3, args.steps // 2), 1) * 1e-3) / 1e9
    if world > 1:
        dist.barrier()

    if rank == 0:
        peak, peak_kind = bench.load_peaks()
        per_rank = [[float(v) for v in s.tolist()] for s in all_stats]
        achieved = k_bytes / (k_ms * 1e-3) / 1e9
        max_halo = max(s[2] for s in per_rank)
        max_fetch = max(s[1] for s in per_rank)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": "partitioned_spmm_rmat_n%d_e%d_d%d" % (n, e, d), "nnz": nnz,
                           "parallelism": "row_partition_%d" % world,
                           "balance": "edges" if not args.row_cost else "edges + %d * rows" % args.row_cost,
                           "halo": best, "trial_ms": trial,
                           "l2": "inputs_larger_than_l2", "rows_per_rank": [int(s[4]) for s in per_rank],
                           "edges_per_rank": [int(s[3]) for s in per_rank],
                           "halo_bytes_per_rank": [int(s[2]) for s in per_rank],
                           "egress_bytes_per_rank": [int(sum(s[5 + o] for s in per_rank)) for o in range(world)],
                           "spmm_ms_per_rank": [round(s[0], 3) for s in per_rank],
                           "fetch_ms_per_rank": [round(s[1], 3) for s in per_rank]},
                "roofline": {"bound": "hbm", "kernel": "spmm_kernel<32,1,4,false> (rank 0 shard)",
                             "achieved": achieved, "peak": peak, "peak_kind": "of " + peak_kind, "unit": "GB/s",
                             "frac": achieved / peak, "frac_of_nominal_8000": achieved / 8000.0,
                             "algorithmic_bytes_per_launch": k_bytes, "avg_launch_ms": k_ms,
                             "traffic": bench.load_traffic("spmm_partitioned_d128")},
                "nvlink": None if max_fetch == 0 else {
                    "halo_fetch_ms_max": max_fetch, "halo_bytes_max": max_halo,
                    "achieved_gbs": max(s[2] / (s[1] * 1e-3) / 1e9 for s in per_rank if s[1] > 0),
                    "peak_gbs": NVLINK_PEER_GBS, "note": "plain peer loads, each needed source row crosses once"},
                "single_gpu_value": single, "speedup_vs_single_gpu": None if single is None else value / single,
                "cpu_baseline": None,
                "e2e": {"value": nnz * d / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
                        "h2d_bytes_per_step": int(bytes_io), "d2h_bytes_per_step": int(bytes_io)},
                "gpu_launches": int(round(launches_per_step)) * args.steps * world, "clocks": clocks}
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle as O
            sh = RowShard(indptr, indices, values, partition_bounds(indptr, 16), 8)
            xs = graphs.randn_features(1, n, d, device=dev).cpu().numpy()
            ip, ix, vals = sh.indptr.cpu().numpy(), sh.indices.cpu().numpy(), sh.values.cpu().numpy()
            O.build()
            O.set_threads(len(os.sched_getaffinity(0)))
            t_best = None
            for _ in range(5):
                t0 = time.perf_counter()
                O.spmm(ip, ix, xs, wmode=O.W_EDGE, values=vals)
                t_best = min(t_best or 1e9, time.perf_counter() - t0)
            line["cpu_baseline"] = {"value": sh.nnz * d / t_best / 1e9, "unit": UNIT,
                                    "cores": len(os.sched_getaffinity(0)), "kind": "port", "seconds": round(t_best, 3),
                                    "sample": "partition 8 of 16 (%d of %d edges), best of 5" % (sh.nnz, nnz)}
        print(json.dumps(line))
    runner.close()
    if world > 1:
        dist.destroy_process_group()
