"""bench.py's leg for the row-partitioned SpMM (R-MAT N=2^24, 2^29 sampled edges, int64 row pointers, fp32
weights 1/in-degree, 128 features), one process per GPU; with one GPU the shard is the whole graph.  Strong
scaling: the graph is fixed, each rank aggregates its edge-balanced row range.  Every rank builds the same graph
from the same seed on its own GPU (integer generator, bit-identical everywhere) and keeps its shard.

Before anything is timed every rank checks rows of its own output against float64 sums formed from the definition
(features are a function of the global row id, so any rank can produce any source row); the line carries the
outcome as "verify" and the process exits non-zero when the check fails."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

METRIC = "aggregation_gedge_feat_per_s"
UNIT = "Gedge*feat/s"
NVLINK_PEER_GBS = 770.0  # peer-copy bandwidth per direction measured between two B200s through NVSwitch (nominal 900)
FEATURE_SEED = 1


def workload_name(n, e, d):
    return "partitioned_spmm_rmat_n%d_e%d_d%d" % (n, e, d)


def _reference_leg(args, device, n, e, d):
    """CPU restatement on all host cores, on the rows of partition 8 of 16 (bounded sample).  The graph is made with
    torch on the GPU (the generator is plain tensor arithmetic); nothing of the CUDA library is loaded or called."""
    from oracle import oracle as O
    from yitu_b200 import graphs
    indptr, indices, values = graphs.spmm_partitioned(device=device, n=n, e=e)
    nnz = indices.numel()
    targets = torch.tensor([(8 * nnz + 15) // 16, (9 * nnz + 15) // 16], device=device)
    lo, hi = torch.searchsorted(indptr, targets).tolist()  # the edge-balanced bounds of partition 8 of 16
    e0, e1 = int(indptr[lo]), int(indptr[hi])
    x = graphs.randn_features(FEATURE_SEED, n, d, device=device).cpu().numpy()
    ip = (indptr[lo:hi + 1] - e0).cpu().numpy()
    ix, vals = indices[e0:e1].cpu().numpy(), values[e0:e1].cpu().numpy()
    del indptr, indices, values
    O.build()
    cores = O.set_threads(len(os.sched_getaffinity(0)))  # torchrun exports OMP_NUM_THREADS=1
    best = None
    reps = max(1, args.steps + args.warmup)
    for _ in range(reps):
        t0 = time.perf_counter()
        O.spmm(ip, ix, x, wmode=O.W_EDGE, values=vals)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    value = (e1 - e0) * d / best / 1e9
    base = {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "seconds": round(best, 3),
            "sample": "partition 8 of 16 (%d rows, %d of %d edges), forward SpMM, full feature matrix; best of %d" % (
                hi - lo, e1 - e0, nnz, reps)}
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": best * 1e3, "higher_is_better": True,
                      "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": workload_name(n, e, d),
                                 "note": "CPU restatement of the reference kernels; the reference has no CPU "
                                         "implementation of this path"},
                      "cpu_baseline": base,
                      "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))
    return base


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


def verify_rows(shard, out, d, n_random=96, chunk=1 << 16):
    """Sampled rows of this rank's output against float64 sums taken from the definition, out[r] = sum_e w_e * x[col_e]
    with x regenerated from the global column ids: the longest row, the last row, the row that holds the largest
    source id, and seeded random ones.  Returns (rows checked, worst |err| / max|truth|, ok) at the parity bar of the
    test suite, |err| <= 1e-5 * (|truth| + max|truth|)."""
    from yitu_b200 import graphs
    dev = out.device
    n_local = shard.n_local
    if n_local == 0:
        return 0, 0.0, True
    deg = shard.indptr[1:] - shard.indptr[:-1]
    gen = torch.Generator(device="cpu").manual_seed(1000 + shard.rank)
    picks = [int(deg.argmax()), n_local - 1, 0]
    if shard.nnz:
        far = int(shard.indices.argmax())
        picks.append(int(torch.searchsorted(shard.indptr, torch.tensor([far], device=dev), right=True)[0]) - 1)
    picks += torch.randint(0, n_local, (n_random,), generator=gen).tolist()
    rows = sorted(set(picks))
    truth = torch.zeros(len(rows), d, dtype=torch.float64, device=dev)
    for i, r in enumerate(rows):
        b, e = int(shard.indptr[r]), int(shard.indptr[r + 1])
        for s in range(b, e, chunk):
            t = min(s + chunk, e)
            cols = shard.indices[s:t].long()
            xs = graphs.randn_rows(FEATURE_SEED, cols, d).double()
            w = shard.values[s:t].double() if shard.values is not None else torch.ones(t - s, dtype=torch.float64, device=dev)
            truth[i] += (w[:, None] * xs).sum(0)
    got = out[torch.tensor(rows, device=dev)].double()
    scale = float(truth.abs().max())
    err = (got - truth).abs()
    ok = bool(torch.isfinite(got).all()) and float((err - 1e-5 * (truth.abs() + scale)).max()) <= 0.0
    return len(rows), float(err.max()) / max(scale, 1e-30), ok


class ShardOnOneGpu:
    """One rank's share of a P-way split, aggregated on ONE GPU from the whole feature matrix (global column ids, no
    exchange): the kernel of that rank of a multi-GPU run, in a form that a single-GPU profiler can capture."""
    mode, schedule, halo_bytes, plan = "local", None, 0, None

    def __init__(self, shard, n, d, device):
        from yitu_b200 import graphs, ops
        self.ops, self.device, self.shard = ops, device, shard
        self.graph = ops.PreparedGraph(shard.indptr, shard.indices, n)
        self.x = graphs.randn_features(FEATURE_SEED, n, d, device=device)
        self.x_local = self.x[shard.row_begin:shard.row_end]
        self.out = torch.empty(shard.n_local, d, device=device)

    def step(self, events=None):
        a = b = None
        if events is not None:
            a = torch.cuda.Event(enable_timing=True)
            a.record()
        out = self.ops.spmm(self.graph, self.x, mode=self.ops.W_EDGE, edge_values=self.shard.values, out=self.out)
        if events is not None:
            b = torch.cuda.Event(enable_timing=True)
            b.record()
            events.append(("spmm", a, b))
        return out

    def close(self):
        pass


def step_timeline(runner, rank, world):
    """Where the time of a push-mode step goes on every rank: one step with events; offsets in ms from the moment
    the step's opening handshake completed on that rank."""
    dev = runner.device
    ev = []
    runner.step(ev)
    torch.cuda.synchronize(dev)
    t0 = [a for tag, a, _ in ev if tag == "start"][0]
    mine = {"rank": rank,
            "push": [[round(t0.elapsed_time(a), 3), round(t0.elapsed_time(b), 3)] for tag, a, b in ev if tag == "push"],
            "ready": {tag[6:]: round(a.elapsed_time(b), 3) for tag, a, b in ev if tag.startswith("ready:")},
            "passes": [[round(t0.elapsed_time(a), 3), round(t0.elapsed_time(b), 3)] for tag, a, b in ev if tag == "spmm"],
            "end": [round(a.elapsed_time(b), 3) for tag, a, b in ev if tag == "end"][0]}
    out = [None] * world
    dist.all_gather_object(out, mine)
    return out


def run(args):
    import bench  # the repo-root script: clock sampler, peak numbers, the secondary workloads
    from yitu_b200 import graphs
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
        _reference_leg(args, dev, n, e, d)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    indptr, indices, values = graphs.spmm_partitioned(device=dev, n=n, e=e)
    nnz = indices.numel()
    one_shard = world == 1 and args.shard_of > 1
    bounds = partition_bounds(indptr, args.shard_of if one_shard else world, row_cost=args.row_cost)
    shard = RowShard(indptr, indices, values, bounds, args.shard if one_shard else rank)
    if one_shard:
        nnz = shard.nnz  # the unit count of this run is the shard's
    del indptr, indices, values
    torch.cuda.empty_cache()
    x_shard = graphs.randn_features(FEATURE_SEED, shard.n_local, d, device=dev, row_begin=shard.row_begin)

    modes = ["local"] if world == 1 else [m for m in args.halo.split(",") if m]
    runners, trial, verify, timelines, schedules = {}, {}, {}, {}, {}
    for mode in modes:
        kw = {}
        name = mode
        if mode.startswith("push"):  # "push", "push1".."push4": at most that many passes; "pushnp": no priority rank; "pushsp": the priority
            # rank aggregates in a single pass
            kw = dict(max_passes=int(mode[4:]) if mode[4:].isdigit() else 3,
                      priority=None if mode.endswith("np") else "auto", priority_own_first=False if mode.endswith("sp") else "auto")
            mode = "push"
        r = ShardOnOneGpu(shard, n, d, dev) if one_shard else PartitionedSpmm(shard, d, dev, mode=mode, **kw)
        r.x_local.copy_(x_shard)
        runners[name] = r
        out = None
        for _ in range(3):
            out = r.step()
        # correctness first: sampled rows of this rank's result against float64, before anything is timed
        k, err, ok = verify_rows(shard, out, d)
        stat = torch.tensor([float(k), err, 0.0 if ok else 1.0], device=dev, dtype=torch.float64)
        if world > 1:
            both = [torch.zeros_like(stat) for _ in range(world)]
            dist.all_gather(both, stat)
            stat = torch.stack(both)
            stat = torch.stack([stat[:, 0].sum(), stat[:, 1].max(), stat[:, 2].sum()])
        verify[name] = {"rows": int(stat[0]), "max_rel_err": float(stat[1]), "ok": float(stat[2]) == 0.0,
                        "bar": "|err| <= 1e-5*(|truth| + max|truth|), float64 truth, every rank checks its own rows"}
        trial[name] = _time_steps(r, 3, world)
        if mode == "push":
            timelines[name] = step_timeline(r, rank, world)
            schedules[name] = r.schedule.describe()
    bad = [k for k, v in verify.items() if not v["ok"]]
    if bad:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "error": "result check failed", "verify": verify}))
        sys.exit(1)
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
    if hasattr(runner, "check"):
        runner.check()  # raises if a wait for a peer's delivery ever ran out: the timed steps would be worthless
    value = nnz * d / (ms_step * 1e-3) / 1e9

    spmm_ms = [a.elapsed_time(b) for tag, a, b in events if tag == "spmm"]
    move_ms = [a.elapsed_time(b) for tag, a, b in events if tag == "fetch"]
    if runner.mode == "push":
        # per step: from the start of the step to the end of this rank's last push kernel (the priority delivery and
        # the main push run side by side)
        t0, ends = None, {}
        for tag, a, b in events:
            if tag == "start":
                t0 = a
            elif tag == "push" and t0 is not None:
                ends[id(t0)] = max(ends.get(id(t0), 0.0), t0.elapsed_time(b))
        move_ms = list(ends.values())
    n_spmm = len(spmm_ms) / args.steps
    n_move = sum(1 for tag, _, _ in events if tag == "fetch") / args.steps
    if runner.mode == "push":
        n_move = (runner._push_first is not None) + (runner._push_rest is not None)
        graphs_used = [g for g, _, _ in runner._passes]
    else:
        graphs_used = [runner.graph]
    # this library's kernels per step on this rank: the gather / push kernels, one SpMM per pass and one hub
    # reduction for every pass whose graph has split rows
    launches = n_move + sum(bench.spmm_launches(g.nnz, g.n_rows, d, g.plan() is not None) for g in graphs_used)
    k_ms = sum(spmm_ms) / args.steps  # SpMM time per step on this rank (all passes)
    k_bytes = shard.nnz * (4 * d + 8) + (shard.n_local + 1) * 8 + 4 * shard.n_local * d
    by_owner = [0.0] * world  # bytes this rank receives from each owner per step
    if getattr(runner, "plan", None) is not None and world > 1:
        off = runner.plan.owner_offsets
        by_owner = [float((off[p + 1] - off[p]) * d * 4) for p in range(world)]
    stats = torch.tensor([k_ms, sum(move_ms) / args.steps if move_ms else 0.0, float(runner.halo_bytes),
                          float(shard.nnz), float(shard.n_local), float(launches), n_spmm] + by_owner,
                         device=dev, dtype=torch.float64)
    all_stats = [torch.zeros_like(stats) for _ in range(world)]
    if world > 1:
        dist.all_gather(all_stats, stats)
    else:
        all_stats = [stats]

    timeline = timelines.get(best)

    # end to end: pinned host shard in, result shard back to pinned host memory, every step.  The copies of
    # neighbouring steps overlap the aggregation: step k+1's features arrive in a staging buffer on a copy-in stream
    # while step k aggregates and step k-1's result leaves from a second staging buffer on a copy-out stream (PCIe is
    # full duplex); every step's H2D and D2H lie inside the timed region.
    h_x = x_shard.cpu().pin_memory()
    h_out = torch.empty(shard.n_local, d).pin_memory()
    stage_in, stage_out = torch.empty_like(x_shard), torch.empty_like(x_shard)
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    class E2E:
        device = dev

        def __init__(self):
            self.in_done = self.consumed = self.out_ready = self.out_free = None

        def prefetch(self):
            with torch.cuda.stream(s_in):
                if self.consumed is not None:
                    s_in.wait_event(self.consumed)
                stage_in.copy_(h_x, non_blocking=True)
                self.in_done = s_in.record_event()

        def step(self, events=None):
            main = torch.cuda.current_stream(dev)
            if self.in_done is None:
                s_in.wait_stream(main)
                self.prefetch()
            main.wait_event(self.in_done)
            runner.x_local.copy_(stage_in, non_blocking=True)
            self.consumed = main.record_event()
            self.prefetch()  # the next step's input, while this one aggregates
            out = runner.step()
            if self.out_free is not None:
                main.wait_event(self.out_free)
            stage_out.copy_(out, non_blocking=True)
            self.out_ready = main.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(self.out_ready)
                h_out.copy_(stage_out, non_blocking=True)
                self.out_free = s_out.record_event()

        def drain(self):
            main = torch.cuda.current_stream(dev)
            main.wait_stream(s_out)
            main.wait_stream(s_in)

    e2e_ms, timed, e2e_runner = None, None, None
    if not args.no_e2e:
        e2e_runner = E2E()
        for _ in range(2):
            e2e_runner.step()
        e2e_runner.drain()
        e2e_steps = max(3, min(args.steps, 6))

        class Timed:
            device = dev

            def step(self, events=None):
                e2e_runner.step()
                if self.left == 1:
                    e2e_runner.drain()  # the last result has to be on the host before the clock stops
                self.left -= 1

        timed = Timed()
        timed.left = e2e_steps
        e2e_ms = _time_steps(timed, e2e_steps, world)
    bytes_io = torch.tensor([h_x.numel() * 4.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(bytes_io)
        dist.barrier()
    torch.cuda.synchronize(dev)
    del stage_in, stage_out, timed
    schedule = runner.schedule.describe() if runner.schedule is not None else None
    runner.close()
    del runner, runners, h_x, h_out, x_shard, shard, e2e_runner
    torch.cuda.empty_cache()

    if rank == 0:
        peak, peak_kind = bench.load_peaks()
        per_rank = [[float(v) for v in s.tolist()] for s in all_stats]
        egress = [sum(s[7 + o] for s in per_rank) for o in range(world)]
        move_max = max(s[1] for s in per_rank)
        roof = bench.roofline(bench.spmm_kernel_name(int(per_rank[0][3]), int(per_rank[0][4]), d) +
                              (" (rank 0 shard, all passes)" if world > 1 else ""),
                              k_bytes, k_ms, "spmm_partitioned_d128" if world == 1 and not args.scale and not one_shard else None)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic",
                "config": {"workload": workload_name(n, e, d) + ("_shard%d_of_%d" % (args.shard, args.shard_of) if one_shard else ""),
                           "nnz": nnz,
                           "parallelism": "row_partition_%d" % world,
                           "balance": "edges" if not args.row_cost else "edges + %d * rows" % args.row_cost,
                           "halo": best, "trial_ms": trial, "schedule": schedule, "timeline_ms": timeline,
                           "other_trials": {k: {"schedule": schedules[k], "timeline_ms": timelines[k]}
                                            for k in timelines if k != best} if args.verbose_trials else None,
                           "l2": "inputs_larger_than_l2", "rows_per_rank": [int(s[4]) for s in per_rank],
                           "edges_per_rank": [int(s[3]) for s in per_rank],
                           "halo_bytes_per_rank": [int(s[2]) for s in per_rank],
                           "egress_bytes_per_rank": [int(v) for v in egress],
                           "spmm_ms_per_rank": [round(s[0], 3) for s in per_rank],
                           "spmm_passes_per_rank": [int(round(s[6])) for s in per_rank],
                           "exchange_ms_per_rank": [round(s[1], 3) for s in per_rank]},
                "verify": verify[best],
                "roofline": roof,
                "nvlink": None if move_max == 0 else {
                    "largest_egress_bytes": max(egress), "its_exchange_ms": per_rank[egress.index(max(egress))][1]
                    if best.startswith("push") else move_max,
                    "achieved_gbs": (max(egress) / (per_rank[egress.index(max(egress))][1] * 1e-3) / 1e9)
                    if best.startswith("push") else max(s[2] / (s[1] * 1e-3) / 1e9 for s in per_rank if s[1] > 0),
                    "peak_gbs": NVLINK_PEER_GBS,
                    "note": ("owner-side push: bytes leaving the busiest owner / duration of its push kernels"
                             if best.startswith("push") else
                             "reader-side peer loads: halo bytes of a rank / duration of its gather kernel (best rank)")},
                "cpu_baseline": None,
                "e2e": None if e2e_ms is None else {
                    "value": nnz * d / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(bytes_io), "d2h_bytes_per_step": int(bytes_io),
                    "mode": "pipelined: copy-in / aggregation / copy-out of neighbouring steps overlap"},
                "gpu_launches": int(round(sum(s[5] for s in per_rank))) * args.steps, "clocks": clocks}
        if not args.no_cpu_baseline:
            try:
                line["cpu_baseline"] = bench.cpu_baseline_partitioned(dev, n, e, d, repeats=5 if world == 1 else 2,
                                                                          min_seconds=10.0 if world == 1 else 0.0)
            except Exception as exc:  # never lose the line to the extra measurement
                line["cpu_baseline"] = {"error": str(exc)[:200]}
        if world == 1 and not args.scale and not args.no_sub_records and not one_shard:
            for key, fn in (("spmm_c2", bench.sub_record_spmm), ("gat_layer", bench.sub_record_gat),
                            ("rgcn_layer", bench.sub_record_rgcn), ("spmm_uniform", bench.sub_record_uniform)):
                try:
                    line[key] = fn(dev)
                except Exception as exc:
                    line[key] = {"error": str(exc)[:200]}
                torch.cuda.empty_cache()
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
