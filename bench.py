#!/usr/bin/env python
"""Benchmark of the GNN aggregation hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload spmm|gat|rgcn|partitioned] [--impl reference]

Prints ONE JSON line.  metric = aggregation throughput in Gedge*feat/s (stored edges x feature width per
second, whole job).  A step is one pass of the workload's hot path over the resident synthetic graph:

  partitioned  N GPUs R-MAT N=2^24, 2^29 sampled edges, int64 row pointers, D=128, rows split into N
                      edge-balanced ranges, halo source rows pushed over NVLink by their owners (strong scaling);
                      with N=1 the whole graph on one GPU
  spmm         1 GPU  R-MAT N=2^21, 2^26 sampled edges (deduplicated), fp32 per-edge symmetric-normalised
                      weights, D=256: forward A*X and the transposed product A^T*G (2 * nnz * D edge-feats)
  gat          1 GPU  uniform random N=2^20, 2^25 edges + self loops, 8 heads x 32: fused GAT forward+backward
  rgcn         1 GPU  4 node types, 8 bipartite R-MAT relations x 4M edges, D=64: mean per relation, sum per type
  uniform      1 GPU  (not a configuration) uniform random N=2^23, 2^27 edges, D=128: no hot rows, the gather ceiling

Default at every N: partitioned - ONE series at 1/2/4/8 GPUs, the same graph throughout.  The N=1 line also
carries the other three configurations as sub-records (spmm_c2, gat_layer, rgcn_layer), each with its own time and
roofline.  Inputs are far larger than L2 (126 MB), so no flush is needed between timed iterations.
`--impl reference` times the CPU restatement of the reference kernels (the reference has no CPU implementation of
this path) on all host cores, on a bounded row slice.

roofline keys: `frac` = algorithmic bytes (every edge counts its whole source row, no cache credit) / kernel time /
measured HBM copy bandwidth - it exceeds 1 where the L2 serves the hot rows of a power-law graph; `dram_frac` =
DRAM bytes per launch as counted by ncu (`traffic`, from the committed capture named in `traffic_source`) / kernel
time / the same peak - the physical share of HBM bandwidth; `compulsory_frac` = bytes that must move at least once
(each source row, index, weight and output row once) / kernel time / peak.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "aggregation_gedge_feat_per_s"
UNIT = "Gedge*feat/s"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def load_traffic(key, kernel):
    """DRAM bytes per launch of a workload's dominant kernel from the committed ncu captures
    (profiles/dram_traffic.json): (bytes, provenance), or (None, why) when there is no capture of THIS kernel on
    this workload - a figure taken with another kernel is not reported."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if key is None or not os.path.exists(path):
        return None, "no capture"
    with open(path) as f:
        rec = json.load(f).get(key)
    if not isinstance(rec, dict):
        return None, "no capture"
    if rec.get("kernel", "").split("<")[0] != kernel.split("<")[0].split(" ")[0]:
        return None, "the capture on file is of %s" % rec.get("kernel")
    return rec["bytes"], rec.get("source")


def spmm_kernel_name(nnz, n_rows, d):
    """The SpMM instantiation that yitu_spmm_csr_f32 picks for scalar weights and aligned rows of d floats: below 64
    edges per row on average (24 for rows of more than 128 floats) the edge-stream kernel, with the chunks of hub rows
    on the warp-per-row kernel; above, the warp-per-row kernel alone."""
    split = nnz < (24 if d > 128 else 64) * n_rows and 64 < d <= 256
    if d > 128:
        return "spmm_stream_kernel<8,4,16,true,true> (+ spmm_kernel<32,1,8,4,false,true> on hub chunks)" if split \
            else "spmm_kernel<32,1,8,4,false,true>"
    return "spmm_stream_kernel<4,8,16,true,true> (+ spmm_kernel<32,1,4,16,false,true> on hub chunks)" if split \
        else "spmm_kernel<32,1,4,16,false,true>"


def spmm_launches(nnz, n_rows, d, has_hub_plan):
    """Kernels one scalar-weight SpMM call launches: the aggregation (two kernels where hub chunks and ordinary rows
    go to different kernels, see spmm_kernel_name) and, with a hub schedule, the reduction of the chunk partials."""
    if not has_hub_plan:
        return 1
    split = nnz < (24 if d > 128 else 64) * n_rows and 64 < d <= 256
    return 3 if split else 2


def roofline(kernel, algorithmic_bytes, avg_launch_ms, traffic_key, compulsory_bytes=None):
    peak, peak_kind = load_peaks()
    achieved = algorithmic_bytes / (avg_launch_ms * 1e-3) / 1e9
    traffic, source = load_traffic(traffic_key, kernel)
    out = {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "peak_kind": "of " + peak_kind,
           "unit": "GB/s", "frac": achieved / peak, "frac_of_nominal_8000": achieved / 8000.0,
           "algorithmic_bytes_per_launch": algorithmic_bytes, "avg_launch_ms": avg_launch_ms,
           "traffic": traffic, "traffic_source": source,
           "dram_frac": None if traffic is None else traffic / (avg_launch_ms * 1e-3) / 1e9 / peak,
           "note": "frac counts algorithmic bytes (L2 hits included, can exceed 1); dram_frac counts DRAM bytes"}
    if compulsory_bytes is not None:
        out["compulsory_bytes_per_launch"] = compulsory_bytes
        out["compulsory_frac"] = compulsory_bytes / (avg_launch_ms * 1e-3) / 1e9 / peak
    return out


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=5)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for nm, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------ workloads
class SpmmWorkload:
    """configs[1]: forward and transposed sum-aggregation SpMM."""
    name = "spmm_rmat_n2097152_e67108864_d256_fwd_bwd"
    dominant_kernel = "spmm_stream_kernel<8,4,16,true,true>"

    def __init__(self, device, n=1 << 21, e=1 << 26, d=256):
        import torch
        from yitu_b200 import graphs, ops
        self.torch, self.ops = torch, ops
        self.n, self.d = n, d
        self.indptr, self.indices, self.values = graphs.spmm_rmat(device=device, n=n, e=e)
        self.nnz = self.indices.numel()
        self.g = ops.PreparedGraph(self.indptr, self.indices, n)
        self.gt = self.g.t_prepared()
        self.values_t = self.values[self.g.transpose()[2].long()].contiguous()  # static weights, permuted once
        self.x = graphs.randn_features(1, n, d, device=device)
        self.grad = graphs.randn_features(2, n, d, device=device)
        self.out = torch.empty_like(self.x)
        self.gout = torch.empty_like(self.x)
        self.g.plan(), self.gt.plan()
        self.units_per_step = 2 * self.nnz * d
        self.launches_per_step = (spmm_launches(self.nnz, n, d, bool(self.g.plan())) +
                                  spmm_launches(self.nnz, n, d, bool(self.gt.plan())))
        self.kernel_launches_per_step = 2
        # algorithmic bytes of ONE SpMM launch: per edge a feature row, a column id and a weight; per row a
        # pointer and the written output row
        self.kernel_bytes = self.nnz * (4 * d + 8) + (n + 1) * 4 + 4 * n * d
        self.compulsory_bytes = self.nnz * 8 + (n + 1) * 4 + 2 * 4 * n * d  # every source row and output row once
        self.traffic_key = "spmm_rmat_d256"
        self.dominant_kernel = spmm_kernel_name(self.nnz, n, d)

    def step(self, kernel_events=None):
        t, ops = self.torch, self.ops
        if kernel_events is not None:
            a, b, c = (t.cuda.Event(enable_timing=True) for _ in range(3))
            a.record()
        ops.spmm(self.g, self.x, mode=ops.W_EDGE, edge_values=self.values, out=self.out)
        if kernel_events is not None:
            b.record()
        ops.spmm(self.gt, self.grad, mode=ops.W_EDGE, edge_values=self.values_t, out=self.gout)
        if kernel_events is not None:
            c.record()
            kernel_events.append((a, b))
            kernel_events.append((b, c))

    def e2e_setup(self):
        t = self.torch
        self.h_x = self.x.cpu().pin_memory()
        self.h_g = self.grad.cpu().pin_memory()
        self.h_out = t.empty(self.x.shape, dtype=t.float32).pin_memory()
        self.h_gout = t.empty(self.x.shape, dtype=t.float32).pin_memory()
        self.h2d = 2 * self.x.numel() * 4
        self.d2h = 2 * self.x.numel() * 4

    def e2e_step(self):
        ops = self.ops
        x = self.h_x.to(self.x.device, non_blocking=True)
        g = self.h_g.to(self.x.device, non_blocking=True)
        out = ops.spmm(self.g, x, mode=ops.W_EDGE, edge_values=self.values)
        gout = ops.spmm(self.gt, g, mode=ops.W_EDGE, edge_values=self.values_t)
        self.h_out.copy_(out, non_blocking=True)
        self.h_gout.copy_(gout, non_blocking=True)

    def e2e_run(self, steps):
        """Pipelined end-to-end loop: the step's two feature matrices are copied in from pinned host memory on a copy-in
        stream, aggregated on the compute stream through the public ops.spmm call, and the two results copied back to
        pinned host memory on a copy-out stream; buffers are double-buffered so that the copy-in of step k+1 and the
        copy-out of step k-1 (PCIe is full duplex) run beside the compute of step k.  Returns ms per step, with every
        step's H2D and D2H inside the timed region."""
        t, ops, dev = self.torch, self.ops, self.x.device
        main = t.cuda.current_stream(dev)
        s_in, s_out = t.cuda.Stream(device=dev), t.cuda.Stream(device=dev)
        bufs = [{k: t.empty_like(self.x) for k in ("x", "g", "out", "gout")} for _ in range(2)]
        in_done = [None, None]
        comp_done = [None, None]
        out_done = [None, None]
        start, stop = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
        t.cuda.synchronize(dev)
        start.record(main)
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        for k in range(steps):
            b = bufs[k % 2]
            with t.cuda.stream(s_in):
                if comp_done[k % 2] is not None:
                    s_in.wait_event(comp_done[k % 2])  # the compute that read this input buffer two steps ago
                b["x"].copy_(self.h_x, non_blocking=True)
                b["g"].copy_(self.h_g, non_blocking=True)
                in_done[k % 2] = s_in.record_event()
            main.wait_event(in_done[k % 2])
            if out_done[k % 2] is not None:
                main.wait_event(out_done[k % 2])  # the copy-out that read this output buffer two steps ago
            ops.spmm(self.g, b["x"], mode=ops.W_EDGE, edge_values=self.values, out=b["out"])
            ops.spmm(self.gt, b["g"], mode=ops.W_EDGE, edge_values=self.values_t, out=b["gout"])
            comp_done[k % 2] = main.record_event()
            with t.cuda.stream(s_out):
                s_out.wait_event(comp_done[k % 2])
                self.h_out.copy_(b["out"], non_blocking=True)
                self.h_gout.copy_(b["gout"], non_blocking=True)
                out_done[k % 2] = s_out.record_event()
        main.wait_stream(s_out)
        stop.record(main)
        t.cuda.synchronize(dev)
        return start.elapsed_time(stop) / steps

    def verify(self):
        """A*1 equals the in-degree exactly; cheap, size-independent."""
        t, ops = self.torch, self.ops
        ones = t.ones(self.n, 4, device=self.x.device)
        deg = (self.indptr[1:] - self.indptr[:-1]).float()
        assert t.equal(ops.spmm(self.g, ones)[:, 0], deg), "SpMM self-check failed"

    def cpu_sample(self, seconds_hint=15.0):
        """CPU baseline sample: the whole forward SpMM (about a second per pass on 16 cores), repeated."""
        lo, hi = 0, self.n
        ip = self.indptr[lo:hi + 1].cpu().numpy().astype("int64")
        e0, e1 = int(ip[0]), int(ip[-1])
        return dict(indptr=ip - e0, indices=self.indices[e0:e1].cpu().numpy(), values=self.values[e0:e1].cpu().numpy(),
                    x=self.x.cpu().numpy(), nnz=e1 - e0, d=self.d,
                    sample="rows [%d,%d) of %d (%d of %d edges), forward SpMM, full feature matrix" % (
                        lo, hi, self.n, e1 - e0, self.nnz))


class GatWorkload:
    """configs[2]: fused GAT layer core forward + backward."""
    name = "gat_uniform_n1048576_e33554432_h8_f32_fwd_bwd"
    dominant_kernel = "gat_fwd_kernel_r64<2,false,false>"

    def __init__(self, device, n=1 << 20, e=1 << 25, H=8, F=32):
        import torch
        from yitu_b200 import graphs, ops
        self.torch, self.ops = torch, ops
        self.n, self.H, self.F, self.d = n, H, F, H * F
        self.indptr, self.indices = graphs.gat_uniform(device=device, n=n, e=e)
        self.nnz = self.indices.numel()
        self.g = ops.PreparedGraph(self.indptr, self.indices, n)
        self.g.transpose()
        self.g.t_prepared().plan()
        self.x = graphs.randn_features(1, n, H * F, device=device).view(n, H, F)
        a_src = graphs.uniform_values(5, (H, F), -0.1, 0.1, device=device)
        a_dst = graphs.uniform_values(6, (H, F), -0.1, 0.1, device=device)
        self.k = (self.x * a_src).sum(-1).contiguous()
        self.q = (self.x * a_dst).sum(-1).contiguous()
        self.grad = graphs.randn_features(2, n, H * F, device=device).view(n, H, F)
        self.units_per_step = 2 * self.nnz * self.d
        self.launches_per_step = 1 + 3  # fused forward; backward = edge kernel, transposed SpMM, per-source sum
        self.kernel_launches_per_step = 1
        self.kernel_bytes = self.nnz * (4 + 4 * H + 4 * H * F) + n * (4 + 4 * H + 4 * H * F + 8 * H)
        self.compulsory_bytes = self.nnz * 4 + n * (4 + 8 * H + 2 * 4 * H * F + 8 * H)
        self.traffic_key = "gat_fwd_h8_f32"

    def step(self, kernel_events=None):
        t, ops = self.torch, self.ops
        if kernel_events is not None:
            a, b = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            a.record()
        out, rmax, rsum = ops.gat_fwd(self.g, self.q, self.k, self.x)
        if kernel_events is not None:
            b.record()
            kernel_events.append((a, b))
        self.res = ops.gat_bwd(self.g, self.q, self.k, self.x, out, rmax, rsum, self.grad)

    def e2e_setup(self):
        t = self.torch
        self.h_x = self.x.cpu().pin_memory()
        self.h_g = self.grad.cpu().pin_memory()
        self.h_out = t.empty(self.x.shape, dtype=t.float32).pin_memory()
        self.h2d = 2 * self.x.numel() * 4
        self.d2h = self.x.numel() * 4

    def e2e_step(self):
        ops = self.ops
        x = self.h_x.to(self.x.device, non_blocking=True)
        g = self.h_g.to(self.x.device, non_blocking=True)
        out, rmax, rsum = ops.gat_fwd(self.g, self.q, self.k, x)
        gq, gk, gx = ops.gat_bwd(self.g, self.q, self.k, x, out, rmax, rsum, g)
        self.h_out.copy_(gx, non_blocking=True)

    def verify(self):
        t, ops = self.torch, self.ops
        out, _, rsum = ops.gat_fwd(self.g, self.q, self.k, t.ones_like(self.x))
        assert float((out - 1.0).abs().max()) < 1e-5, "GAT self-check failed (softmax weights must sum to 1)"

    def cpu_sample(self, seconds_hint=15.0):
        lo, hi = 0, self.n
        ip = self.indptr[lo:hi + 1].cpu().numpy().astype("int64")
        e0, e1 = int(ip[0]), int(ip[-1])
        return dict(indptr=ip - e0, indices=self.indices[e0:e1].cpu().numpy(), q=self.q[lo:hi].cpu().numpy(),
                    k=self.k.cpu().numpy(), x=self.x.cpu().numpy(), nnz=e1 - e0, d=self.d, gat=True,
                    sample="rows [%d,%d) of %d (%d of %d edges), GAT forward (edge softmax + SpMM)" % (
                        lo, hi, self.n, e1 - e0, self.nnz))


class RgcnWorkload:
    """configs[3]: hetero RGCN aggregation: per destination type one pass over the stitched relations."""
    name = "rgcn_4types_8rel_x4M_d64"
    dominant_kernel = "spmm_wide_kernel<8,1,true>"

    def __init__(self, device, d=64):
        import torch
        from yitu_b200 import graphs, ops
        from yitu_b200.xgnn_h import Block, stitch_csr
        self.torch, self.ops, self.d = torch, ops, d
        sizes = graphs.HETERO_TYPES
        rels = graphs.hetero_rgcn(device=device)
        self.feats = [graphs.randn_features(10 + r, sizes[st], d, device=device) for r, (st, dt, _, _) in enumerate(rels)]
        self.groups = []
        self.nnz, self.kernel_bytes = 0, 0
        for dt in sorted({r[1] for r in rels}):
            ids = [i for i, r in enumerate(rels) if r[1] == dt]
            st_blk = stitch_csr([Block([sizes[dt], sizes[rels[i][0]]], [rels[i][2], rels[i][3]]) for i in ids]).to(device)
            xcat = torch.cat([self.feats[i] for i in ids])
            g = ops.prepared(st_blk.adj_sparse[0], st_blk.adj_sparse[1], xcat.size(0), ops.STITCH_MASK)
            w = g.segment_mean_weights()
            g.plan()
            self.groups.append((g, w, xcat, torch.empty(sizes[dt], d, device=device), st_blk))
            self.nnz += g.nnz
            self.kernel_bytes += g.nnz * (4 * d + 8) + (sizes[dt] + 1) * 4 + 4 * sizes[dt] * d
        self.kernel_bytes //= len(self.groups)
        self.compulsory_bytes = None
        self.units_per_step = self.nnz * d
        self.launches_per_step = sum(1 + (1 if g.plan() else 0) for g, *_ in self.groups)
        self.kernel_launches_per_step = len(self.groups)
        self.traffic_key = "rgcn_d64"

    def step(self, kernel_events=None):
        t, ops = self.torch, self.ops
        for g, w, xcat, out, _ in self.groups:
            if kernel_events is not None:
                a, b = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
                a.record()
            ops.spmm(g, xcat, mode=ops.W_EDGE, edge_values=w, out=out)
            if kernel_events is not None:
                b.record()
                kernel_events.append((a, b))

    def e2e_setup(self):
        self.h_x = [xc.cpu().pin_memory() for _, _, xc, _, _ in self.groups]
        self.h_out = [o.cpu().pin_memory() for _, _, _, o, _ in self.groups]
        self.h2d = sum(x.numel() * 4 for x in self.h_x)
        self.d2h = sum(o.numel() * 4 for o in self.h_out)

    def e2e_step(self):
        ops = self.ops
        for (g, w, xcat, out, _), hx, ho in zip(self.groups, self.h_x, self.h_out):
            x = hx.to(xcat.device, non_blocking=True)
            ho.copy_(ops.spmm(g, x, mode=ops.W_EDGE, edge_values=w), non_blocking=True)

    def verify(self):
        t, ops = self.torch, self.ops
        g, w, xcat, out, _ = self.groups[0]
        res = ops.spmm(g, t.ones_like(xcat), mode=ops.W_EDGE, edge_values=w)[:, 0]
        assert float((res - res.round()).abs().max()) < 1e-4, "RGCN self-check failed (sum of per-relation means of 1)"

    def cpu_sample(self, seconds_hint=15.0):
        g, w, xcat, out, _ = self.groups[0]
        return dict(indptr=g.indptr.cpu().numpy().astype("int64"), indices=g.indices.cpu().numpy(),
                    values=w.cpu().numpy(), x=xcat.cpu().numpy(), nnz=g.nnz, d=self.d, mask=0xFFFFFF,
                    sample="destination type 0: %d rows, %d edges (of %d), stitched mean aggregation" % (
                        g.n_rows, g.nnz, self.nnz))


class UniformWorkload:
    """Not one of the configurations: the SpMM of the headline (128 features, fp32 edge weights, int64 row pointers) on a
    UNIFORM random graph, 2^23 nodes and 2^27 sampled edges.  Every source row is referenced about 16 times from all
    over the row range, so the 126 MB L2 cannot keep a hot set (the feature matrix is 4.3 GB) and the algorithmic
    bytes ARE the DRAM bytes: this is the machine's random-row gather ceiling, the figure the R-MAT numbers (where
    the L2 serves the hub rows) should be read against."""
    name = "spmm_uniform_n8388608_e134217728_d128"

    def __init__(self, device, n=1 << 23, e=1 << 27, d=128):
        import torch
        from yitu_b200 import graphs, ops
        self.torch, self.ops, self.n, self.d = torch, ops, n, d
        src, dst = graphs.uniform_edges(9, n, n, e, device=device)
        self.indptr, self.indices = graphs.csr_by_destination(src, dst, n, n, ptr_dtype=torch.int64)
        del src, dst
        self.nnz = self.indices.numel()
        inv = 1.0 / graphs.in_degrees(self.indptr).clamp(min=1.0)
        self.values = torch.repeat_interleave(inv, self.indptr[1:] - self.indptr[:-1])
        self.g = ops.PreparedGraph(self.indptr, self.indices, n)
        self.g.plan()
        self.x = graphs.randn_features(1, n, d, device=device)
        self.out = torch.empty_like(self.x)
        self.units_per_step = self.nnz * d
        self.kernel_bytes = self.nnz * (4 * d + 8) + (n + 1) * 8 + 4 * n * d
        self.compulsory_bytes = self.nnz * 8 + (n + 1) * 8 + 2 * 4 * n * d
        self.traffic_key = "spmm_uniform_d128"
        self.dominant_kernel = spmm_kernel_name(self.nnz, n, d)
        self.launches_per_step = spmm_launches(self.nnz, n, d, bool(self.g.plan()))
        self.kernel_launches_per_step = 1

    def step(self, kernel_events=None):
        t, ops = self.torch, self.ops
        if kernel_events is not None:
            a, b = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            a.record()
        ops.spmm(self.g, self.x, mode=ops.W_EDGE, edge_values=self.values, out=self.out)
        if kernel_events is not None:
            b.record()
            kernel_events.append((a, b))

    def e2e_setup(self):
        t = self.torch
        self.h_x = self.x.cpu().pin_memory()
        self.h_out = t.empty(self.x.shape, dtype=t.float32).pin_memory()
        self.h2d = self.d2h = self.x.numel() * 4

    def e2e_step(self):
        ops = self.ops
        x = self.h_x.to(self.x.device, non_blocking=True)
        self.h_out.copy_(ops.spmm(self.g, x, mode=ops.W_EDGE, edge_values=self.values), non_blocking=True)

    def cpu_sample(self, seconds_hint=15.0):
        hi = self.n // 8
        ip = self.indptr[:hi + 1].cpu().numpy().astype("int64")
        e1 = int(ip[-1])
        return dict(indptr=ip, indices=self.indices[:e1].cpu().numpy(), values=self.values[:e1].cpu().numpy(),
                    x=self.x.cpu().numpy(), nnz=e1, d=self.d,
                    sample="rows [0,%d) of %d (%d of %d edges), forward SpMM, full feature matrix" % (hi, self.n, e1, self.nnz))

    def verify(self):
        t, ops = self.torch, self.ops
        out = ops.spmm(self.g, t.ones(self.n, 4, device=self.x.device), mode=ops.W_EDGE, edge_values=self.values)[:, 0]
        has = (self.indptr[1:] > self.indptr[:-1]).float()
        assert float((out - has).abs().max()) < 1e-5, "SpMM self-check failed (weights 1/in-degree of a row sum to one)"


def cpu_baseline(sample, repeats=5, min_seconds=10.0):
    """Times the CPU restatement (oracle/yitu_oracle.c, OpenMP over destination rows) on the sample."""
    from oracle import oracle as O
    cores = len(os.sched_getaffinity(0))
    O.build()
    cores = O.set_threads(cores)  # torchrun exports OMP_NUM_THREADS=1: ask for every core explicitly
    best, spent, done = None, 0.0, 0
    while done < repeats or (spent < min_seconds and done < 40):  # at least `repeats` passes and about 10 s of CPU work
        done += 1
        t0 = time.perf_counter()
        if sample.get("gat"):
            O.gat_forward(sample["indptr"], sample["indices"], sample["q"], sample["k"], sample["x"])
        else:
            O.spmm(sample["indptr"], sample["indices"], sample["x"], wmode=O.W_EDGE, values=sample["values"],
                   index_mask=sample.get("mask", 0))
        dt = time.perf_counter() - t0
        spent += dt
        best = dt if best is None else min(best, dt)
    out = {"value": sample["nnz"] * sample["d"] / best / 1e9, "unit": UNIT, "cores": cores, "kind": "port",
           "sample": sample["sample"] + "; best of %d passes (%.1f s of CPU work)" % (done, spent),
           "seconds": round(best, 3)}
    if not sample.get("gat") and not sample.get("mask"):
        out["scipy_single_thread"] = scipy_sanity(sample)
    return out


def scipy_sanity(sample, max_edges=4_000_000):
    """Single-thread scipy.sparse CSR x dense on the first rows of the sample holding at most max_edges edges — the
    library the reference builds its CSR with (YiTu_GNN/data/dataset.py:119-122); a sanity figure beside the port."""
    import numpy as np
    try:
        import scipy.sparse as sp
    except ImportError:
        return None
    ip = np.asarray(sample["indptr"], dtype=np.int64)
    rows = int(np.searchsorted(ip, max_edges, side="right")) - 1
    rows = max(1, min(rows, ip.shape[0] - 1))
    e = int(ip[rows])
    x = np.asarray(sample["x"], dtype=np.float32)
    a = sp.csr_matrix((np.asarray(sample["values"][:e], dtype=np.float32), np.asarray(sample["indices"][:e]), ip[:rows + 1]),
                      shape=(rows, x.shape[0]))
    t0 = time.perf_counter()
    a @ x
    dt = time.perf_counter() - t0
    return {"value": e * sample["d"] / dt / 1e9, "unit": UNIT, "cores": 1,
            "sample": "rows [0,%d) (%d edges)" % (rows, e), "seconds": round(dt, 3)}


WORKLOADS = {"spmm": SpmmWorkload, "gat": GatWorkload, "rgcn": RgcnWorkload, "uniform": UniformWorkload}


def cpu_baseline_partitioned(dev, n, e, d, repeats=5, min_seconds=10.0):
    """CPU baseline of the partitioned workload: the rows of partition 8 of 16 (1/16 of the edges) of the same graph,
    whole feature matrix, OpenMP restatement on all host cores."""
    import torch
    from yitu_b200 import graphs
    indptr, indices, values = graphs.spmm_partitioned(device=dev, n=n, e=e)
    nnz = indices.numel()
    lo, hi = torch.searchsorted(indptr, torch.tensor([(8 * nnz + 15) // 16, (9 * nnz + 15) // 16], device=dev)).tolist()
    e0, e1 = int(indptr[lo]), int(indptr[hi])
    sample = dict(indptr=(indptr[lo:hi + 1] - e0).cpu().numpy(), indices=indices[e0:e1].cpu().numpy(),
                  values=values[e0:e1].cpu().numpy(), nnz=e1 - e0, d=d,
                  sample="partition 8 of 16 (%d rows, %d of %d edges), forward SpMM, full feature matrix" % (
                      hi - lo, e1 - e0, nnz))
    del indptr, indices, values
    sample["x"] = graphs.randn_features(1, n, d, device=dev).cpu().numpy()
    torch.cuda.empty_cache()
    out = cpu_baseline(sample, repeats=repeats, min_seconds=min_seconds)
    out.pop("scipy_single_thread", None)
    return out


def _measure(wl, steps=5, warmup=3):
    """(ms per step, mean ms of the dominant kernel's launches) by CUDA events, after `warmup` untimed steps."""
    import torch
    wl.verify()
    for _ in range(warmup):
        wl.step()
    torch.cuda.synchronize()
    events = []
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        wl.step(events)
    b.record()
    torch.cuda.synchronize()
    kms = [x.elapsed_time(y) for x, y in events]
    return a.elapsed_time(b) / steps, sum(kms) / len(kms), kms


def sub_record_spmm(dev, steps=5):
    """configs[1] beside the headline: forward + transposed SpMM, D=256, with the roofline of its kernel."""
    wl = SpmmWorkload(dev)
    ms, k_ms, _ = _measure(wl, steps)
    return {"workload": wl.name, "nnz": wl.nnz, "ms_per_step": ms, "value": wl.units_per_step / (ms * 1e-3) / 1e9,
            "unit": UNIT, "roofline": roofline(wl.dominant_kernel, wl.kernel_bytes, k_ms, wl.traffic_key, wl.compulsory_bytes)}


def sub_record_uniform(dev, steps=5):
    """The headline's kernel where the L2 cannot help: the random-row gather ceiling of the machine (see UniformWorkload)."""
    wl = UniformWorkload(dev)
    ms, k_ms, _ = _measure(wl, steps)
    return {"workload": wl.name, "nnz": wl.nnz, "ms_per_step": ms, "value": wl.units_per_step / (ms * 1e-3) / 1e9,
            "unit": UNIT, "note": "uniform random graph: no hot rows, algorithmic bytes = DRAM bytes",
            "roofline": roofline(wl.dominant_kernel, wl.kernel_bytes, k_ms, wl.traffic_key, wl.compulsory_bytes)}


def sub_record_gat(dev, steps=5):
    """The other half of the headline metric, "GAT layer ms": fused GAT layer core on the uniform 8x32 graph
    (configs[2]), forward, backward and both, with the roofline of the forward kernel."""
    wl = GatWorkload(dev)
    total, fwd, _ = _measure(wl, steps)
    return {"workload": wl.name, "nnz": wl.nnz, "fwd_ms": fwd, "bwd_ms": total - fwd, "fwd_bwd_ms": total,
            "value": wl.units_per_step / (total * 1e-3) / 1e9, "unit": UNIT,
            "roofline": roofline(wl.dominant_kernel, wl.kernel_bytes, fwd, wl.traffic_key, wl.compulsory_bytes)}


def sub_record_rgcn(dev, steps=5):
    """configs[3]: hetero RGCN aggregation, one stitched pass per destination type (4 launches per step)."""
    wl = RgcnWorkload(dev)
    ms, k_ms, kms = _measure(wl, steps)
    per_type = [sum(kms[i::len(wl.groups)]) / steps for i in range(len(wl.groups))]
    return {"workload": wl.name, "nnz": wl.nnz, "ms_per_step": ms, "ms_per_destination_type": per_type,
            "value": wl.units_per_step / (ms * 1e-3) / 1e9, "unit": UNIT,
            "roofline": roofline(wl.dominant_kernel, wl.kernel_bytes, k_ms, wl.traffic_key)}


def run_reference_gpu_comparison(args):
    """Times the reference's own CUDA kernels (compiled unmodified for sm_100a into oracle/_ref by
    `make -C oracle ref_gpu ref_gpu_ccsrc`) beside this library on graphs inside the reference's limits:
    fewer than 2^24 edges for the ccsrc neighbour-group table (float32 storage) and at most 65535 destination
    rows per launch for the YiTu_H kernels.  Prints one JSON line; not the headline benchmark."""
    import glob
    import importlib
    import torch
    from yitu_b200 import YiTu_GNN_kernel as K, graph_ext, graphs
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    if not glob.glob(os.path.join(ref_dir, "graph_ext_ref*.so")) or not glob.glob(os.path.join(ref_dir, "yitu_gnn_kernel_ref*.so")):
        print(json.dumps({"workload": "reference_gpu_comparison", "unavailable": "oracle/_ref builds are absent"}))
        return
    sys.path.insert(0, ref_dir)
    ref_h = importlib.import_module("graph_ext_ref")
    ref_c = importlib.import_module("yitu_gnn_kernel_ref")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)

    def timed(fn, reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    out = {"workload": "reference_gpu_comparison", "unit": "ms", "rows": []}
    # ccsrc SAG (unweighted neighbour sum), R-MAT 2^18 nodes, 2^23 sampled edges, 64 and 256 features
    # (self-loops keep the last node non-empty: with an empty last node the reference's group table ends in 0 and
    # its kernel adds uninitialised shared memory to one output row)
    n = 1 << 18
    src, dst = graphs.rmat_edges(1, n, n, 1 << 23, device=dev)
    indptr, indices = graphs.csr_by_destination(src, dst, n, n, self_loops=True)
    pp, p2n = K.build_part(32, indptr.cpu())
    graph = (indptr, indices, torch.ones(n, device=dev), pp.int().to(dev), p2n.int().to(dev), 32, 32, 2)
    for d in (64, 256):
        x = graphs.randn_features(1, n, d, device=dev)
        t_ref = timed(lambda: ref_c.SAG(x, *graph), 5)
        t_new = timed(lambda: K.SAG(x, *graph), 20)
        err = float((ref_c.SAG(x, *graph) - K.SAG(x, *graph)).abs().max())
        out["rows"].append({"op": "YiTu_GNN_kernel.SAG", "n": n, "nnz": indices.numel(), "d": d, "reference_ms": t_ref,
                            "this_ms": t_new, "speedup": t_ref / t_new, "max_abs_diff": err})
    # graph_ext sddmm_forward + spmm_forward (GAT attention + aggregation), 65535 rows, 8 heads x 32
    n = 65535
    src, dst = graphs.uniform_edges(2, n, n, n * 32, device=dev)
    indptr, indices = graphs.csr_by_destination(src, dst, n, n, self_loops=True)
    H, F = 8, 32
    xh = graphs.randn_features(3, n, H * F, device=dev).view(n, H, F)
    q = graphs.uniform_values(4, (1, n, H), -1, 1, device=dev)
    k = graphs.uniform_values(5, (n, H), -1, 1, device=dev)
    t_ref = timed(lambda: ref_h.spmm_forward(ref_h.sddmm_forward(indptr, indices, q, k), indptr, indices, xh), 5)
    t_two = timed(lambda: graph_ext.spmm_forward(graph_ext.sddmm_forward(indptr, indices, q, k), indptr, indices, xh), 20)
    t_fused = timed(lambda: graph_ext.gat_forward(indptr, indices, q[0], k, xh), 20)
    err = float((ref_h.spmm_forward(ref_h.sddmm_forward(indptr, indices, q, k), indptr, indices, xh) -
                 graph_ext.gat_forward(indptr, indices, q[0], k, xh)[0]).abs().max())
    out["rows"].append({"op": "graph_ext.sddmm_forward+spmm_forward", "n": n, "nnz": indices.numel(), "d": H * F,
                        "reference_ms": t_ref, "this_ms_two_operators": t_two, "this_ms_fused": t_fused,
                        "speedup": t_ref / t_fused, "max_abs_diff": err})
    # the backward of the same pair: the reference scatters with atomicAdd (spmm_cuda.cu:24-42, sddmm_cuda.cu:36-67)
    attn = graph_ext.sddmm_forward(indptr, indices, q, k)
    gout = graphs.randn_features(6, n, H * F, device=dev).view(n, H, F)

    def ref_bwd():
        ga, gx = ref_h.spmm_backward(attn, indptr, indices, xh, gout)
        return ref_h.sddmm_backward(indptr, indices, q, k, attn, ga) + [gx]

    def two_bwd():
        ga, gx = graph_ext.spmm_backward(attn, indptr, indices, xh, gout)
        return graph_ext.sddmm_backward(indptr, indices, q, k, attn, ga) + [gx]

    fo, fmax, fsum = graph_ext.gat_forward(indptr, indices, q[0], k, xh)
    t_ref = timed(ref_bwd, 5)
    t_two = timed(two_bwd, 20)
    t_fused = timed(lambda: graph_ext.gat_backward(indptr, indices, q[0], k, xh, fo, fmax, fsum, gout), 20)
    r, o = ref_bwd(), graph_ext.gat_backward(indptr, indices, q[0], k, xh, fo, fmax, fsum, gout)
    err = max(float((r[0][0] - o[0]).abs().max()), float((r[1] - o[1]).abs().max()), float((r[2] - o[2]).abs().max()))
    out["rows"].append({"op": "graph_ext.spmm_backward+sddmm_backward", "n": n, "nnz": indices.numel(), "d": H * F,
                        "reference_ms": t_ref, "this_ms_two_operators": t_two, "this_ms_fused": t_fused,
                        "speedup": t_ref / t_fused, "max_abs_diff": err})
    print(json.dumps(out))


def run_layer_fusion(args):
    """Layer-level effect of the fused epilogues on the benchmark graphs: the GCN layer tail (norm * aggregate, ReLU)
    and the GAT layer tail (mean over heads, ELU), forward and forward+backward, fused into the aggregation kernels
    against the same kernels followed by separate element-wise torch operators (the reference's formulation).
    Prints one JSON line; not the headline benchmark."""
    import torch
    from yitu_b200 import graphs, ops
    from yitu_b200.nn.layers import aggregate
    from yitu_b200.xgnn_h import Block, sparse
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    reps = max(3, args.steps)

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    out = {"workload": "layer_epilogue_fusion", "unit": "ms", "reps": reps, "rows": []}
    shift = args.scale
    # GCN layer tail on the D=256 R-MAT graph: relu(norm * (A h))
    n, e, d = (1 << 21) >> shift, (1 << 26) >> shift, 256
    indptr, indices, _ = graphs.spmm_rmat(device=dev, n=n, e=e)
    blk = Block([n, n], [indptr, indices])
    norm = ops.degree_norm(indptr, ops.DEG_INV)
    h = graphs.randn_features(1, n, d, device=dev).requires_grad_()
    gy = graphs.randn_features(2, n, d, device=dev)

    def gcn(fused, backward):
        if fused:
            y = aggregate(blk, h, row_scale=norm, activation="relu")
        else:
            y = torch.relu(norm.view(-1, 1) * aggregate(blk, h))
        if backward:
            y.backward(gy)
            h.grad = None

    err = float((aggregate(blk, h, row_scale=norm, activation="relu") -
                 torch.relu(norm.view(-1, 1) * aggregate(blk, h))).abs().max())
    row = {"layer": "GCN tail relu(norm*A h)", "n": n, "nnz": indices.numel(), "d": d, "max_abs_diff": err}
    for backward in (False, True):
        key = "fwd_bwd" if backward else "fwd"
        row["unfused_%s_ms" % key] = timed(lambda: gcn(False, backward))
        row["fused_%s_ms" % key] = timed(lambda: gcn(True, backward))
    out["rows"].append(row)
    del blk, h, gy, indptr, indices, norm
    torch.cuda.empty_cache()
    # GAT layer tail on the 8x32 uniform graph: elu(mean_h(softmax-weighted aggregation))
    n, e, H, F = (1 << 20) >> shift, (1 << 25) >> shift, 8, 32
    indptr, indices = graphs.gat_uniform(device=dev, n=n, e=e)
    blk = Block([n, n], [indptr, indices])
    x = graphs.randn_features(1, n, H * F, device=dev).view(n, H, F).requires_grad_()
    q = graphs.uniform_values(5, (n, H), -1, 1, device=dev).requires_grad_()
    k = graphs.uniform_values(6, (n, H), -1, 1, device=dev).requires_grad_()
    gy = graphs.randn_features(2, n, F, device=dev)

    def gat(fused, backward):
        if fused:
            y = sparse.fused_gat(blk, q, k, x, head_mean=True, activation="elu")
        else:
            y = torch.nn.functional.elu(torch.mean(sparse.fused_gat(blk, q, k, x), dim=1))
        if backward:
            y.backward(gy)
            x.grad = q.grad = k.grad = None

    err = float((sparse.fused_gat(blk, q, k, x, head_mean=True, activation="elu") -
                 torch.nn.functional.elu(torch.mean(sparse.fused_gat(blk, q, k, x), dim=1))).abs().max())
    row = {"layer": "GAT tail elu(mean_heads(attention aggregation))", "n": n, "nnz": indices.numel(), "heads": H,
           "feats": F, "max_abs_diff": err}
    for backward in (False, True):
        key = "fwd_bwd" if backward else "fwd"
        row["unfused_%s_ms" % key] = timed(lambda: gat(False, backward))
        row["fused_%s_ms" % key] = timed(lambda: gat(True, backward))
    out["rows"].append(row)
    del blk, x, q, k, gy, indptr, indices
    torch.cuda.empty_cache()
    # hetero RGCN layer for the destination type with the most relations: per-relation linear maps + one stitched pass;
    # "unfused" concatenates the per-relation GEMM results first, as a list-of-tensors formulation does
    if not shift:
        from yitu_b200.nn.layers import StitchedRGCNConv, _AggregateFunction
        sizes = graphs.HETERO_TYPES
        rels = graphs.hetero_rgcn(device=dev)
        by_dst = {}
        for i, r in enumerate(rels):
            by_dst.setdefault(r[1], []).append(i)
        dt, ids = max(by_dst.items(), key=lambda kv: len(kv[1]))
        relations = [("r%d" % i, Block([sizes[dt], sizes[rels[i][0]]], [rels[i][2], rels[i][3]])) for i in ids]
        layer = StitchedRGCNConv(relations, 64, 64, reduce="sum").to(dev)
        xs = {"r%d" % i: graphs.randn_features(20 + i, sizes[rels[i][0]], 64, device=dev).requires_grad_() for i in ids}
        gy = graphs.randn_features(3, sizes[dt], 64, device=dev)

        def rgcn(fused, backward):
            if fused:
                y = layer(xs)
            else:
                h = torch.cat([layer.fcs[name](xs[name]) for name in layer.names])
                y = _AggregateFunction.apply(h, layer._graph(h.device, h.size(0)), layer._weights)
            if backward:
                y.backward(gy)
                for v in xs.values():
                    v.grad = None
                layer.zero_grad()

        row = {"layer": "hetero RGCN, %d relations into one destination type (GEMMs + stitched mean aggregation)" % len(ids),
               "n_dst": sizes[dt], "nnz": sum(int(rels[i][3].numel()) for i in ids), "d": 64}
        for backward in (False, True):
            key = "fwd_bwd" if backward else "fwd"
            row["unfused_%s_ms" % key] = timed(lambda: rgcn(False, backward))
            row["fused_%s_ms" % key] = timed(lambda: rgcn(True, backward))
        out["rows"].append(row)
    print(json.dumps(out))


def run_reorder(args):
    """Locality reordering (yitu_b200.rabbit) measured by what it is for: the D=256 aggregation before and after the
    renumbering, on a graph with planted communities behind shuffled ids and on the R-MAT benchmark graph, plus the
    time of the reordering itself.  Prints one JSON line; not the headline benchmark."""
    import torch
    from yitu_b200 import graphs, ops, rabbit
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    reps = max(3, args.steps)
    n, e, d = (1 << 21) >> args.scale, (1 << 26) >> args.scale, 256

    def timed(fn, reps=reps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    def spmm_ms(ei):
        ip, ix = ops.coo_to_csr(ei[0].contiguous(), ei[1].contiguous(), n, n, self_loops=True)
        g = ops.PreparedGraph(ip, ix, n)
        g.plan()
        x = graphs.randn_features(1, n, d, device=dev)
        ms = timed(lambda: ops.spmm(g, x))
        return ms, ix.numel()

    out = {"workload": "locality_reordering", "n": n, "d": d, "unit": "ms", "rows": []}
    cases = (("planted communities of 1024 nodes, 90% of edges inside, ids shuffled",
              lambda: graphs.planted_community_edges(7, n, 1024, e, 0.9, device=dev)),
             ("R-MAT (0.57,0.19,0.19,0.05)", lambda: graphs.rmat_edges(1, n, n, e, device=dev)))
    for name, make in cases:
        src, dst = make()
        ei = torch.stack([src, dst]).to(torch.int32)
        del src, dst
        before_ms, nnz = spmm_ms(ei)
        span_before = rabbit.avg_edge_span(ei)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        new_id, levels, top = rabbit.reorder_ids(ei, n)
        torch.cuda.synchronize()
        reorder_s = time.perf_counter() - t0
        ei2 = rabbit.relabel(ei, new_id)
        del ei
        after_ms, _ = spmm_ms(ei2)
        out["rows"].append({"graph": name, "nnz": nnz, "levels": levels, "top_communities": top,
                            "reorder_seconds": reorder_s, "avg_edge_span_before": span_before,
                            "avg_edge_span_after": rabbit.avg_edge_span(ei2),
                            "decider_says_reorder": bool(span_before ** 0.5 > n ** 0.5 / 100),
                            "spmm_before_ms": before_ms, "spmm_after_ms": after_ms, "speedup": before_ms / after_ms})
        del ei2, new_id
        torch.cuda.empty_cache()
    print(json.dumps(out))


def run_single(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    kw = {}
    if args.scale and args.workload in ("spmm", "gat", "uniform"):
        base_n, base_e = {"spmm": (1 << 21, 1 << 26), "gat": (1 << 20, 1 << 25), "uniform": (1 << 23, 1 << 27)}[args.workload]
        kw = dict(n=base_n >> args.scale, e=base_e >> args.scale)
    wl = WORKLOADS[args.workload](dev, **kw)

    if args.impl == "reference":
        base = cpu_baseline(wl.cpu_sample(), repeats=max(1, args.steps + args.warmup))
        line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["seconds"] * 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": wl.name, "note": "CPU restatement of the reference kernels; the reference has "
                           "no CPU implementation of this path"},
                "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    wl.verify()
    for _ in range(max(3, args.warmup)):
        wl.step()
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    time.sleep(0.3)
    kernel_events = []
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.steps):
        wl.step(kernel_events)
    stop.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms_total = start.elapsed_time(stop)
    ms_step = ms_total / args.steps
    value = wl.units_per_step / (ms_step * 1e-3) / 1e9
    kms = [a.elapsed_time(b) for a, b in kernel_events]
    k_avg_ms = sum(kms) / len(kms)

    # end to end: pinned host features in, results back to pinned host memory, every step
    e2e = None
    if not args.no_e2e:
        wl.e2e_setup()
        for _ in range(2):
            wl.e2e_step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e_steps = max(2, min(args.steps, 5))
        e0.record()
        for _ in range(e_steps):
            wl.e2e_step()
        e1.record()
        torch.cuda.synchronize()
        e2e_ms = e0.elapsed_time(e1) / e_steps
        e2e = {"value": wl.units_per_step / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h, "ms_per_step": e2e_ms, "mode": "serial"}
        if hasattr(wl, "e2e_run"):
            # the same bytes per step with copy-in / compute / copy-out of neighbouring steps overlapped
            piped_ms = wl.e2e_run(max(8, e_steps))
            e2e["serial_value"] = e2e["value"]
            if piped_ms < e2e_ms:
                e2e.update(value=wl.units_per_step / (piped_ms * 1e-3) / 1e9, ms_per_step=piped_ms,
                           mode="pipelined (double-buffered copy-in / compute / copy-out streams)")

    base = None if args.no_cpu_baseline else cpu_baseline(wl.cpu_sample())
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": wl.name, "nnz": wl.nnz, "l2": "inputs_larger_than_l2",
                       "edge_feats_per_step": wl.units_per_step},
            "roofline": roofline(wl.dominant_kernel, wl.kernel_bytes, k_avg_ms, None if args.scale else wl.traffic_key,
                                 getattr(wl, "compulsory_bytes", None)),
            "cpu_baseline": base,
            "e2e": e2e,
            "gpu_launches": wl.launches_per_step * args.steps, "clocks": clocks}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=["spmm", "gat", "rgcn", "uniform", "partitioned", "refgpu", "layers", "reorder"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--scale", type=int, default=0, help="shrink the graph by 2^SCALE (profiling / development)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling)")
    ap.add_argument("--no-sub-records", action="store_true",
                    help="default workload at N=1: skip the spmm_c2 / gat_layer / rgcn_layer sub-records")
    ap.add_argument("--halo", default="push,peer",
                    help="partitioned, N>1: exchange modes to try for 3 steps each, the fastest is timed "
                         "(push | push1..push4 | pushnp | peer | allgather)")
    ap.add_argument("--verbose-trials", action="store_true",
                    help="partitioned: keep schedule and per-rank timeline of the exchange modes that lost the trial")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="partitioned, 1 GPU: aggregate only shard --shard of a SHARD_OF-way split (the kernel one rank of a "
                         "multi-GPU run executes, without the exchange: for single-GPU profiling)")
    ap.add_argument("--shard", type=int, default=0)
    ap.add_argument("--row-cost", type=int, default=0,
                    help="partitioned: balance edges + ROW_COST * rows instead of edges alone (not the prescribed split)")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload is None:
        args.workload = "partitioned"  # one series at every N: the same graph on 1, 2, 4 and 8 GPUs
    if args.workload == "partitioned":
        import bench_partitioned
        bench_partitioned.run(args)
        return
    if int(os.environ.get("RANK", "0")) != 0:
        return  # single-GPU workloads: extra ranks have nothing to do
    if args.workload == "refgpu":
        run_reference_gpu_comparison(args)
        return
    if args.workload == "layers":
        run_layer_fusion(args)
        return
    if args.workload == "reorder":
        run_reorder(args)
        return
    run_single(args)


if __name__ == "__main__":
    main()
