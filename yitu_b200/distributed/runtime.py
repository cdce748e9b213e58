"""Execution of the row-partitioned SpMM on one rank (CUDA).

Per step:  [handshake: features of every rank are in place]  ->  fetch the halo rows this rank needs from its
peers' shards (peer loads over NVLink through CUDA-IPC mappings, each needed row crosses the link once)  ->
SpMM over [own rows | halo rows].  With overlap=True the shard's edges are split by source: the own-source part
runs on the compute stream while the halo is fetched on a second stream; the halo-source part follows and
accumulates.  mode="allgather" replaces the fetch by one NCCL all-gather of padded shards.

No collective carries feature data in the peer mode; no multicast load is used anywhere.
"""
import ctypes as C

import torch
import torch.distributed as dist

from .. import ops
from .._lib import check, lib
from .partition import HaloPlan, allgather_columns, split_local_halo


class SharedBuffer:
    """Device memory that other processes on the same node can map (yitu_shared_alloc / yitu_shared_open)."""

    def __init__(self, n_floats, device):
        self.device = torch.device(device)
        self.n_floats = int(n_floats)
        self.ptr = C.c_void_p()
        self.handle = (C.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            check(lib().yitu_shared_alloc(max(self.n_floats, 1) * 4, C.byref(self.ptr), self.handle))
        self.__cuda_array_interface__ = {"shape": (self.n_floats,), "typestr": "<f4", "data": (self.ptr.value, False),
                                         "version": 2}
        self._opened = []

    def tensor(self):
        return torch.as_tensor(self, device=self.device)

    def handle_bytes(self):
        return bytes(self.handle)

    def open_peer(self, handle_bytes):
        buf = (C.c_ubyte * 64).from_buffer_copy(handle_bytes)
        p = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib().yitu_shared_open(buf, C.byref(p)))
        self._opened.append(p)
        return p.value

    def close(self):
        with torch.cuda.device(self.device):
            for p in self._opened:
                lib().yitu_shared_close(p)
            self._opened = []
            if self.ptr:
                lib().yitu_shared_free(self.ptr)
                self.ptr = C.c_void_p()


class PartitionedSpmm:
    def __init__(self, shard, d, device, group=None, mode="peer", overlap=True, weight_mode=ops.W_EDGE, row_blocks=1):
        self.shard, self.d, self.device, self.group = shard, int(d), torch.device(device), group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and mode != "local") else 1
        self.rank = shard.rank
        self.mode = mode if self.world > 1 else "local"  # "local": the shard is the whole graph, no exchange
        self.row_blocks = int(row_blocks) if self.mode == "peer" else 1
        self.overlap = overlap and self.mode == "peer" and self.row_blocks <= 1
        self.weight_mode = weight_mode
        n_local = shard.n_local
        self.out = torch.empty(n_local, d, dtype=torch.float32, device=self.device)
        self._token = torch.zeros(1, device=self.device)
        if self.mode == "allgather":
            sizes = [shard.bounds[p + 1] - shard.bounds[p] for p in range(self.world)]
            self.max_rows = max(sizes)
            self.rep = torch.empty(self.world * self.max_rows, d, dtype=torch.float32, device=self.device)
            self.x_local = self.rep[self.rank * self.max_rows: self.rank * self.max_rows + n_local]
            self._slot = self.rep[self.rank * self.max_rows: (self.rank + 1) * self.max_rows]
            cols = allgather_columns(shard.indices, shard.bounds, self.max_rows)
            self.graph = ops.PreparedGraph(shard.indptr, cols, self.rep.size(0))
            self.plan = None
            self.halo_bytes = (self.world - 1) * self.max_rows * d * 4
            return
        row_bounds = None
        if self.row_blocks > 1:
            # edge-balanced row blocks inside the shard: block b is aggregated while the halo rows that only later
            # blocks need are still in flight
            probe = ops.PreparedGraph(shard.indptr, torch.empty(0, dtype=torch.int32, device=self.device), 0)
            row_bounds = ops.partition_rows(probe, self.row_blocks).tolist()
        self.plan = HaloPlan(shard, row_bounds)
        n_halo = self.plan.n_halo
        self.shared = SharedBuffer((n_local + n_halo) * d, self.device)
        self.xbuf = self.shared.tensor().view(n_local + n_halo, d)
        self.x_local, self.x_halo = self.xbuf[:n_local], self.xbuf[n_local:]
        self.halo_bytes = n_halo * d * 4
        self.graph = ops.PreparedGraph(shard.indptr, self.plan.local_indices, n_local + n_halo)
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, self.shared.handle_bytes(), group=group)
            ptrs = [self.shared.ptr.value if p == self.rank else self.shared.open_peer(handles[p])
                    for p in range(self.world)]
            self._ptrs = (C.c_void_p * self.world)(*ptrs)
            self._bounds = (C.c_int64 * (self.world + 1))(*shard.bounds)
            self.side = torch.cuda.Stream(device=self.device, priority=-1)
            if self.plan.row_bounds is not None:
                self.blocks = []
                rb = self.plan.row_bounds
                ip_all = shard.indptr
                for b in range(len(rb) - 1):
                    e0, e1 = int(ip_all[rb[b]]), int(ip_all[rb[b + 1]])
                    g_b = ops.PreparedGraph((ip_all[rb[b]:rb[b + 1] + 1] - e0).contiguous(),
                                            self.plan.local_indices[e0:e1].contiguous(), n_local + n_halo)
                    v_b = None if shard.values is None else shard.values[e0:e1].contiguous()
                    self.blocks.append((g_b, v_b, self.out[rb[b]:rb[b + 1]], torch.cuda.Event()))
            else:
                self.row_blocks = 1
            if self.overlap:
                (ipo, ixo, vo), (iph, ixh, vh) = split_local_halo(shard, self.plan)
                self.g_own = ops.PreparedGraph(ipo, ixo, n_local)
                self.g_halo = ops.PreparedGraph(iph, ixh, n_halo)
                self.v_own, self.v_halo = vo, vh

    # ------------------------------------------------------------------------------------------
    def handshake(self):
        """Stream-ordered all-reduce of one float: nobody reads a peer's shard before every rank's earlier work
        (the writes of its features) has been enqueued and finished."""
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)

    def _mark(self, events, tag):
        if events is None:
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(self.device))
        return ev

    def fetch_halo(self, events=None):
        if self.mode != "peer" or self.plan.n_halo == 0:
            return
        a = self._mark(events, "fetch")
        self._fetch_halo()
        if events is not None:
            events.append(("fetch", a, self._mark(events, "fetch")))

    def _fetch_halo(self, first=0, last=None):
        """Gather halo rows [first, last) of the plan's list into their slots of the halo buffer."""
        last = self.plan.n_halo if last is None else last
        if last <= first:
            return
        st = torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            check(lib().yitu_halo_gather_f32(self.world, self._ptrs, self._bounds,
                                             C.c_void_p(self.plan.halo_ids.data_ptr() + 4 * first), last - first, self.d,
                                             C.c_void_p(self.x_halo.data_ptr() + 4 * self.d * first),
                                             C.c_void_p(st.cuda_stream)))

    def _spmm(self, g, x, vals, accumulate=False, events=None):
        a = self._mark(events, "spmm")
        out = ops.spmm(g, x, mode=self.weight_mode if vals is not None else ops.W_NONE, edge_values=vals,
                       out=self.out, accumulate=accumulate)
        if events is not None:
            events.append(("spmm", a, self._mark(events, "spmm")))
        return out

    def step(self, events=None, fence=False):
        """One aggregation over this rank's rows; returns the [n_local, d] output (reused between steps).
        `events`, if a list, receives (tag, start, end) CUDA-event triples around every SpMM and halo fetch.
        fence=True adds a second handshake once this rank's halo has arrived, so that no rank's later work (which may
        overwrite its feature shard, as a training step does) starts before every peer has finished reading it."""
        sh = self.shard
        if self.mode == "local":
            return self._spmm(self.graph, self.x_local, sh.values, events=events)
        self.handshake()
        if self.mode == "allgather":
            dist.all_gather_into_tensor(self.rep, self._slot, group=self.group)
            return self._spmm(self.graph, self.rep, sh.values, events=events)
        if fence:
            self.fetch_halo(events)
            self.handshake()
            return self._spmm(self.graph, self.xbuf, sh.values, events=events)
        if self.row_blocks > 1:
            main = torch.cuda.current_stream(self.device)
            self.side.wait_stream(main)
            off = self.plan.chunk_offsets
            with torch.cuda.stream(self.side):
                for b, (_, _, _, ready) in enumerate(self.blocks):
                    a = self._mark(events, "fetch")
                    self._fetch_halo(off[b], off[b + 1])
                    if events is not None:
                        events.append(("fetch", a, self._mark(events, "fetch")))
                    ready.record(self.side)
            for g_b, v_b, out_b, ready in self.blocks:
                main.wait_event(ready)
                a = self._mark(events, "spmm")
                ops.spmm(g_b, self.xbuf, mode=self.weight_mode if v_b is not None else ops.W_NONE, edge_values=v_b,
                         out=out_b)
                if events is not None:
                    events.append(("spmm", a, self._mark(events, "spmm")))
            return self.out
        if not self.overlap:
            self.fetch_halo(events)
            return self._spmm(self.graph, self.xbuf, sh.values, events=events)
        main = torch.cuda.current_stream(self.device)
        self.side.wait_stream(main)
        with torch.cuda.stream(self.side):
            self.fetch_halo(events)
        self._spmm(self.g_own, self.x_local, self.v_own, events=events)
        main.wait_stream(self.side)
        return self._spmm(self.g_halo, self.x_halo, self.v_halo, accumulate=True, events=events)

    def close(self):
        if getattr(self, "shared", None) is not None:
            self.shared.close()


class _PartitionedAggregateFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, owner):
        ctx.owner = owner
        owner.fwd.x_local.copy_(x_local)
        return owner.fwd.step(fence=True).clone()

    @staticmethod
    def backward(ctx, grad_out):
        owner = ctx.owner
        owner.bwd.x_local.copy_(grad_out)
        return owner.bwd.step(fence=True).clone(), None


class PartitionedAggregate:
    """Differentiable y = A x over a row-partitioned square graph: rank p holds rows [bounds[p], bounds[p+1]) of x and
    of y.  Forward runs the partitioned SpMM over this rank's rows of A; backward runs it over the same row range of
    A^T (pull-style, no atomics, no reduction across ranks), fetching the halo rows of the upstream gradient from the
    peers' shards.  The reference's multi-GPU layers reduce partial results across ranks instead
    (YiTu_GNN/distributed/communication.py:230-264).

    Built from the whole graph on every rank (indptr / indices / values are the global CSR, as in the reference's
    partitioning step, which also starts from the full graph)."""

    def __init__(self, indptr, indices, values, d, device, group=None, bounds=None, mode="peer"):
        from .partition import RowShard, partition_bounds
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        n = indptr.numel() - 1
        self.bounds = list(bounds) if bounds is not None else partition_bounds(indptr, world)
        self.row_begin, self.row_end = self.bounds[rank], self.bounds[rank + 1]
        whole = ops.PreparedGraph(indptr, indices, n)
        t_indptr, t_rows, t_perm = whole.transpose()
        t_values = None if values is None else values[t_perm.long()]
        wm = ops.W_EDGE if values is not None else ops.W_NONE
        self.fwd = PartitionedSpmm(RowShard(indptr, indices, values, self.bounds, rank), d, device, group, mode,
                                   overlap=False, weight_mode=wm)
        self.bwd = PartitionedSpmm(RowShard(t_indptr, t_rows, t_values, self.bounds, rank), d, device, group, mode,
                                   overlap=False, weight_mode=wm)

    def __call__(self, x_local):
        return _PartitionedAggregateFunction.apply(x_local, self)

    def close(self):
        self.fwd.close()
        self.bwd.close()
