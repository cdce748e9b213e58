"""Execution of the row-partitioned SpMM on one rank (CUDA).  Every rank keeps [own rows | halo rows] of the
feature matrix in one buffer that its peers can map (CUDA IPC); three ways of filling the halo part:

  mode="push"       the OWNER of a row writes it into the halo buffers of the ranks that need it (peer stores
                    over NVLink, each needed row crosses once), starting at the first moment of the step.  A rank
                    aggregates in passes (PushSchedule): the edges whose sources have arrived first, then, into the
                    same output, those of the owners that deliver later, so most of the aggregation runs while the
                    slowest owner is still sending.  Deliveries are announced by 64-bit flags that
                    the owner stores into the reader's memory after its push; the reader's stream waits for the
                    flags of the owners a pass needs (bounded wait), so no collective runs inside a step.
  mode="peer"       the READER fetches the rows with peer loads, then aggregates: two serial steps.
  mode="allgather"  one NCCL all-gather of shards padded to the largest, then the aggregation.

No collective carries feature data in the push and peer modes (NCCL moves one float per synchronisation point);
no multicast load is used anywhere.
"""
import ctypes as C
import os

import torch
import torch.distributed as dist

from .. import ops
from .._lib import check, lib
from ..ops import _ptr
from .partition import (HaloPlan, PushSchedule, allgather_columns, exchange_need_lists, owner_edge_counts,
                        source_passes)


class SharedBuffer:
    """Device memory that other processes on the same node can map (yitu_shared_alloc / yitu_shared_open)."""

    FLAG_BYTES = 256  # 32 delivery flags of 64 bits behind the floats: [0..15] "all rows", [16..31] "priority rows"

    @staticmethod
    def flags_offset(n_floats):
        """Byte offset of the flag block in a buffer of n_floats floats (256-byte aligned)."""
        return (max(int(n_floats), 1) * 4 + 255) // 256 * 256

    def __init__(self, n_floats, device):
        self.device = torch.device(device)
        self.n_floats = int(n_floats)
        self.ptr = C.c_void_p()
        self.handle = (C.c_ubyte * 64)()
        self.flags_off = self.flags_offset(self.n_floats)
        with torch.cuda.device(self.device):
            check(lib().yitu_shared_alloc(self.flags_off + self.FLAG_BYTES, C.byref(self.ptr), self.handle))
            self.flags_tensor().zero_()
        self.__cuda_array_interface__ = {"shape": (self.n_floats,), "typestr": "<f4", "data": (self.ptr.value, False),
                                         "version": 2}
        self._opened = []

    def tensor(self):
        return torch.as_tensor(self, device=self.device)

    def flags_tensor(self):
        """The 32 delivery flags as an int64 tensor (a view of the same allocation)."""
        class _View:
            pass
        v = _View()
        v.__cuda_array_interface__ = {"shape": (32,), "typestr": "<i8", "data": (self.ptr.value + self.flags_off, False),
                                      "version": 2}
        self._flags_view = v
        return torch.as_tensor(v, device=self.device)

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
    """One rank of the row-partitioned SpMM.  Write this rank's feature rows into `x_local`, call step(), read the
    [n_local, d] result (a buffer reused between steps).  All ranks of `group` must construct, step and close
    together.  x_local may be rewritten as soon as step() has been enqueued in the push and all-gather modes; in the
    peer mode the peers read it during THEIR step, so rewrite it only after a step(fence=True) or a barrier."""

    def __init__(self, shard, d, device, group=None, mode="push", weight_mode=ops.W_EDGE, max_passes=3,
                 priority="auto", priority_own_first="auto"):
        self.shard, self.d, self.device, self.group = shard, int(d), torch.device(device), group
        self.world = dist.get_world_size(group) if (dist.is_initialized() and mode != "local") else 1
        self.rank = shard.rank
        self.mode = mode if self.world > 1 else "local"  # "local": the shard is the whole graph, no exchange
        self.weight_mode = weight_mode
        self.schedule = None
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
        if self.mode not in ("local", "peer", "push"):
            raise RuntimeError("mode must be 'push', 'peer', 'allgather' or 'local', got %r" % (mode,))
        self.plan = HaloPlan(shard)
        n_halo = self.plan.n_halo
        self.shared = SharedBuffer((n_local + n_halo) * d, self.device)
        self.xbuf = self.shared.tensor().view(n_local + n_halo, d)
        self.x_local, self.x_halo = self.xbuf[:n_local], self.xbuf[n_local:]
        self.halo_bytes = n_halo * d * 4
        self.graph = None
        if self.mode != "push":
            self.graph = ops.PreparedGraph(shard.indptr, self.plan.local_indices, n_local + n_halo)
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, self.shared.handle_bytes(), group=group)
            ptrs = [self.shared.ptr.value if p == self.rank else self.shared.open_peer(handles[p])
                    for p in range(self.world)]
            self._ptrs = (C.c_void_p * self.world)(*ptrs)
            self._bounds = (C.c_int64 * (self.world + 1))(*shard.bounds)
            if self.mode == "push":
                self._setup_push(ptrs, max_passes, priority, priority_own_first)

    # ------------------------------------------------------------------------------------------ push set-up
    def _setup_push(self, ptrs, max_passes, priority, priority_own_first="auto"):
        sh, plan, world, rank, d = self.shard, self.plan, self.world, self.rank, self.d
        need_rows, recv_ids, recv_counts = exchange_need_lists(plan, rank, world, self.group)
        mine = torch.tensor(owner_edge_counts(sh, world), dtype=torch.int64, device=self.device)
        blocks = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(blocks, mine, group=self.group)
        rows = [sh.bounds[p + 1] - sh.bounds[p] for p in range(world)]
        self.schedule = PushSchedule(need_rows, [b.tolist() for b in blocks], rows, d, max_passes=max_passes,
                                     priority=priority, priority_own_first=priority_own_first)
        offsets = [None] * world  # offsets[q][p]: first halo slot that rank q reserves for owner p's rows
        dist.all_gather_object(offsets, list(plan.owner_offsets), group=self.group)
        send_ids = (recv_ids - sh.row_begin).to(torch.int32)
        starts = [sum(recv_counts[:q]) for q in range(world)]
        # where rank q keeps its delivery flags: behind its [own | halo] rows
        flags_at = [ptrs[q] + SharedBuffer.flags_offset((rows[q] + sum(need_rows[q])) * d) for q in range(world)]

        def push_args(dests, kind):
            """(push arguments, signal arguments) for the destinations that need rows of this rank; kind 0 raises
            the reader's "all rows of owner `rank` are here" flag, kind 1 its "priority rows" flag."""
            dests = [q for q in dests if q != rank and recv_counts[q] > 0]
            if not dests:
                return None
            ids = torch.cat([send_ids[starts[q]:starts[q] + recv_counts[q]] for q in dests]).contiguous()
            begin = [0]
            for q in dests:
                begin.append(begin[-1] + recv_counts[q])
            # destination pointer = base of q's buffer + (its own rows + the slots before this owner's) rows
            dst = [ptrs[q] + 4 * d * (rows[q] + offsets[q][rank]) for q in dests]
            flags = [flags_at[q] + 8 * (16 * kind + rank) for q in dests]
            return ((len(dests), (C.c_void_p * len(dests))(*dst), (C.c_int64 * (len(dests) + 1))(*begin), ids),
                    (len(dests), (C.c_void_p * len(dests))(*flags)))

        prio = self.schedule.priority
        self._push_first = push_args([prio], 1) if prio is not None else None
        self._push_rest = push_args([q for q in range(world) if q != prio], 0)
        self._passes = []
        for (ip, li, vals, wait), (owners, _) in zip(source_passes(sh, plan, self.schedule.passes[rank]),
                                                     self.schedule.passes[rank]):
            mask = 0
            for p in owners:
                if p != rank and need_rows[rank][p] > 0:
                    mask |= 1 << p
            self._passes.append((ops.PreparedGraph(ip, li, sh.n_local + plan.n_halo), vals, mask))
        self.graph = self._passes[0][0]
        self.push_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self.first_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self._flags = self.shared.flags_tensor()
        self._flag_base = 16 if rank == prio else 0  # the priority reader waits for the priority deliveries
        self._work_counter = torch.zeros(2, dtype=torch.int64, device=self.device)
        self._wait_error = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._step = 0
        self.wait_timeout_ns = 2_000_000_000

    # SMs of the priority delivery: every owner sends to the one priority rank at once, so that rank's ingress (one link
    # direction shared by all of them) paces the transfer; a few SMs per owner keep it fed, and the main push keeps its own
    FIRST_SMS = int(os.environ.get("YITU_PUSH_FIRST_SMS", "12"))  # development switch: the environment overrides

    def _push(self, args, counter=0, n_sms=0):
        (n_dests, dst, begin, ids), (n_flags, flags) = args
        st = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            check(lib().yitu_halo_push_f32(n_dests, dst, begin, _ptr(ids), _ptr(self.x_local), self.d,
                                           C.c_void_p(self._work_counter.data_ptr() + 8 * counter), n_sms, st))
            check(lib().yitu_flags_signal(n_flags, flags, self._step, st))

    def _wait_for(self, mask):
        if mask:
            st = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
            with torch.cuda.device(self.device):
                check(lib().yitu_flags_wait(C.c_void_p(self._flags.data_ptr() + 8 * self._flag_base), mask, self._step,
                                            self.wait_timeout_ns, _ptr(self._wait_error), st))

    def check(self):
        """Synchronises and raises if a wait for a peer's delivery ever ran out (the results of that step are wrong)."""
        torch.cuda.synchronize(self.device)
        if self.mode == "push" and int(self._wait_error) != 0:
            raise RuntimeError("rank %d: the rows of rank %d did not arrive within %.1f s" % (
                self.rank, int(self._wait_error) - 1, self.wait_timeout_ns * 1e-9))

    # ------------------------------------------------------------------------------------------
    def handshake(self):
        """Stream-ordered all-reduce of one float: it completes on a rank only after every rank's earlier work on
        its stream has finished (features written, previous aggregation done with the halo buffer)."""
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)

    def _mark(self, events):
        if events is None:
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(self.device))
        return ev

    def fetch_halo(self, events=None):
        """Peer mode: gather this rank's halo rows from the owners' shards (peer loads)."""
        if self.mode != "peer" or self.plan.n_halo == 0:
            return
        a = self._mark(events)
        st = torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            check(lib().yitu_halo_gather_f32(self.world, self._ptrs, self._bounds, _ptr(self.plan.halo_ids),
                                             self.plan.n_halo, self.d, _ptr(self.x_halo), C.c_void_p(st.cuda_stream)))
        if events is not None:
            events.append(("fetch", a, self._mark(events)))

    def _spmm(self, g, x, vals, accumulate=False, events=None):
        a = self._mark(events)
        out = ops.spmm(g, x, mode=self.weight_mode if vals is not None else ops.W_NONE, edge_values=vals,
                       out=self.out, accumulate=accumulate)
        if events is not None:
            events.append(("spmm", a, self._mark(events)))
        return out

    def _step_push(self, events):
        main = torch.cuda.current_stream(self.device)
        ps = self.push_stream
        self._step += 1
        self.handshake()  # every shard is written, every halo buffer is free
        t0 = self._mark(events)
        if events is not None:
            events.append(("start", t0, t0))
        ps.wait_stream(main)
        # this rank's rows leave from the first moment of the step; each push is followed by the flags that tell its
        # destinations "the rows of this owner are in place".  The priority delivery runs BESIDE the main push, on its
        # own stream and SMs: the priority rank's ingress limits it, and the owner's egress must not idle meanwhile.
        if self._push_first is not None:
            fs = self.first_stream
            fs.wait_stream(main)
            with torch.cuda.stream(fs):
                a = self._mark(events)
                self._push(self._push_first, counter=1, n_sms=self.FIRST_SMS)
                if events is not None:
                    events.append(("push", a, self._mark(events)))
        with torch.cuda.stream(ps):
            a = self._mark(events)
            if self._push_rest is not None:
                self._push(self._push_rest)
            if events is not None:
                events.append(("push", a, self._mark(events)))
        for j, (g, vals, mask) in enumerate(self._passes):
            self._wait_for(mask)  # the owners whose rows this pass gathers
            if events is not None:
                events.append(("ready:pass%d" % j, t0, self._mark(events)))
            self._spmm(g, self.xbuf, vals, accumulate=j > 0, events=events)
        main.wait_stream(ps)  # this rank's shard has been read: it may be rewritten once the step returns
        if self._push_first is not None:
            main.wait_stream(self.first_stream)
        if events is not None:
            events.append(("end", t0, self._mark(events)))
        return self.out

    def step(self, events=None, fence=False):
        """One aggregation over this rank's rows; returns the [n_local, d] output (reused between steps).
        `events`, if a list, receives (tag, start, end) CUDA-event triples around every SpMM, halo fetch and push.
        fence=True (peer mode) adds a second handshake once this rank's halo has arrived, so that no rank's later work
        (which may overwrite its feature shard, as a training step does) starts before every peer has finished
        reading it; the push mode needs no fence (a rank's shard is read by that rank alone)."""
        sh = self.shard
        if self.mode == "local":
            return self._spmm(self.graph, self.x_local, sh.values, events=events)
        if self.mode == "push":
            return self._step_push(events)
        self.handshake()
        if self.mode == "allgather":
            dist.all_gather_into_tensor(self.rep, self._slot, group=self.group)
            return self._spmm(self.graph, self.rep, sh.values, events=events)
        self.fetch_halo(events)
        if fence:
            self.handshake()
        return self._spmm(self.graph, self.xbuf, sh.values, events=events)

    def close(self):
        """Collective: waits for this rank's work and for every peer (nobody may still be reading or writing a
        mapped buffer) before the mappings are closed and the buffer is freed."""
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)
        self._flags = None
        if getattr(self, "shared", None) is not None:
            self.shared.close()
            self.shared = None


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

    def __init__(self, indptr, indices, values, d, device, group=None, bounds=None, mode="push"):
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
                                   weight_mode=wm)
        self.bwd = PartitionedSpmm(RowShard(t_indptr, t_rows, t_values, self.bounds, rank), d, device, group, mode,
                                   weight_mode=wm)

    def __call__(self, x_local):
        return _PartitionedAggregateFunction.apply(x_local, self)

    def close(self):
        self.fwd.close()
        self.bwd.close()
