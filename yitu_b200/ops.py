"""Tensor-level wrappers over the C ABI: argument checks, output allocation, stream forwarding, and the
per-graph cache of derived structures (hub-row schedule, transposed graph).

torch is plumbing here (device memory, the current stream); every aggregation runs in libyitu_b200.so.
"""
import ctypes as C
import weakref

import torch

from . import _lib
from ._lib import (ACT_ELU, ACT_NONE, ACT_RELU, Csr, GatArgs, GatBwdArgs, HubPlan, SpmmArgs, SpmmBwdArgs, W_EDGE,
                   W_EDGE_HEAD, W_NODE, W_NONE, check, lib)

DEFAULT_CHUNK_EDGES = 512
STITCH_MASK = 0xFFFFFF
ACTIVATIONS = {None: ACT_NONE, "none": ACT_NONE, "relu": ACT_RELU, "elu": ACT_ELU}


def activation_code(activation):
    if isinstance(activation, int):
        return activation
    try:
        return ACTIVATIONS[activation]
    except KeyError:
        raise RuntimeError("activation must be None, 'relu' or 'elu', got %r" % (activation,))


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(t, name, dtype=None):
    """Input contract of the reference bindings: CUDA, contiguous (ccsrc/kernel/YiTu_GNN.cpp:65-69) and,
    for graph_ext, an exact dtype (YiTu_GNN/YiTu_H/src/common.h:6-12).  Violations raise RuntimeError."""
    if not isinstance(t, torch.Tensor):
        raise RuntimeError("%s must be a tensor" % name)
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))
    return t


def expect(t, name, shape=None, numel=None, dtype=torch.float32, device=None):
    """Host-side argument check of the tensor-level wrappers (no device synchronisation): the kernels receive raw
    pointers, so a tensor that is short, of another dtype, strided, or on another device must be stopped here,
    as a RuntimeError, before it becomes an out-of-bounds read on the GPU.  None passes (optional arguments)."""
    if t is None:
        return None
    if not isinstance(t, torch.Tensor):
        raise RuntimeError("%s must be a tensor, got %s" % (name, type(t).__name__))
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)
    if device is not None and t.device != device:
        raise RuntimeError("%s is on %s, the graph is on %s" % (name, t.device, device))
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise RuntimeError("%s must have shape %s, got %s" % (name, tuple(shape), tuple(t.shape)))
    if numel is not None and t.numel() != numel:
        raise RuntimeError("%s must hold %d values, got %d" % (name, numel, t.numel()))
    return t


def make_csr(indptr, indices, n_cols, index_mask=0):
    is64 = indptr.dtype == torch.int64
    if not is64 and indptr.dtype != torch.int32:
        raise RuntimeError("row pointers must be int32 or int64, got %s" % indptr.dtype)
    if indices.dtype != torch.int32:
        raise RuntimeError("column indices must be int32, got %s" % indices.dtype)
    return Csr(indptr.numel() - 1, int(n_cols), indices.numel(), _ptr(indptr), int(is64), int(index_mask),
               _ptr(indices))


class PreparedGraph:
    """Derived structures of one CSR, built on first use and kept while the row-pointer tensor lives.

    The reference prepares its schedule on the host once per graph (build_part,
    examples/YiTu_GNN/single/gcn/main.py:90-100) and passes it with every call; the operators here take the
    reference's arguments unchanged and find their own schedule through this cache instead.
    """

    def __init__(self, indptr, indices, n_cols, index_mask=0):
        self.indptr, self.indices = indptr, indices
        self.n_rows, self.n_cols, self.nnz = indptr.numel() - 1, int(n_cols), indices.numel()
        self.index_mask = int(index_mask)
        self.device = indptr.device
        self.csr = make_csr(indptr, indices, n_cols, index_mask)
        self._plans = {}
        self._transpose = None
        self._t_prepared = None
        self._seg_mean = None

    # hub-row schedule ---------------------------------------------------------------------------
    def plan(self, chunk_edges=DEFAULT_CHUNK_EDGES):
        """(HubPlan struct or None, tensors kept alive)."""
        if chunk_edges in self._plans:
            return self._plans[chunk_edges]
        L = lib()
        with torch.cuda.device(self.device):
            ws_bytes = L.yitu_hub_plan_workspace_bytes(self.n_rows)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=self.device)
            n_chunks = C.c_int64(0)
            check(L.yitu_hub_plan_count(C.byref(self.csr), chunk_edges, _ptr(ws), ws_bytes, C.byref(n_chunks),
                                        _stream(self.device)))
            n = n_chunks.value
            if n == 0:
                result = None
            else:
                rows = torch.empty(n, dtype=torch.int32, device=self.device)
                begins = torch.empty(n, dtype=torch.int64, device=self.device)
                check(L.yitu_hub_plan_fill(C.byref(self.csr), chunk_edges, _ptr(ws), n, _ptr(rows), _ptr(begins),
                                           _stream(self.device)))
                result = (HubPlan(chunk_edges, 0, n, _ptr(rows), _ptr(begins)), rows, begins)
        self._plans[chunk_edges] = result
        return result

    # transposed graph ---------------------------------------------------------------------------
    def transpose(self):
        """(t_indptr, t_rows, t_perm): CSC of this graph; t_perm[j] = CSR position of transposed edge j."""
        if self._transpose is None:
            L = lib()
            with torch.cuda.device(self.device):
                ws_bytes = L.yitu_csr_transpose_workspace_bytes(self.n_rows, self.n_cols, self.nnz)
                ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=self.device)
                t_indptr = torch.empty(self.n_cols + 1, dtype=self.indptr.dtype, device=self.device)
                t_rows = torch.empty(self.nnz, dtype=torch.int32, device=self.device)
                t_perm = torch.empty(self.nnz, dtype=torch.int32, device=self.device)
                check(L.yitu_csr_transpose(C.byref(self.csr), _ptr(t_indptr), _ptr(t_rows), _ptr(t_perm), _ptr(ws),
                                           ws_bytes, _stream(self.device)))
            self._transpose = (t_indptr, t_rows, t_perm)
        return self._transpose

    def t_prepared(self):
        if self._t_prepared is None:
            t_indptr, t_rows, _ = self.transpose()
            self._t_prepared = PreparedGraph(t_indptr, t_rows, self.n_rows, 0)
        return self._t_prepared

    def segment_mean_weights(self):
        """values[e] = 1 / #edges of e's (row, segment): mean per relation, summed over relations."""
        if self._seg_mean is None:
            vals = torch.empty(self.nnz, dtype=torch.float32, device=self.device)
            with torch.cuda.device(self.device):
                check(lib().yitu_segment_mean_weights_f32(C.byref(self.csr), _ptr(vals), _stream(self.device)))
            self._seg_mean = vals
        return self._seg_mean


_PREPARED = weakref.WeakValueDictionary()  # memory identity of (indptr, indices) + n_cols + mask -> PreparedGraph


def prepared(indptr, indices, n_cols, index_mask=0):
    """PreparedGraph of a CSR, found by the MEMORY the two tensors occupy (address, length, in-place version counter,
    device), not by the Python tensor objects: callers in the reference's style hand over a fresh tensor object per
    call (a view, an attribute lookup that re-wraps the same storage) and must not pay for a new transpose and hub
    schedule each time.  The table holds its entries weakly; every tensor object that was passed in keeps the entry
    alive (it also pins the memory, so an address cannot be reused while its entry exists), and the derived structures
    die with the last of them.  An in-place modification bumps the version counter and leads to a rebuild."""
    key = (indptr.data_ptr(), indptr.numel(), indptr._version, indices.data_ptr(), indices.numel(), indices._version,
           str(indptr.device), indptr.dtype, int(n_cols), int(index_mask))
    g = _PREPARED.get(key)
    if g is None:
        g = PreparedGraph(indptr, indices, n_cols, index_mask)
        _PREPARED[key] = g
    held = getattr(indptr, "_yitu_prepared", None)
    if held is None or held[0] != key[:8]:
        held = (key[:8], {})
        indptr._yitu_prepared = held
    held[1][key[8:]] = g
    return g


def spmm(graph, x, *, n_heads=1, mode=W_NONE, edge_values=None, edge_perm=None, norm_dst=None, norm_src=None,
         row_scale=None, alpha=1.0, out=None, accumulate=False, chunk_edges=DEFAULT_CHUNK_EDGES, bias=None,
         activation=None, x_shared_heads=False):
    """out[r,h,k] = act(alpha*row_scale[r] * sum_e w(e,h) * x[col_e,h,k] + bias[h,k]) through yitu_spmm_csr_f32.

    x: [n_cols, H*F] or [n_cols, H, F] float32 CUDA; returns a tensor shaped like x with n_rows rows.
    x_shared_heads (per-head edge values only): x is [n_cols, F] and every head reads the same row; the result is
    [n_rows, H, F]."""
    if not isinstance(x, torch.Tensor) or x.dtype != torch.float32:
        raise RuntimeError("features must be a float32 tensor, got %s" % getattr(x, "dtype", type(x).__name__))
    if x.dim() < 2 or x.size(0) != graph.n_cols:
        raise RuntimeError("features have shape %s, the graph has %d source nodes" % (tuple(x.shape), graph.n_cols))
    dev = graph.device
    if not x.is_contiguous():
        x = x.contiguous()
    expect(x, "features", device=dev)
    per_edge = {W_EDGE: graph.nnz, W_EDGE_HEAD: graph.nnz * n_heads}.get(mode)
    if per_edge is not None and edge_values is None:
        raise RuntimeError("this weight mode needs edge_values")
    expect(edge_values, "edge_values", numel=per_edge, device=dev)
    expect(edge_perm, "edge_perm", numel=graph.nnz, dtype=torch.int32, device=dev)
    if mode == W_NODE and (norm_dst is None or norm_src is None):
        raise RuntimeError("W_NODE needs norm_dst and norm_src")
    expect(norm_dst, "norm_dst", numel=graph.n_rows, device=dev)
    expect(norm_src, "norm_src", numel=graph.n_cols, device=dev)
    expect(row_scale, "row_scale", numel=graph.n_rows, device=dev)
    x2 = x.reshape(x.size(0), -1)
    x_width = x2.size(1)
    D = x_width * n_heads if x_shared_heads else x_width
    if D % n_heads:
        raise RuntimeError("feature width %d is not a multiple of n_heads=%d" % (D, n_heads))
    expect(bias, "bias", numel=D, device=dev)
    expect(out, "out", numel=graph.n_rows * D, device=dev)
    if out is None:
        shape = (graph.n_rows, n_heads, x_width) if x_shared_heads else (graph.n_rows,) + tuple(x.shape[1:])
        out = torch.empty(shape, dtype=torch.float32, device=x.device)
        accumulate = False
    a = SpmmArgs()
    a.graph = graph.csr
    a.n_heads, a.n_feats = n_heads, D // n_heads
    a.weight_mode, a.accumulate = mode, int(accumulate)
    a.edge_values, a.edge_perm = _ptr(edge_values), _ptr(edge_perm)
    a.norm_dst, a.norm_src, a.row_scale = _ptr(norm_dst), _ptr(norm_src), _ptr(row_scale)
    a.alpha = float(alpha)
    a.activation = activation_code(activation)
    a.bias, a.x_shared_heads = _ptr(bias), int(bool(x_shared_heads))
    a.x, a.x_stride = _ptr(x2), x_width
    a.out, a.out_stride = _ptr(out), D
    keep = None
    if chunk_edges:
        pl = graph.plan(chunk_edges)
        if pl is not None:
            scratch = torch.empty(pl[0].n_chunks * D, dtype=torch.float32, device=x.device)
            a.plan = C.pointer(pl[0])
            a.scratch, a.scratch_bytes = _ptr(scratch), scratch.numel() * 4
            keep = (pl, scratch)
    with torch.cuda.device(x.device):
        check(lib().yitu_spmm_csr_f32(C.byref(a), _stream(x.device)))
    del keep
    return out


def epilogue_grad(y, grad_y, row_scale=None, activation=None):
    """grad_y * act'(y) * row_scale[r] in one pass (yitu_epilogue_grad_f32); y, grad_y are [n_rows, ...] float32."""
    n_rows = grad_y.size(0)
    width = grad_y.numel() // max(n_rows, 1)
    grad_y = grad_y.contiguous()
    out = torch.empty_like(grad_y)
    code = activation_code(activation)
    with torch.cuda.device(grad_y.device):
        check(lib().yitu_epilogue_grad_f32(n_rows, max(width, 1), code, _ptr(y) if code else None, _ptr(grad_y),
                                           _ptr(row_scale), _ptr(out), _stream(grad_y.device)))
    return out


def _hub_plan(graph, chunk_edges):
    """(pointer to the HubPlan struct or None, number of chunks, objects to keep alive)."""
    if not chunk_edges:
        return None, 0, None
    pl = graph.plan(chunk_edges)
    if pl is None:
        return None, 0, None
    return C.pointer(pl[0]), pl[0].n_chunks, pl


def _heads_feats(graph, x, name):
    """(H, F) of a [n_cols, H, F] float32 source-feature tensor on the graph's device."""
    if not isinstance(x, torch.Tensor) or x.dim() != 3:
        raise RuntimeError("%s must be a [n_src, heads, feats] tensor" % name)
    expect(x, name, shape=(graph.n_cols, x.size(1), x.size(2)), device=graph.device)
    return x.size(1), x.size(2)


def edge_dot(graph, grad_out, x, chunk_edges=DEFAULT_CHUNK_EDGES):
    """grad_a[e,h] = <grad_out[row_e,h,:], x[col_e,h,:]>; grad_out [n_rows,H,F], x [n_cols,H,F]."""
    H, F = _heads_feats(graph, x, "x")
    expect(grad_out, "grad_out", shape=(graph.n_rows, H, F), device=graph.device)
    grad_a = torch.empty((graph.nnz, H), dtype=torch.float32, device=x.device)
    plan, _, keep = _hub_plan(graph, chunk_edges)
    with torch.cuda.device(x.device):
        check(lib().yitu_edge_dot_f32(C.byref(graph.csr), H, F, _ptr(grad_out), _ptr(x), _ptr(grad_a), plan,
                                      _stream(x.device)))
    del keep
    return grad_a


def spmm_bwd_supported(n_heads, n_feats):
    lph = n_feats // 4
    return n_heads <= 32 and n_feats % 4 == 0 and n_heads * n_feats <= 512 and lph <= 32 and (lph & (lph - 1)) == 0


def spmm_bwd(graph, values, x, grad_out, chunk_edges=DEFAULT_CHUNK_EDGES):
    """(grad_values [nnz,H], grad_x [n_cols,H,F]) of the multi-head SpMM with per-edge values, in one pass over the
    transposed graph (yitu_spmm_bwd_f32); shapes outside spmm_bwd_supported take edge_dot + the transposed spmm."""
    H, F = _heads_feats(graph, x, "x")
    dev = x.device
    expect(values, "values", shape=(graph.nnz, H), device=dev)
    expect(grad_out, "grad_out", shape=(graph.n_rows, H, F), device=dev)
    t_indptr, t_rows, t_perm = graph.transpose()
    a = SpmmBwdArgs()
    a.graph = graph.csr
    a.n_heads, a.n_feats = H, F
    grad_values = torch.empty((graph.nnz, H), dtype=torch.float32, device=dev)
    grad_x = torch.empty((graph.n_cols, H, F), dtype=torch.float32, device=dev)
    a.edge_values, a.x, a.grad_out = _ptr(values), _ptr(x), _ptr(grad_out)
    a.t_indptr, a.t_rows, a.t_perm = _ptr(t_indptr), _ptr(t_rows), _ptr(t_perm)
    a.grad_values, a.grad_x = _ptr(grad_values), _ptr(grad_x)
    t_plan, t_chunks, keep = _hub_plan(graph.t_prepared(), chunk_edges)
    if t_plan is not None:
        scratch = torch.empty(t_chunks * H * F, dtype=torch.float32, device=dev)
        a.t_plan, a.scratch, a.scratch_bytes = t_plan, _ptr(scratch), scratch.numel() * 4
    with torch.cuda.device(dev):
        check(lib().yitu_spmm_bwd_f32(C.byref(a), _stream(dev)))
    del keep
    return grad_values, grad_x


def _query_key(graph, query, key, batched):
    """Checks query [B, n_rows, H] (batched) or [n_rows, H] and key [n_cols, H]; returns (B, H)."""
    if not isinstance(key, torch.Tensor) or key.dim() != 2:
        raise RuntimeError("key must be a [n_src, heads] tensor")
    H = key.size(1)
    expect(key, "key", shape=(graph.n_cols, H), device=graph.device)
    if not isinstance(query, torch.Tensor) or query.dim() != (3 if batched else 2):
        raise RuntimeError("query must be a %s tensor" % ("[segments, n_dst, heads]" if batched else "[n_dst, heads]"))
    B = query.size(0) if batched else 1
    expect(query, "query", shape=(B, graph.n_rows, H) if batched else (graph.n_rows, H), device=graph.device)
    return B, H


def edge_softmax_fwd(graph, query, key, slope=0.2, chunk_edges=DEFAULT_CHUNK_EDGES):
    """attn [nnz,H]; query [B,n_rows,H], key [n_cols,H]."""
    B, H = _query_key(graph, query, key, batched=True)
    attn = torch.zeros((graph.nnz, H), dtype=torch.float32, device=key.device)
    plan, _, keep = _hub_plan(graph, chunk_edges)
    with torch.cuda.device(key.device):
        check(lib().yitu_edge_softmax_fwd_f32(C.byref(graph.csr), B, H, slope, _ptr(query), _ptr(key), _ptr(attn), plan,
                                              _stream(key.device)))
    del keep
    return attn


def edge_softmax_bwd(graph, query, key, attn, grad_attn, slope=0.2, chunk_edges=DEFAULT_CHUNK_EDGES):
    """(grad_query [B,n_rows,H], grad_key [n_cols,H])."""
    B, H = _query_key(graph, query, key, batched=True)
    expect(attn, "attn", shape=(graph.nnz, H), device=graph.device)
    expect(grad_attn, "grad_attn", shape=(graph.nnz, H), device=graph.device)
    grad_q = torch.empty_like(query)
    edge_grad = torch.zeros_like(attn)
    grad_k = torch.empty_like(key)
    t_indptr, _, t_perm = graph.transpose()
    plan, _, keep = _hub_plan(graph, chunk_edges)
    t_plan, _, t_keep = _hub_plan(graph.t_prepared(), chunk_edges)
    L = lib()
    with torch.cuda.device(key.device):
        st = _stream(key.device)
        check(L.yitu_edge_softmax_bwd_f32(C.byref(graph.csr), B, H, slope, _ptr(query), _ptr(key), _ptr(attn),
                                          _ptr(grad_attn), _ptr(grad_q), _ptr(edge_grad), plan, st))
        check(L.yitu_edge_gather_sum_f32(graph.n_cols, _ptr(t_indptr), int(t_indptr.dtype == torch.int64),
                                         _ptr(t_perm), H, _ptr(edge_grad), _ptr(grad_k), t_plan, st))
    del keep, t_keep
    return grad_q, grad_k


def _gat_args(graph, query, key, x, out, row_max, row_sum, slope, head_mean=False, activation=None, out_heads=None):
    a = GatArgs()
    a.graph = graph.csr
    a.n_heads, a.n_feats, a.slope = x.size(1), x.size(2), slope
    a.head_mean, a.activation = int(bool(head_mean)), activation_code(activation)
    a.query, a.key, a.x = _ptr(query), _ptr(key), _ptr(x)
    a.out, a.row_max, a.row_sum = _ptr(out), _ptr(row_max), _ptr(row_sum)
    a.out_heads = _ptr(out_heads)
    return a


def gat_fused_supported(graph, n_heads, n_feats, backward=True):
    return graph.index_mask == 0 and n_heads <= 32 and n_feats % 4 == 0 and n_heads * n_feats <= 512


def gat_fwd(graph, query, key, x, slope=0.2, head_mean=False, activation=None, chunk_edges=DEFAULT_CHUNK_EDGES,
            keep_heads=True):
    """Fused scores + edge softmax + aggregation: (out [n_rows,H,F], row_max [n_rows,H], row_sum [n_rows,H]).
    head_mean: out is act(mean over heads), [n_rows,F], and a fourth tensor comes back: the per-head result
    [n_rows,H,F] that gat_bwd needs (None with keep_heads=False: inference, nothing is written but the mean).
    Rows longer than chunk_edges are split over several warps (0: never)."""
    H, F = _heads_feats(graph, x, "x")
    if _query_key(graph, query, key, batched=False)[1] != H:
        raise RuntimeError("query / key have %d heads, x has %d" % (key.size(1), H))
    dev = x.device
    shape = (graph.n_rows, F) if head_mean else (graph.n_rows, H, F)
    out = torch.empty(shape, dtype=torch.float32, device=dev)
    out_heads = torch.empty((graph.n_rows, H, F), dtype=torch.float32, device=dev) if head_mean and keep_heads else None
    row_max = torch.empty((graph.n_rows, H), dtype=torch.float32, device=dev)
    row_sum = torch.empty((graph.n_rows, H), dtype=torch.float32, device=dev)
    a = _gat_args(graph, query, key, x, out, row_max, row_sum, slope, head_mean, activation, out_heads)
    plan, n_chunks, keep = _hub_plan(graph, chunk_edges)
    L = lib()
    if plan is not None:
        nbytes = L.yitu_gat_fwd_scratch_bytes(n_chunks, H, F)
        scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=dev)
        a.plan, a.scratch, a.scratch_bytes = plan, _ptr(scratch), nbytes
    with torch.cuda.device(dev):
        check(L.yitu_gat_fwd_f32(C.byref(a), _stream(dev)))
    del keep
    if head_mean:
        return out, row_max, row_sum, out_heads
    return out, row_max, row_sum


def gat_bwd(graph, query, key, x, out, row_max, row_sum, grad_out, slope=0.2, head_mean=False, out_heads=None,
            chunk_edges=DEFAULT_CHUNK_EDGES):
    """(grad_query, grad_key, grad_x) of gat_fwd; grad_out is the gradient of the pre-activation output
    ([n_rows,F] with head_mean, which also needs out_heads, the fourth result of gat_fwd)."""
    H, F = _heads_feats(graph, x, "x")
    if _query_key(graph, query, key, batched=False)[1] != H:
        raise RuntimeError("query / key have %d heads, x has %d" % (key.size(1), H))
    dev = x.device
    want = (graph.n_rows, F) if head_mean else (graph.n_rows, H, F)
    if not isinstance(grad_out, torch.Tensor) or tuple(grad_out.shape) != want or not grad_out.is_contiguous():
        raise RuntimeError("grad_out must be contiguous with shape %s, got %s" % (want, tuple(getattr(grad_out, "shape", ()))))
    expect(grad_out, "grad_out", device=dev)
    if head_mean and out_heads is None:
        raise RuntimeError("the backward of a head-mean forward needs out_heads (the fourth result of gat_fwd)")
    expect(out, "out", shape=want, device=dev)
    expect(out_heads, "out_heads", shape=(graph.n_rows, H, F), device=dev)
    expect(row_max, "row_max", shape=(graph.n_rows, H), device=dev)
    expect(row_sum, "row_sum", shape=(graph.n_rows, H), device=dev)
    t_indptr, t_rows, t_perm = graph.transpose()
    b = GatBwdArgs()
    b.fwd = _gat_args(graph, query, key, x, out, row_max, row_sum, slope, head_mean, None, out_heads)
    grad_q = torch.empty_like(query)
    grad_k = torch.empty_like(key)
    grad_x = torch.empty_like(x)
    lph = F // 4
    one_pass = lph <= 32 and (lph & (lph - 1)) == 0
    edge_attn = None if one_pass else torch.empty((graph.nnz, H), dtype=torch.float32, device=dev)
    edge_grad = torch.empty((graph.nnz, H), dtype=torch.float32, device=dev)
    b.grad_out = _ptr(grad_out)
    b.t_indptr, b.t_rows, b.t_perm = _ptr(t_indptr), _ptr(t_rows), _ptr(t_perm)
    b.grad_query, b.grad_key, b.grad_x = _ptr(grad_q), _ptr(grad_k), _ptr(grad_x)
    b.edge_attn, b.edge_grad = _ptr(edge_attn), _ptr(edge_grad)
    plan, n_chunks, keep = _hub_plan(graph, chunk_edges)
    t_plan, t_chunks, t_keep = _hub_plan(graph.t_prepared(), chunk_edges)
    L = lib()
    nbytes = L.yitu_gat_bwd_scratch_bytes(graph.n_rows, n_chunks, t_chunks, H, F)
    scratch = torch.empty(max(nbytes // 4, 1), dtype=torch.float32, device=dev)
    b.fwd.plan, b.t_plan = plan, t_plan
    b.scratch, b.scratch_bytes = _ptr(scratch), nbytes
    with torch.cuda.device(dev):
        check(L.yitu_gat_bwd_f32(C.byref(b), _stream(dev)))
    del keep, t_keep
    return grad_q, grad_k, grad_x


def partition_rows(graph, n_parts):
    """Edge-balanced contiguous row ranges as an int64 device tensor [n_parts+1]."""
    bounds = torch.empty(n_parts + 1, dtype=torch.int64, device=graph.device)
    with torch.cuda.device(graph.device):
        check(lib().yitu_partition_rows(C.byref(graph.csr), n_parts, _ptr(bounds), _stream(graph.device)))
    return bounds


def partition_rows_host(indptr, n_parts):
    """Same partition from a CPU row-pointer tensor (int32 or int64)."""
    indptr = indptr.contiguous()
    bounds = torch.empty(n_parts + 1, dtype=torch.int64)
    check(lib().yitu_partition_rows_host(indptr.numel() - 1, _ptr(indptr), int(indptr.dtype == torch.int64), n_parts,
                                         _ptr(bounds)))
    return bounds


def coo_to_csr(src, dst, n_src, n_dst, self_loops=False, ptr_dtype=torch.int32):
    """Edge list (int32 CUDA tensors) -> (indptr, indices) by destination on the device: duplicates dropped,
    optional self-loops, ascending columns — what the reference builds with scipy on the host
    (YiTu_GNN/data/dataset.py:117-129)."""
    require_cuda(src, "src", torch.int32)
    require_cuda(dst, "dst", torch.int32)
    if src.numel() != dst.numel():
        raise RuntimeError("src and dst differ in length")
    dev = src.device
    n_edges = src.numel()
    L = lib()
    cap = n_edges + (n_dst if self_loops else 0)
    indptr = torch.empty(n_dst + 1, dtype=ptr_dtype, device=dev)
    indices = torch.empty(max(cap, 1), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        ws_bytes = L.yitu_coo_to_csr_workspace_bytes(n_edges, n_dst, int(self_loops))
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        nnz = C.c_int64(0)
        check(L.yitu_coo_to_csr(n_src, n_dst, n_edges, _ptr(src), _ptr(dst), int(self_loops), _ptr(indptr),
                                int(ptr_dtype == torch.int64), _ptr(indices), C.byref(nnz), _ptr(ws), ws_bytes,
                                _stream(dev)))
    return indptr, indices[:nnz.value].clone()


DEG_SQRT, DEG_RSQRT, DEG_INV = 0, 1, 2


def degree_norm(indptr, mode=DEG_SQRT):
    """float32 [n_rows] from d = max(in-degree, 1): sqrt(d) (the reference's `degrees`,
    YiTu_GNN/data/dataset.py:131-133), 1/sqrt(d), or 1/d."""
    n = indptr.numel() - 1
    out = torch.empty(n, dtype=torch.float32, device=indptr.device)
    with torch.cuda.device(indptr.device):
        check(lib().yitu_degree_norm_f32(n, _ptr(indptr), int(indptr.dtype == torch.int64), mode, _ptr(out),
                                         _stream(indptr.device)))
    return out


def stitch_csr_device(indptrs, indices, n_cols):
    """Device stitch_csr over CUDA int32 block tables: (indptr, indices) of the segmented CSR, on the device."""
    n_blocks = len(indptrs)
    n_rows = indptrs[0].numel() - 1 if n_blocks else 0
    dev = indptrs[0].device
    total = sum(int(i.numel()) for i in indices)
    out_ip = torch.empty(n_rows + 1, dtype=torch.int32, device=dev)
    out_id = torch.empty(max(total, 1), dtype=torch.int32, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    PP = C.c_void_p * max(n_blocks, 1)
    ncols = (C.c_int64 * max(n_blocks, 1))(*[int(c) for c in n_cols])
    with torch.cuda.device(dev):
        check(lib().yitu_stitch_csr(n_blocks, n_rows, PP(*[t.data_ptr() for t in indptrs]),
                                    PP(*[t.data_ptr() for t in indices]), ncols, _ptr(out_ip), _ptr(out_id), _ptr(flag),
                                    _stream(dev)))
    if int(flag) != 0:
        raise AssertionError("stitched column exceeds 2**24")
    return out_ip, out_id[:total]
