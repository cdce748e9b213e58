"""Message-passing DSL of YiTu_GNN/YiTu_H/xgnn_h/mp.py:32-135 (`Fn`, `Graph`, `HeteroGraph`) that EXECUTES.

In the reference the DSL only records operations for its tracing compiler (eager calls return zero tensors,
mp.py:7-29) and the kernels are reached after trace -> optimise -> stitch -> execute.  Here the same calls run
directly on the B200 operators: per-edge values stay symbolic (`EdgeExpr`) until a `reduce_func` consumes them, and the
reduction picks the kernel by the shape of the expression, as the reference's optimiser does by pattern
(xgnn_h/optimizer.py:20-111):

    aggregate_sum(copy_u(x))                                           -> sparse.gspmm(block, None, x)
    aggregate_sum(u_mul_e(x, edge_softmax(LeakyReLU_0.2(u_add_v(k, q)))))  -> sparse.fused_gat(block, q, k, x)
    aggregate_sum(u_mul_e(x, e))                                       -> sparse.gspmm(block, e, x)

Anything else is evaluated edge by edge with torch indexing (correct, slow).  Layers written against the
reference's DSL (YiTu_GNN/YiTu_H/test/common/model.py:7-106) run unchanged on a `Graph` made from a `Block`.
"""
import torch
import torch.nn.functional as F

from . import block, sparse

_MASK = 0xFFFFFF


class Fn:
    """Operation descriptors, field for field those of the reference (mp.py:32-70)."""

    @classmethod
    def copy_u(cls, u, e):
        return {'func': 'copy_u', 'u': u, 'out': e}

    @classmethod
    def u_add_v(cls, u, v, e):
        return {'func': 'u_add_v', 'u': u, 'v': v, 'out': e}

    @classmethod
    def u_mul_e(cls, u, e, v):
        return {'func': 'u_mul_e', 'u': u, 'e': e, 'out': v}

    @classmethod
    def edge_softmax(cls, e1, e2):
        return {'func': 'edge_softmax', 'e': e1, 'out': e2}

    @classmethod
    def aggregate_sum(cls, e, v):
        return {'func': 'aggregate_sum', 'e': e, 'out': v}


class EdgeExpr:
    """A per-edge value that has not been computed yet.  torch functions applied to it are recorded when a kernel
    can absorb them (LeakyReLU before an edge softmax) and otherwise force the value (`materialize`)."""

    def __init__(self, graph, op, **args):
        self.graph, self.op, self.args = graph, op, args

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is F.leaky_relu and isinstance(args[0], EdgeExpr) and not kwargs.get('inplace', False):
            slope = args[1] if len(args) > 1 else kwargs.get('negative_slope', 0.01)
            return EdgeExpr(args[0].graph, 'leaky_relu', e=args[0], slope=float(slope))
        args = [a.materialize() if isinstance(a, EdgeExpr) else a for a in args]
        kwargs = {k: (v.materialize() if isinstance(v, EdgeExpr) else v) for k, v in kwargs.items()}
        return func(*args, **kwargs)

    # -- structure tests used by Graph.reduce_func -------------------------------------------------
    def is_gat_attention(self):
        """edge_softmax(LeakyReLU_0.2(u_add_v(k, q))) -> (k, q) or None."""
        if self.op != 'edge_softmax':
            return None
        e = self.args['e']
        if not (isinstance(e, EdgeExpr) and e.op == 'leaky_relu' and abs(e.args['slope'] - 0.2) < 1e-12):
            return None
        s = e.args['e']
        if not (isinstance(s, EdgeExpr) and s.op == 'u_add_v'):
            return None
        return s.args['u'], s.args['v']

    # -- generic evaluation ------------------------------------------------------------------------
    def materialize(self):
        g, a = self.graph, self.args
        rows, cols = g._edge_endpoints()
        if self.op == 'copy_u':
            return a['u'][cols]
        if self.op == 'u_add_v':   # u: per source node, v: per destination node
            return a['u'][cols] + a['v'][rows]
        if self.op == 'leaky_relu':
            return F.leaky_relu(_value(a['e']), a['slope'])
        if self.op == 'u_mul_e':
            return a['u'][cols] * _value(a['e']).unsqueeze(-1)
        if self.op == 'edge_softmax':
            gat = self.is_gat_attention()
            if gat is not None:
                key, query = gat
                return sparse.fused_gsddmm(g.blk, query, key)
            return _segment_softmax(_value(a['e']), rows, g.num_dst_nodes())
        raise RuntimeError("unknown edge operation %r" % self.op)


def _value(e):
    return e.materialize() if isinstance(e, EdgeExpr) else e


def _segment_softmax(scores, rows, n_rows):
    """Softmax of scores [E, ...] over the edges of each destination row, with torch scatter operations."""
    idx = rows.view(-1, *([1] * (scores.dim() - 1))).expand_as(scores)
    top = torch.full((n_rows,) + tuple(scores.shape[1:]), float('-inf'), dtype=scores.dtype, device=scores.device)
    top = top.scatter_reduce(0, idx, scores.detach(), reduce='amax', include_self=True)
    ex = torch.exp(scores - top[rows])
    den = torch.zeros_like(top).index_add_(0, rows, ex)
    return ex / den[rows]


class Graph:
    """One block of edges with named source / destination / edge data (mp.py:73-135)."""

    def __init__(self, blk: block.Block):
        self.blk = blk
        self.edge = dict()
        self.src_node = dict()
        self.dst_node = dict()
        self._endpoints = None

    @staticmethod
    def from_csr(indptr, indices, n_src, right_norm=None):
        """Graph over a CSR by destination (int32 tensors).  right_norm defaults to 1/in_degree as a column, the
        tensor the reference attaches in from_dglgraph (mp.py:160-167)."""
        n_dst = indptr.numel() - 1
        if right_norm is None:
            deg = (indptr[1:] - indptr[:-1]).to(torch.float32)
            right_norm = torch.div(1.0, deg).unsqueeze(-1)
        return Graph(block.Block([n_dst, n_src], [indptr, indices], right_norm))

    def device(self):
        for v in self.src_node.values():
            return v.device
        raise RuntimeError

    def num_edges(self):
        return self.blk.num_edges()

    def num_src_nodes(self):
        return self.blk.num_src_nodes()

    def num_dst_nodes(self):
        return self.blk.num_dst_nodes()

    def num_features(self):
        n_features = None
        for v in self.src_node.values():
            if v.dim() != 3:
                continue
            if not n_features:
                n_features = v.size(-1)
            assert n_features == v.size(-1)
        assert n_features
        return n_features

    def right_norm(self):
        return self.blk.right_norm

    def _edge_endpoints(self):
        """(destination row, source column) of every edge, int64, built once."""
        if self._endpoints is None:
            indptr, indices = self.blk.adj_sparse
            deg = (indptr[1:] - indptr[:-1]).long()
            rows = torch.repeat_interleave(torch.arange(deg.numel(), device=indptr.device), deg)
            self._endpoints = (rows, (indices & _MASK).long())
        return self._endpoints

    def _lookup(self, name):
        for data in (self.edge, self.src_node, self.dst_node):   # the reference's search order (mp.py:117-126)
            if name in data:
                return data[name]
        raise KeyError("no graph data named %r" % name)

    def message_func(self, desc: dict):
        func = desc['func']
        if func == 'copy_u':
            value = EdgeExpr(self, 'copy_u', u=self._lookup(desc['u']))
        elif func == 'u_add_v':
            value = EdgeExpr(self, 'u_add_v', u=self._lookup(desc['u']), v=self._lookup(desc['v']))
        elif func == 'u_mul_e':
            value = EdgeExpr(self, 'u_mul_e', u=self._lookup(desc['u']), e=self._lookup(desc['e']))
        elif func == 'edge_softmax':
            value = EdgeExpr(self, 'edge_softmax', e=self._lookup(desc['e']))
        else:
            raise RuntimeError("unknown message function %r" % func)
        self.edge[desc['out']] = value

    def reduce_func(self, desc):
        if desc['func'] != 'aggregate_sum':
            raise RuntimeError("unknown reduce function %r" % desc['func'])
        self.dst_node[desc['out']] = self._aggregate_sum(self._lookup(desc['e']))

    def _aggregate_sum(self, e):
        if isinstance(e, EdgeExpr) and e.op == 'copy_u' and e.args['u'].dim() == 3:
            return sparse.gspmm(self.blk, None, e.args['u'])
        if isinstance(e, EdgeExpr) and e.op == 'u_mul_e' and e.args['u'].dim() == 3:
            x, w = e.args['u'], e.args['e']
            gat = w.is_gat_attention() if isinstance(w, EdgeExpr) else None
            if gat is not None and gat[0].dim() == 2 and gat[1].dim() == 2:
                key, query = gat
                return sparse.fused_gat(self.blk, query, key, x)
            return sparse.gspmm(self.blk, _value(w).contiguous(), x)
        msg = _value(e)
        rows, _ = self._edge_endpoints()
        out = torch.zeros((self.num_dst_nodes(),) + tuple(msg.shape[1:]), dtype=msg.dtype, device=msg.device)
        return out.index_add_(0, rows, msg)

    @staticmethod
    def from_dglgraph(graph):
        raise ImportError("from_dglgraph needs DGL; build the graph with Graph.from_csr(indptr, indices, n_src)")


class HeteroGraph:
    """(source type, edge type, destination type) -> Graph (mp.py:170-235)."""

    def __init__(self):
        self.device = None
        self.etypes = []
        self.nty2num = {}
        self.idx2rel = {}
        self.rel2idx = {}
        self.hetero_graph = {}

    def __iter__(self):
        return iter(self.hetero_graph.items())

    @staticmethod
    def from_blocks(relations: dict, nty2num: dict = None):
        """relations maps (sty, ety, dty) to a Block or a Graph."""
        h = HeteroGraph()
        for (sty, ety, dty), g in relations.items():
            g = g if isinstance(g, Graph) else Graph(g)
            h.device = g.blk.adj_sparse[0].device
            if ety not in h.etypes:
                h.etypes.append(ety)
            h.nty2num[sty] = g.num_src_nodes()
            h.nty2num[dty] = g.num_dst_nodes()
            h.idx2rel[len(h.idx2rel)] = [sty, ety, dty]
            h.rel2idx[sty, ety, dty] = len(h.rel2idx)
            h.hetero_graph[sty, ety, dty] = g
        if nty2num:
            h.nty2num.update(nty2num)
        return h

    @staticmethod
    def from_dglgraph(graph):
        raise ImportError("from_dglgraph needs DGL; build the graph with HeteroGraph.from_blocks(...)")
