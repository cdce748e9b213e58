"""Message-passing DSL of YiTu_GNN/YiTu_H/xgnn_h/mp.py:32-135 (`Fn`, `Graph`, `HeteroGraph`) that EXECUTES.

In the reference the DSL only records operations for its tracing compiler (eager calls return zero tensors,
mp.py:7-29) and the kernels are reached after trace -> optimise -> stitch -> execute.  Here the same calls run
directly on the B200 operators: per-edge values stay symbolic (`EdgeExpr`) until a `reduce_func` consumes them, and the
reduction picks the kernel by the shape of the expression, as the reference's optimiser does by pattern
(xgnn_h/optimizer.py:20-111):

    aggregate_sum(copy_u(x))                                           -> sparse.gspmm(block, None, x)
    aggregate_sum(u_mul_e(x, edge_softmax(LeakyReLU_0.2(u_add_v(k, q)))))  -> sparse.fused_gat(block, q, k, x)
    aggregate_sum(u_mul_e(x, e))                                       -> sparse.gspmm(block, e, x)
    edge_softmax(LeakyReLU_0.2(u_add_v(k, q))) asked for its values       -> sparse.fused_gsddmm(block, q, k)

There is no fallback: an expression that none of the kernels evaluates raises a RuntimeError that names it.

Stitching across relations is automatic.  On a Graph that belongs to a HeteroGraph, reduce_func returns a deferred
result (`DeferredAgg`).  The operations a layer applies to it - squeeze(1), multiplication by the per-relation norm
column, the mean over heads - are recorded, the `+` with which a hetero convolution adds the relations of one
destination type (YiTu_GNN/YiTu_H/test/common/model.py:164-168) joins the deferred results, and the first real use
computes them together: the relations are stitched into one segmented CSR (stitch_csr) and ONE aggregation kernel
(for attention: one segmented edge softmax and one SpMM) runs per destination type.  The per-relation norm becomes
a per-edge weight norm_r[row], so it survives the stitch - the reference's stitcher loses it
(xgnn_h/stitcher.py:283-299).  Layers and models written against the reference's DSL
(model.py:7-106,137-171,197-285) run unchanged.
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

    # -- evaluation --------------------------------------------------------------------------------
    def describe(self):
        inner = {k: (v.describe() if isinstance(v, EdgeExpr) else "tensor%s" % (tuple(v.shape),) if torch.is_tensor(v) else repr(v))
                 for k, v in self.args.items()}
        return "%s(%s)" % (self.op, ", ".join("%s=%s" % kv for kv in inner.items()))

    def materialize(self):
        """The per-edge values, when a kernel produces them: the GAT attention pattern is the fused SDDMM + edge
        softmax.  No other bare per-edge expression has a kernel."""
        gat = self.is_gat_attention()
        if gat is not None and gat[0].dim() == 2 and gat[1].dim() == 2:
            key, query = gat
            return sparse.fused_gsddmm(self.graph.blk, query, key)
        raise RuntimeError("no kernel evaluates the per-edge expression %s: supported are aggregate_sum(copy_u(x)), "
                           "aggregate_sum(u_mul_e(x, e)) and edge_softmax(LeakyReLU_0.2(u_add_v(k, q)))" % self.describe())


def _value(e):
    return e.materialize() if isinstance(e, EdgeExpr) else e


class _Term:
    """One relation's aggregation: kind 'sum' (copy_u), 'weighted' (u_mul_e with given edge values) or 'gat'."""

    def __init__(self, graph, kind, x, query=None, key=None, values=None):
        self.graph, self.kind, self.x, self.query, self.key, self.values = graph, kind, x, query, key, values
        self.scale = None  # per-destination factor [n_dst] recorded from a multiplication by the norm column

    def shape(self):
        x = self.x
        return (self.graph.num_dst_nodes(),) + tuple(x.shape[1:])

    def compute(self):
        blk, x = self.graph.blk, self.x
        if self.kind == 'gat':
            out = sparse.fused_gat(blk, self.query, self.key, x)
        elif self.kind == 'weighted':
            out = sparse.gspmm(blk, self.values, x)
        elif x.dim() == 2:
            out = sparse.gspmm(blk, None, x.unsqueeze(1)).squeeze(1)
        else:
            out = sparse.gspmm(blk, None, x)
        if self.scale is not None:
            out = out * self.scale.view(-1, *([1] * (out.dim() - 1)))
        return out


class DeferredAgg:
    """The not yet computed result of reduce_func on a graph of a HeteroGraph: a sum over `terms` (one per relation),
    then the recorded `post` operations ('squeeze1', 'mean1'), then a factor alpha.  Behaves like the tensor it
    stands for: any torch function or method other than the recorded ones computes it first."""

    def __init__(self, terms, post=(), alpha=1.0):
        self.terms, self.post, self.alpha = list(terms), tuple(post), float(alpha)
        self._value = None

    # -- what it looks like ------------------------------------------------------------------------
    @property
    def shape(self):
        shp = list(self.terms[0].shape())
        for op in self.post:
            if len(shp) == 3:
                del shp[1]
        return torch.Size(shp)

    def size(self, dim=None):
        return self.shape if dim is None else self.shape[dim]

    def dim(self):
        return len(self.shape)

    @property
    def device(self):
        return self.terms[0].x.device

    @property
    def dtype(self):
        return self.terms[0].x.dtype

    # -- recorded operations -----------------------------------------------------------------------
    def _n_dst(self):
        return self.terms[0].graph.num_dst_nodes()

    def _copy(self, terms=None, post=None, alpha=None):
        return DeferredAgg(self.terms if terms is None else terms, self.post if post is None else post,
                           self.alpha if alpha is None else alpha)

    def squeeze(self, dim=None):
        if dim in (1, -2) and not self.post and self.dim() == 3 and self.shape[1] == 1:
            return self._copy(post=('squeeze1',))
        return self.materialize().squeeze() if dim is None else self.materialize().squeeze(dim)

    def mean(self, dim=None, **kw):
        if dim in (1, -2) and not self.post and not kw and self.dim() == 3:
            return self._copy(post=('mean1',))
        return self.materialize().mean(dim, **kw) if dim is not None else self.materialize().mean(**kw)

    def _scaled(self, t):
        """self * t for a per-destination column t (the norm of GCNLayer, model.py:30), else None."""
        n = self._n_dst()
        if (torch.is_tensor(t) and t.numel() == n and not t.requires_grad and t.dtype == self.dtype and
                (t.dim() == 1 or tuple(t.shape) == (n,) + (1,) * (t.dim() - 1)) and t.dim() <= self.dim() and
                all(term.scale is None for term in self.terms) and self.alpha == 1.0):
            terms = []
            for term in self.terms:
                c = _Term(term.graph, term.kind, term.x, term.query, term.key, term.values)
                c.scale = t.reshape(-1).contiguous()
                terms.append(c)
            return self._copy(terms=terms)
        return None

    def __mul__(self, other):
        if isinstance(other, (int, float)):
            return self._copy(alpha=self.alpha * other)
        out = self._scaled(other)
        return out if out is not None else self.materialize() * _real(other)

    __rmul__ = __mul__

    def __truediv__(self, other):
        if isinstance(other, (int, float)):
            return self._copy(alpha=self.alpha / other)
        return self.materialize() / _real(other)

    def __add__(self, other):
        if (isinstance(other, DeferredAgg) and other.post == self.post and other.alpha == self.alpha and
                other._n_dst() == self._n_dst() and other.shape == self.shape):
            return self._copy(terms=self.terms + other.terms)
        return self.materialize() + _real(other)

    __radd__ = __add__

    def __getattr__(self, name):
        # any other tensor attribute or method: compute, then behave like the tensor
        if name.startswith('__'):
            raise AttributeError(name)
        return getattr(self.materialize(), name)

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        d = args[0] if args else None
        if func is torch.squeeze and isinstance(d, DeferredAgg) and len(args) + len(kwargs) == 2:
            return d.squeeze(args[1] if len(args) > 1 else kwargs.get('dim'))
        if func is torch.mean and isinstance(d, DeferredAgg) and set(kwargs) <= {'dim'} and len(args) + len(kwargs) == 2:
            return d.mean(args[1] if len(args) > 1 else kwargs['dim'])
        if func in (torch.multiply, torch.mul) and len(args) == 2 and not kwargs:
            a, b = args
            return a * b if isinstance(a, DeferredAgg) else b * a
        if func is torch.add and len(args) == 2 and not kwargs:
            a, b = args
            return a + b if isinstance(a, DeferredAgg) else b + a
        if func in (torch.div, torch.true_divide) and len(args) == 2 and not kwargs and isinstance(d, DeferredAgg):
            return d / args[1]
        args = [_real(a) for a in args]
        kwargs = {k: _real(v) for k, v in kwargs.items()}
        return func(*args, **kwargs)

    # -- evaluation --------------------------------------------------------------------------------
    def materialize(self):
        if self._value is None:
            out = self._stitched() if len(self.terms) > 1 else None
            if out is None:
                out = self.terms[0].compute()
                for term in self.terms[1:]:
                    out = out + term.compute()
            for op in self.post:
                out = torch.squeeze(out, 1) if op == 'squeeze1' else torch.mean(out, dim=1)
            self._value = out if self.alpha == 1.0 else out * self.alpha
        return self._value

    def _stitched(self):
        """All relations of this destination type in one pass over their stitched CSR, or None when they do not fit
        one kernel (mixed kinds, different widths, more than 16 relations, graphs of different HeteroGraphs)."""
        terms = self.terms
        hetero = terms[0].graph.hetero
        kinds = {t.kind for t in terms}
        if (hetero is None or len(kinds) != 1 or len(terms) > 16 or any(t.graph.hetero is not hetero for t in terms) or
                len({tuple(t.x.shape[1:]) for t in terms}) != 1 or len({t.graph.relation for t in terms}) != len(terms)):
            return None
        kind = kinds.pop()
        sblk, seg, rows = hetero.stitched([t.graph for t in terms])
        if kind == 'gat':
            if any(t.scale is not None for t in terms):
                return None
            x = torch.cat([t.x for t in terms]).contiguous()
            attn = sparse.fused_gsddmm(sblk, torch.stack([t.query for t in terms]).contiguous(),
                                       torch.cat([t.key for t in terms]).contiguous())
            return sparse.gspmm(sblk, attn, x)
        if kind != 'sum':
            return None
        from ..nn.layers import aggregate  # the fixed-weight aggregation with scalar edge weights
        x = torch.cat([t.x for t in terms])
        weights = None
        if any(t.scale is not None for t in terms):
            # the per-relation norm as a per-edge weight: weight(e) = norm_{relation(e)}[row(e)]
            ones = torch.ones(sblk.size[0], dtype=x.dtype, device=x.device)
            table = torch.stack([t.scale if t.scale is not None else ones for t in terms])
            weights = table[seg, rows].contiguous()
        wide = x.reshape(x.size(0), -1)
        out = aggregate(sblk, wide, weights=weights, index_mask=_MASK)
        return out.view((out.size(0),) + tuple(x.shape[1:]))


def _real(v):
    return v.materialize() if isinstance(v, DeferredAgg) else v


class Graph:
    """One block of edges with named source / destination / edge data (mp.py:73-135)."""

    def __init__(self, blk: block.Block):
        self.blk = blk
        self.edge = dict()
        self.src_node = dict()
        self.dst_node = dict()
        self._endpoints = None
        self.hetero = None   # the HeteroGraph this graph belongs to (then reductions are deferred and stitched)
        self.relation = None

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
        term = self._term(self._lookup(desc['e']))
        if self.hetero is not None and self.hetero.stitch:
            self.dst_node[desc['out']] = DeferredAgg([term])
        else:
            self.dst_node[desc['out']] = term.compute()

    def _term(self, e):
        """The aggregation that aggregate_sum(e) stands for, as one of the kernel patterns."""
        if isinstance(e, EdgeExpr) and e.op == 'copy_u' and e.args['u'].dim() in (2, 3):
            return _Term(self, 'sum', e.args['u'])
        if isinstance(e, EdgeExpr) and e.op == 'u_mul_e' and e.args['u'].dim() == 3:
            x, w = e.args['u'], e.args['e']
            gat = w.is_gat_attention() if isinstance(w, EdgeExpr) else None
            if gat is not None and gat[0].dim() == 2 and gat[1].dim() == 2:
                key, query = gat
                return _Term(self, 'gat', x, query=query, key=key)
            return _Term(self, 'weighted', x, values=_value(w).contiguous())
        what = e.describe() if isinstance(e, EdgeExpr) else "a tensor of shape %s" % (tuple(e.shape),)
        raise RuntimeError("no kernel evaluates aggregate_sum(%s): supported are aggregate_sum(copy_u(x)) and "
                           "aggregate_sum(u_mul_e(x, e)) with x of shape [n_src, heads, feats]" % what)

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
        self.stitch = True     # defer reductions and stitch the relations of a destination type (False: one kernel each)
        self._stitched = {}

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
            g.hetero, g.relation = h, (sty, ety, dty)
        if nty2num:
            h.nty2num.update(nty2num)
        return h

    def stitched(self, graphs):
        """(stitched Block, relation index of every edge, destination row of every edge) for the given relations of
        one destination type, built once per set of relations (stitch_csr on the device)."""
        key = tuple(g.relation for g in graphs)
        if key not in self._stitched:
            sblk = block.stitch_csr([g.blk for g in graphs])
            indptr, indices = sblk.adj_sparse
            deg = (indptr[1:] - indptr[:-1]).long()
            rows = torch.repeat_interleave(torch.arange(deg.numel(), device=indptr.device), deg)
            self._stitched[key] = (sblk, (indices >> 24).long(), rows)
        return self._stitched[key]

    @staticmethod
    def from_dglgraph(graph):
        raise ImportError("from_dglgraph needs DGL; build the graph with HeteroGraph.from_blocks(...)")
