"""Layer-level modules of the YiTu_H path over the B200 kernels.

GCNLayer, GATLayer and HeteroGraphConv carry the mathematics of the reference's layers
(YiTu_GNN/YiTu_H/test/common/model.py:7-30, 61-106, 137-171); there they are written against the message-passing
DSL and reach the kernels through the tracing compiler, here they call the operators directly and take a
`Block` (xgnn_h/block.py) where the reference takes an `mp.Graph` wrapping one.  StitchedRGCNConv is the fused
form of HeteroGraphConv over GCNLayers for one destination type: one pass over the stitched relations.
"""
import torch
from torch import autograd, nn

from .. import ops
from ..xgnn_h import sparse
from ..xgnn_h.block import Block, stitch_csr


def _block_of(graph):
    return graph if isinstance(graph, Block) else graph.blk


class _AggregateFunction(autograd.Function):
    """y = A x with fixed per-edge weights (or none): forward SpMM, backward the transposed SpMM."""

    @staticmethod
    def forward(ctx, x, graph, weights):
        ctx.graph, ctx.weights = graph, weights
        mode = ops.W_NONE if weights is None else ops.W_EDGE
        return ops.spmm(graph, x.contiguous(), mode=mode, edge_values=weights)

    @staticmethod
    def backward(ctx, grad_out):
        g, w = ctx.graph, ctx.weights
        gt = g.t_prepared()
        if w is None:
            return ops.spmm(gt, grad_out.contiguous(), mode=ops.W_NONE), None, None
        return ops.spmm(gt, grad_out.contiguous(), mode=ops.W_EDGE, edge_values=w, edge_perm=g.transpose()[2]), None, None


def aggregate(block, x, weights=None, index_mask=0):
    """Differentiable sum (or fixed-weight sum) of source rows per destination row; x is [n_src, D]."""
    g = ops.prepared(block.adj_sparse[0], block.adj_sparse[1], x.size(0), index_mask)
    return _AggregateFunction.apply(x, g, weights)


class GCNLayer(nn.Module):
    """norm * (A (x W^T + b)) — model.py:7-30; `norm` is the per-destination 1/in_degree column (mp.py:165-167)."""

    def __init__(self, in_features: int, out_features: int):
        nn.Module.__init__(self)
        self.fc = nn.Linear(in_features, out_features)

    def forward(self, graph, norm, x):
        if isinstance(x, (list, tuple)):
            assert len(x) == 2
            x = x[0]
        h = aggregate(_block_of(graph), self.fc(x))
        return torch.multiply(norm, h)


class GATLayer(nn.Module):
    """mean over heads of softmax-weighted aggregation — model.py:61-106."""

    def __init__(self, in_features: int, out_features: int, n_heads: int):
        nn.Module.__init__(self)
        self.n_heads, self.n_features = n_heads, out_features
        self.linear_q = nn.Linear(n_heads * out_features, n_heads)
        self.linear_k = nn.Linear(n_heads * out_features, n_heads)
        self.linear_v = nn.Linear(in_features, n_heads * out_features)

    def forward(self, graph, x):
        if isinstance(x, (list, tuple)):
            assert len(x) == 2
            h_src, h_dst = self.linear_v(x[0]), self.linear_v(x[1])
        elif isinstance(x, torch.Tensor):
            h_src = h_dst = self.linear_v(x)
        else:
            raise TypeError
        q = self.linear_q(h_dst)
        k = self.linear_k(h_src)
        h_src = h_src.view(-1, self.n_heads, self.n_features)
        out = sparse.fused_gat(_block_of(graph), q, k, h_src)
        return torch.mean(out, dim=1)


class HeteroGraphConv(nn.Module):
    """Per relation (src type, edge type, dst type) one conv; results summed per destination type and divided by
    the number of relations that reach it — model.py:137-171.  `hgraph` maps (sty, ety, dty) to a Block."""

    def __init__(self, convs: dict):
        nn.Module.__init__(self)
        self.convs = nn.ModuleDict(convs)

    def forward(self, hgraph, xs: dict, norms: dict = None):
        counts, outputs = {}, {}
        items = hgraph.items() if isinstance(hgraph, dict) else hgraph
        for (sty, ety, dty), graph in items:
            if norms:
                res = self.convs[ety](graph, norms[str((sty, ety, dty))], (xs[sty], xs[dty]))
            else:
                res = self.convs[ety](graph, (xs[sty], xs[dty]))
            counts[dty] = counts.get(dty, 0) + 1
            outputs[dty] = res if dty not in outputs else outputs[dty] + res
        return {dty: res / counts[dty] for dty, res in outputs.items()}


class StitchedRGCNConv(nn.Module):
    """HeteroGraphConv over GCNLayers (norm = 1/in_degree per relation) for ONE destination type in one kernel pass:
    the relations are stitched into a segmented CSR (stitch_csr), every edge carries 1/(in-degree of its row within
    its relation), and out = reduce_r mean_{relation r}(x_r W_r^T + b_r).  reduce="mean" divides by the number of
    relations as the reference does (model.py:169-170); reduce="sum" adds the per-relation means."""

    def __init__(self, relations, in_features: int, out_features: int, reduce: str = "mean"):
        """relations: list of (edge type name, Block) that share the destination type."""
        nn.Module.__init__(self)
        assert reduce in ("mean", "sum")
        self.names = [name for name, _ in relations]
        self.fcs = nn.ModuleDict({name: nn.Linear(in_features, out_features) for name in self.names})
        self.reduce = reduce
        blocks = [blk for _, blk in relations]
        self.n_src = [blk.size[1] for blk in blocks]
        self.block = stitch_csr(blocks)
        self._weights = None

    def _graph(self, device, n_cols):
        if self.block.adj_sparse[0].device != device:
            self.block.to(device)
            self._weights = None
        g = ops.prepared(self.block.adj_sparse[0], self.block.adj_sparse[1], n_cols, ops.STITCH_MASK)
        if self._weights is None:
            self._weights = g.segment_mean_weights()
        return g

    def forward(self, xs: dict):
        """xs maps edge type name -> source features [n_src_r, in_features]."""
        h = torch.cat([self.fcs[name](xs[name]) for name in self.names])
        g = self._graph(h.device, h.size(0))
        out = _AggregateFunction.apply(h, g, self._weights)
        return out / len(self.names) if self.reduce == "mean" else out
