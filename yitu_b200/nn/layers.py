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
    """y = act(row_scale * (A x) + bias) with fixed per-edge weights (or none): one SpMM with a fused epilogue
    forward; backward one element-wise pass (activation derivative and row scale) and the transposed SpMM."""

    @staticmethod
    def forward(ctx, x, graph, weights, row_scale=None, bias=None, activation=None):
        ctx.graph, ctx.weights, ctx.row_scale, ctx.activation = graph, weights, row_scale, activation
        ctx.has_bias = bias is not None
        mode = ops.W_NONE if weights is None else ops.W_EDGE
        y = ops.spmm(graph, x.contiguous(), mode=mode, edge_values=weights, row_scale=row_scale,
                     bias=None if bias is None else bias.detach().contiguous(), activation=activation)
        if activation is not None:
            ctx.save_for_backward(y)
        return y

    @staticmethod
    def backward(ctx, grad_out):
        g, w = ctx.graph, ctx.weights
        grad_out = grad_out.contiguous()
        if ctx.activation is not None or ctx.row_scale is not None:
            y = ctx.saved_tensors[0] if ctx.activation is not None else None
            grad_bias = None
            if ctx.has_bias:  # the bias sits inside the row scale's reach only through the activation
                grad_pre = ops.epilogue_grad(y, grad_out, None, ctx.activation) if y is not None else grad_out
                grad_bias = grad_pre.reshape(-1, grad_pre.size(-1)).sum(0)
                grad_agg = ops.epilogue_grad(None, grad_pre, ctx.row_scale, None) if ctx.row_scale is not None else grad_pre
            else:
                grad_agg = ops.epilogue_grad(y, grad_out, ctx.row_scale, ctx.activation)
        else:
            grad_agg = grad_out
            grad_bias = grad_out.reshape(-1, grad_out.size(-1)).sum(0) if ctx.has_bias else None
        gt = g.t_prepared()
        if w is None:
            grad_x = ops.spmm(gt, grad_agg, mode=ops.W_NONE)
        else:
            grad_x = ops.spmm(gt, grad_agg, mode=ops.W_EDGE, edge_values=w, edge_perm=g.transpose()[2])
        return grad_x, None, None, None, grad_bias, None


def aggregate(block, x, weights=None, index_mask=0, row_scale=None, bias=None, activation=None):
    """Differentiable sum (or fixed-weight sum) of source rows per destination row; x is [n_src, D].  row_scale
    [n_dst], bias [D] and activation (None / "relu" / "elu") are applied in the kernel's epilogue:
    act(row_scale * sum + bias)."""
    g = ops.prepared(block.adj_sparse[0], block.adj_sparse[1], x.size(0), index_mask)
    return _AggregateFunction.apply(x, g, weights, row_scale, bias, activation)


class GCNLayer(nn.Module):
    """norm * (A (x W^T + b)) — model.py:7-30; `norm` is the per-destination 1/in_degree column (mp.py:165-167).
    The multiplication by norm runs in the aggregation kernel's epilogue, and so does `activation` (the ReLU the
    reference's GCNModel applies between layers, model.py:46-49) when one is given."""

    def __init__(self, in_features: int, out_features: int, activation: str = None):
        nn.Module.__init__(self)
        self.fc = nn.Linear(in_features, out_features)
        self.activation = activation

    def forward(self, graph, norm, x):
        if isinstance(x, (list, tuple)):
            assert len(x) == 2
            x = x[0]
        blk = _block_of(graph)
        h = self.fc(x)
        n_dst = blk.adj_sparse[0].numel() - 1
        if norm.numel() == n_dst and norm.dtype == torch.float32 and not norm.requires_grad:
            return aggregate(blk, h, row_scale=norm.reshape(-1).contiguous(), activation=self.activation)
        out = torch.multiply(norm, aggregate(blk, h))
        return sparse._TORCH_ACT[self.activation](out)


class GATLayer(nn.Module):
    """mean over heads of softmax-weighted aggregation — model.py:61-106; `activation` fuses the ELU the
    reference's GATModel applies between layers (model.py:126-129)."""

    def __init__(self, in_features: int, out_features: int, n_heads: int, activation: str = None):
        nn.Module.__init__(self)
        self.n_heads, self.n_features, self.activation = n_heads, out_features, activation
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
        # mean over heads (and the optional activation) inside the aggregation kernel
        return sparse.fused_gat(_block_of(graph), q, k, h_src, head_mean=True, activation=self.activation)


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


class _LinearIntoFunction(autograd.Function):
    """h = [x_0 W_0^T + b_0 ; x_1 W_1^T + b_1 ; ...]: every relation's GEMM writes its rows of ONE buffer, the source
    feature matrix of the stitched graph — no concatenation pass over the results."""

    @staticmethod
    def forward(ctx, n_rel, *tensors):
        xs, ws, bs = tensors[:n_rel], tensors[n_rel:2 * n_rel], tensors[2 * n_rel:]
        rows = [x.size(0) for x in xs]
        h = torch.empty(sum(rows), ws[0].size(0), dtype=xs[0].dtype, device=xs[0].device)
        off = 0
        for x, w, b, n in zip(xs, ws, bs, rows):
            torch.addmm(b, x, w.t(), out=h[off:off + n])
            off += n
        ctx.n_rel, ctx.rows = n_rel, rows
        ctx.save_for_backward(*xs, *ws)
        return h

    @staticmethod
    def backward(ctx, grad_h):
        n_rel = ctx.n_rel
        saved = ctx.saved_tensors
        xs, ws = saved[:n_rel], saved[n_rel:]
        gxs, gws, gbs = [], [], []
        off = 0
        for i, (x, w, n) in enumerate(zip(xs, ws, ctx.rows)):
            g = grad_h[off:off + n]
            off += n
            gxs.append(g @ w if ctx.needs_input_grad[1 + i] else None)
            gws.append(g.t() @ x if ctx.needs_input_grad[1 + n_rel + i] else None)
            gbs.append(g.sum(0) if ctx.needs_input_grad[1 + 2 * n_rel + i] else None)
        return (None, *gxs, *gws, *gbs)


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
        fcs = [self.fcs[name] for name in self.names]
        h = _LinearIntoFunction.apply(len(fcs), *[xs[name] for name in self.names], *[fc.weight for fc in fcs],
                                      *[fc.bias for fc in fcs])
        g = self._graph(h.device, h.size(0))
        out = _AggregateFunction.apply(h, g, self._weights)
        return out / len(self.names) if self.reduce == "mean" else out


class StitchedRGATConv(nn.Module):
    """HeteroGraphConv over GATLayers (model.py:61-106,137-171) for ONE destination type over the stitched relations:
    the attention of every relation is normalised inside its own segment of the row (the segmented edge softmax of
    graph_ext.sddmm_forward, queries [n_relations, n_dst, H]) and one multi-head SpMM over the stitched graph adds the
    relations up; then the mean over heads and, with reduce="mean", the division by the number of relations.
    Each relation has its own linear_v / linear_q / linear_k, as one GATLayer per edge type has in the reference."""

    def __init__(self, relations, in_features: int, out_features: int, n_heads: int, reduce: str = "mean"):
        """relations: list of (edge type name, Block) that share the destination type."""
        nn.Module.__init__(self)
        assert reduce in ("mean", "sum")
        self.names = [name for name, _ in relations]
        self.n_heads, self.n_features, self.reduce = n_heads, out_features, reduce
        self.layers = nn.ModuleDict({name: GATLayer(in_features, out_features, n_heads) for name in self.names})
        self.block = stitch_csr([blk for _, blk in relations])

    def forward(self, xs: dict, x_dst):
        """xs maps edge type name -> source features [n_src_r, in_features]; x_dst [n_dst, in_features]."""
        if self.block.adj_sparse[0].device != x_dst.device:
            self.block.to(x_dst.device)
        hs, ks, qs = [], [], []
        for name in self.names:
            layer = self.layers[name]
            h_src = layer.linear_v(xs[name])
            hs.append(h_src)
            ks.append(layer.linear_k(h_src))
            qs.append(layer.linear_q(layer.linear_v(x_dst)))
        h = torch.cat(hs).view(-1, self.n_heads, self.n_features)
        attn = sparse.fused_gsddmm(self.block, torch.stack(qs).contiguous(), torch.cat(ks).contiguous())
        out = torch.mean(sparse.gspmm(self.block, attn, h.contiguous()), dim=1)
        return out / len(self.names) if self.reduce == "mean" else out
