"""Autograd operators of YiTu_GNN/YiTu_H/xgnn_h/sparse.py:7-120 over the B200 kernels, plus the fused GAT
operator the reference lowers to two calls (fused_gsddmm then gspmm)."""
import torch
from torch import autograd

from .. import graph_ext, ops
from . import block


class GSPMMFunction(autograd.Function):
    @staticmethod
    def forward(ctx, adj_sparse, adj_values, x):
        y = graph_ext.spmm_forward(adj_values, adj_sparse[0], adj_sparse[1], x)
        ctx.adj_sparse = adj_sparse
        ctx.save_for_backward(adj_values, x)
        return y

    @staticmethod
    def backward(ctx, grad_out):
        values, x = ctx.saved_tensors
        assert len(ctx.needs_input_grad) == 3
        assert ctx.needs_input_grad[0] is False
        grad_a, grad_x = graph_ext.spmm_backward(values, ctx.adj_sparse[0], ctx.adj_sparse[1], x,
                                                 grad_out.contiguous())
        return None, grad_a, grad_x


class GSPMMSumFunction(autograd.Function):
    """gspmm with edge=None: the reference materialises a [E,H] tensor of ones and multiplies by it
    (xgnn_h/sparse.py:43-48); the same sum is taken here with the unweighted kernel, forward and transposed."""

    @staticmethod
    def forward(ctx, adj_sparse, x):
        g = ops.prepared(adj_sparse[0], adj_sparse[1], x.size(0), ops.STITCH_MASK)
        ctx.graph = g
        return ops.spmm(g, x.contiguous(), n_heads=x.size(1), mode=ops.W_NONE)

    @staticmethod
    def backward(ctx, grad_out):
        return None, ops.spmm(ctx.graph.t_prepared(), grad_out.contiguous(), n_heads=grad_out.size(1), mode=ops.W_NONE)


def gspmm(block: block.Block, edge: torch.Tensor, x: torch.Tensor):
    assert x.dim() == 3
    if edge is None:
        return GSPMMSumFunction.apply(block.adj_sparse, x)
    return GSPMMFunction.apply(block.adj_sparse, edge, x)


class GSDDMMFunction(autograd.Function):
    @staticmethod
    def forward(ctx, adj_sparse, query, key):
        attn_values = graph_ext.sddmm_forward(adj_sparse[0], adj_sparse[1], query, key)
        ctx.adj_sparse = adj_sparse
        ctx.save_for_backward(query, key, attn_values)
        return attn_values

    @staticmethod
    def backward(ctx, grad_out):
        query, key, attn_values = ctx.saved_tensors
        assert len(ctx.needs_input_grad) == 3
        assert ctx.needs_input_grad[0] is False
        grad_query, grad_key = graph_ext.sddmm_backward(ctx.adj_sparse[0], ctx.adj_sparse[1], query, key,
                                                        attn_values, grad_out.contiguous())
        return None, grad_query, grad_key


def fused_gsddmm(block: block.Block, query: torch.Tensor, key: torch.Tensor):
    if query.dim() == 2:
        query = query.unsqueeze(0)
    return GSDDMMFunction.apply(block.adj_sparse, query, key)


class HFUSEDFunction(autograd.Function):
    @staticmethod
    def forward(ctx, spmm_sparse, spmm_values, spmm_x, sddmm_sparse, sddmm_query, sddmm_key):
        spmm_out, attn_values = graph_ext.hfused_forward(spmm_values, spmm_sparse[0], spmm_sparse[1], spmm_x,
                                                         sddmm_sparse[0], sddmm_sparse[1], sddmm_query, sddmm_key)
        ctx.spmm_sparse = spmm_sparse
        ctx.sddmm_sparse = sddmm_sparse
        ctx.save_for_backward(sddmm_query, sddmm_key)
        return spmm_out, attn_values

    @staticmethod
    def backward(ctx, grad_out):
        raise NotImplementedError  # as in the reference (sparse.py:108-110)


def hfused_spddmm(spmm_block: block.Block, spmm_values, spmm_x, sddmm_block: block.Block, sddmm_query, sddmm_key):
    if sddmm_query.dim() == 2:
        sddmm_query = sddmm_query.unsqueeze(0)
    return HFUSEDFunction.apply(spmm_block.adj_sparse, spmm_values, spmm_x, sddmm_block.adj_sparse, sddmm_query,
                                sddmm_key)


class FusedGATFunction(autograd.Function):
    """gspmm(fused_gsddmm(q, k), x) as one kernel per direction; no [E,H] attention tensor is kept.  With
    head_mean the layer's mean over heads (and an optional ReLU / ELU) is part of the same kernel, and the backward
    kernels read the [n_dst,F] gradient directly."""

    @staticmethod
    def forward(ctx, adj_sparse, query, key, x, head_mean=False, activation=None):
        # the per-head result of a head-mean forward is only written when a backward pass may follow
        keep = any(ctx.needs_input_grad[1:4])
        res = graph_ext.gat_forward(adj_sparse[0], adj_sparse[1], query, key, x, head_mean, activation, keep_heads=keep)
        out, row_max, row_sum = res[:3]
        ctx.adj_sparse, ctx.head_mean, ctx.activation = adj_sparse, head_mean, activation
        ctx.out_heads = res[3] if head_mean else None
        ctx.save_for_backward(query, key, x, out, row_max, row_sum)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        query, key, x, out, row_max, row_sum = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        if ctx.activation is not None:
            grad_out = ops.epilogue_grad(out, grad_out, None, ctx.activation)
        gq, gk, gx = graph_ext.gat_backward(ctx.adj_sparse[0], ctx.adj_sparse[1], query, key, x, out, row_max,
                                            row_sum, grad_out, ctx.head_mean, ctx.out_heads)
        return None, gq, gk, gx, None, None


_TORCH_ACT = {None: lambda t: t, "relu": torch.relu, "elu": torch.nn.functional.elu}


def fused_gat(block: block.Block, query: torch.Tensor, key: torch.Tensor, x: torch.Tensor, head_mean: bool = False,
              activation: str = None):
    """Attention + aggregation of a GAT layer (YiTu_GNN/YiTu_H/test/common/model.py:96-105) for an unstitched
    block: query [n_dst,H], key [n_src,H], x [n_src,H,F] -> [n_dst,H,F]; with head_mean the layer's
    torch.mean(dim=1) (model.py:106) and the model's activation (model.py:126-129) are fused: -> [n_dst,F].
    Shapes the fused kernels do not cover, and stitched blocks (relation ids in the top index bits, which the fused
    kernels would take for column ids), take the two-operator route."""
    assert x.dim() == 3 and query.dim() == 2
    if activation not in _TORCH_ACT:
        raise RuntimeError("activation must be None, 'relu' or 'elu', got %r" % (activation,))
    if not block.is_stitched() and graph_ext.gat_supported(block.adj_sparse[0], block.adj_sparse[1], x.size(1),
                                                            x.size(2)):
        return FusedGATFunction.apply(block.adj_sparse, query.contiguous(), key.contiguous(), x.contiguous(),
                                      head_mean, activation)
    out = gspmm(block, fused_gsddmm(block, query, key), x)
    if head_mean:
        out = torch.mean(out, dim=1)
    return _TORCH_ACT[activation](out)
