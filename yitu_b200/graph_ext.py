"""Drop-in for the reference extension module `graph_ext` (YiTu_GNN/YiTu_H/src/entry.cpp:184-193): same
function names, argument order, return containers, dtype/rank checks.  Column indices may carry a segment
(relation) id in their top 8 bits (xgnn_h/block.py:52-54); columns are always masked with 0xffffff, as the
reference kernels do.

Additions that the reference does not have: gat_forward / gat_backward, the fused layer core.
"""
import torch

from . import ops
from ._lib import W_EDGE_HEAD

_F32, _I32 = torch.float32, torch.int32
_MASK = ops.STITCH_MASK
SLOPE = 0.2  # LeakyReLU slope fixed by the reference kernels (sddmm_cuda.cu:19)


def _need(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _graph(indptr, indices, n_cols):
    return ops.prepared(indptr, indices, n_cols, _MASK)


def b2gemm(x, w_a, w_b):
    """[x w_a^T, x w_b^T] (fc_cuda.cu:4-75, one strided-batched SGEMM there; a library GEMM here too)."""
    for t, n in ((x, "x"), (w_a, "w_a"), (w_b, "w_b")):
        ops.require_cuda(t, n, _F32)
    _need(x.dim() == 2 and w_a.dim() == 2 and w_a.shape == w_b.shape, "b2gemm: bad shapes")
    y = torch.matmul(x, torch.stack([w_a, w_b]).transpose(1, 2))
    return [y[0], y[1]]


def b2gemm_backward(x, w_a, w_b, grad_a, grad_b):
    """[dx, dw_a, dw_b] (fc_cuda.cu:77-215)."""
    for t, n in ((x, "x"), (w_a, "w_a"), (w_b, "w_b"), (grad_a, "grad_a"), (grad_b, "grad_b")):
        ops.require_cuda(t, n, _F32)
    dx = torch.addmm(torch.mm(grad_a, w_a), grad_b, w_b)
    return [dx, torch.mm(grad_a.t(), x), torch.mm(grad_b.t(), x)]


def spmm_forward(values, indptr, indices, features):
    """out[r,h,k] = sum_i values[i,h] * features[col_i,h,k] (spmm_cuda.cu:4-21,44-62)."""
    ops.require_cuda(values, "values", _F32)
    ops.require_cuda(indptr, "indptr", _I32)
    ops.require_cuda(indices, "indices", _I32)
    ops.require_cuda(features, "features", _F32)
    _need(values.dim() == 2 and indptr.dim() == 1 and indices.dim() == 1 and features.dim() == 3,
          "spmm_forward: bad ranks")
    g = _graph(indptr, indices, features.size(0))
    return ops.spmm(g, features, n_heads=features.size(1), mode=W_EDGE_HEAD, edge_values=values)


def spmm_backward(values, indptr, indices, features, grad_out):
    """[grad_a [E,H], grad_x [n_src,H,F]] (spmm_cuda.cu:24-42,64-86), no atomics."""
    ops.require_cuda(values, "values", _F32)
    ops.require_cuda(indptr, "indptr", _I32)
    ops.require_cuda(indices, "indices", _I32)
    ops.require_cuda(features, "features", _F32)
    ops.require_cuda(grad_out, "grad_out", _F32)
    _need(values.dim() == 2 and indptr.dim() == 1 and indices.dim() == 1 and features.dim() == 3 and
          grad_out.dim() == 3, "spmm_backward: bad ranks")
    g = _graph(indptr, indices, features.size(0))
    if ops.spmm_bwd_supported(features.size(1), features.size(2)):
        return list(ops.spmm_bwd(g, values, features, grad_out))  # both gradients from one pass over the transposed graph
    grad_a = ops.edge_dot(g, grad_out, features)
    _, _, t_perm = g.transpose()
    grad_x = ops.spmm(g.t_prepared(), grad_out, n_heads=grad_out.size(1), mode=W_EDGE_HEAD, edge_values=values,
                      edge_perm=t_perm)
    return [grad_a, grad_x]


def sddmm_forward(indptr, indices, query, key):
    """attn [E,H]: per-(row, segment) softmax of LeakyReLU(query[seg,row,h] + key[col,h]) (sddmm_cuda.cu:5-33)."""
    ops.require_cuda(indptr, "indptr", _I32)
    ops.require_cuda(indices, "indices", _I32)
    ops.require_cuda(query, "query", _F32)
    ops.require_cuda(key, "key", _F32)
    _need(indptr.dim() == 1 and indices.dim() == 1 and query.dim() == 3 and key.dim() == 2, "sddmm_forward: bad ranks")
    _need(query.size(-1) == key.size(-1), "sddmm_forward: head counts differ")
    _need(query.size(1) == indptr.size(0) - 1, "sddmm_forward: query rows != graph rows")
    g = _graph(indptr, indices, key.size(0))
    return ops.edge_softmax_fwd(g, query, key, SLOPE)


def sddmm_backward(indptr, indices, query, key, attn_values, grad_out):
    """[grad_query, grad_key] (sddmm_cuda.cu:36-67,91-118)."""
    ops.require_cuda(indptr, "indptr", _I32)
    ops.require_cuda(indices, "indices", _I32)
    for t, n in ((query, "query"), (key, "key"), (attn_values, "attn_values"), (grad_out, "grad_out")):
        ops.require_cuda(t, n, _F32)
    _need(query.dim() == 3 and key.dim() == 2 and attn_values.dim() == 2 and grad_out.dim() == 2,
          "sddmm_backward: bad ranks")
    _need(query.size(-1) == key.size(-1) and indices.size(0) == attn_values.size(0) and
          attn_values.shape == grad_out.shape, "sddmm_backward: shapes differ")
    g = _graph(indptr, indices, key.size(0))
    gq, gk = ops.edge_softmax_bwd(g, query, key, attn_values, grad_out, SLOPE)
    return [gq, gk]


def hfused_forward(spmm_values, spmm_indptr, spmm_indices, spmm_features, sddmm_indptr, sddmm_indices, sddmm_query,
                   sddmm_key):
    """[spmm_out, attn]: an SpMM on one block and an independent SDDMM on another (hfused_cuda.cu:5-45,96-137).
    The reference fuses them horizontally into one launch; here they are two launches on the same stream."""
    _need(spmm_indptr.size(0) == sddmm_indptr.size(0), "hfused_forward: the two blocks need equal row counts")
    attn = sddmm_forward(sddmm_indptr, sddmm_indices, sddmm_query, sddmm_key)
    out = spmm_forward(spmm_values, spmm_indptr, spmm_indices, spmm_features)
    return [out, attn]


def hfused_backward(spmm_values, spmm_indptr, spmm_indices, spmm_features, spmm_grad, sddmm_indptr, sddmm_indices,
                    sddmm_query, sddmm_key, sddmm_attn, sddmm_grad):
    """[grad_query, grad_key] — the reference computes four gradients and returns these two
    (hfused_cuda.cu:139-187); hfused_backward_all returns all four."""
    return hfused_backward_all(spmm_values, spmm_indptr, spmm_indices, spmm_features, spmm_grad, sddmm_indptr,
                               sddmm_indices, sddmm_query, sddmm_key, sddmm_attn, sddmm_grad)[2:]


def hfused_backward_all(spmm_values, spmm_indptr, spmm_indices, spmm_features, spmm_grad, sddmm_indptr, sddmm_indices,
                        sddmm_query, sddmm_key, sddmm_attn, sddmm_grad):
    grad_a, grad_x = spmm_backward(spmm_values, spmm_indptr, spmm_indices, spmm_features, spmm_grad)
    grad_q, grad_k = sddmm_backward(sddmm_indptr, sddmm_indices, sddmm_query, sddmm_key, sddmm_attn, sddmm_grad)
    return [grad_a, grad_x, grad_q, grad_k]


# ------------------------------------------------------------------------------------------ fused GAT
def gat_supported(indptr, indices, n_heads, n_feats):
    return n_heads <= 32 and n_feats % 4 == 0 and n_heads * n_feats <= 512


def gat_forward(indptr, indices, query, key, features, head_mean=False, activation=None, keep_heads=True):
    """[out [n_dst,H,F], row_max [n_dst,H], row_sum [n_dst,H]]: sddmm_forward + spmm_forward in one pass, for an
    unstitched graph (every segment id 0).  query [n_dst,H], key [n_src,H], features [n_src,H,F].
    head_mean / activation fuse the layer's mean over heads (out [n_dst,F]) and the model's ReLU / ELU; with
    head_mean the list has a fourth entry, the per-head result the backward needs."""
    ops.require_cuda(indptr, "indptr", _I32)
    ops.require_cuda(indices, "indices", _I32)
    for t, n in ((query, "query"), (key, "key"), (features, "features")):
        ops.require_cuda(t, n, _F32)
    _need(query.dim() == 2 and key.dim() == 2 and features.dim() == 3, "gat_forward: bad ranks")
    g = ops.prepared(indptr, indices, features.size(0), 0)
    return list(ops.gat_fwd(g, query, key, features, SLOPE, head_mean, activation, keep_heads=keep_heads))


def gat_backward(indptr, indices, query, key, features, out, row_max, row_sum, grad_out, head_mean=False,
                 out_heads=None):
    """[grad_query, grad_key, grad_features] of gat_forward; grad_out is taken with respect to the values before
    the activation."""
    for t, n in ((query, "query"), (key, "key"), (features, "features"), (out, "out"), (row_max, "row_max"),
                 (row_sum, "row_sum"), (grad_out, "grad_out")):
        ops.require_cuda(t, n, _F32)
    g = ops.prepared(indptr, indices, features.size(0), 0)
    return list(ops.gat_bwd(g, query, key, features, out, row_max, row_sum, grad_out, SLOPE, head_mean, out_heads))
