"""Drop-in for the reference extension module `YiTu_GNN.YiTu_GNN_kernel`
(ccsrc/kernel/YiTu_GNN.cpp:247-258): same function names, argument order, return containers and input
checks, with every aggregation running in libyitu_b200.so.

The neighbour-group arguments (part_pointers, part2Node, partSize, dimWorker, warpPerBlock) describe the
reference kernel's own schedule; they are validated like the reference validates them and otherwise unused.
The dense X*W products stay torch GEMMs, as in the reference (torch::mm, YiTu_GNN_kernel.cu:276,471-472).

BACKWARD_USES_FORWARD_CSR: the reference's backward kernels aggregate d_output with the FORWARD CSR
(YiTu_GNN_kernel.cu:448-466, :733-745), which is the gradient only when the adjacency is symmetric.  The
default here is the true transpose (identical on symmetric graphs); set the flag to reproduce the reference
on directed graphs.
"""
import ctypes as C

import torch

from . import ops
from ._lib import W_NODE, W_NONE, check, lib

BACKWARD_USES_FORWARD_CSR = False


def _graph_inputs(row_pointers, column_index, part_pointers, part2Node):
    ops.require_cuda(row_pointers, "row_pointers")
    ops.require_cuda(column_index, "column_index")
    ops.require_cuda(part_pointers, "part_pointers")
    ops.require_cuda(part2Node, "part2Node")


def _prepared(row_pointers, column_index, n_nodes):
    return ops.prepared(row_pointers, column_index, n_nodes)


def _aggregate(g, x, transpose, **kw):
    if transpose and not BACKWARD_USES_FORWARD_CSR:
        return ops.spmm(g.t_prepared(), x, **kw)
    return ops.spmm(g, x, **kw)


def SAG(input, row_pointers, column_index, degrees, part_pointers, part2Node, partSize, dimWorker, warpPerBlock):
    """Unweighted neighbour sum A*X (ccsrc/kernel/YiTu_GNN_kernel.cu:104-257; `degrees` is accepted, unused)."""
    ops.require_cuda(input, "input")
    ops.require_cuda(degrees, "degrees")
    _graph_inputs(row_pointers, column_index, part_pointers, part2Node)
    g = _prepared(row_pointers, column_index, input.size(0))
    return ops.spmm(g, input, mode=W_NONE)


def forward(input, weight, row_pointers, column_index, degrees, part_pointers, part2Node, partSize, dimWorker,
            warpPerBlock):
    """[A_hat (X W)], A_hat[i,j] = degrees[i]*degrees[j] on stored (i,j) (YiTu_GNN_kernel.cu:264-415)."""
    ops.require_cuda(input, "input")
    ops.require_cuda(weight, "weight")
    ops.require_cuda(degrees, "degrees")
    _graph_inputs(row_pointers, column_index, part_pointers, part2Node)
    tmp = torch.mm(input, weight)
    g = _prepared(row_pointers, column_index, input.size(0))
    return [ops.spmm(g, tmp, mode=W_NODE, norm_dst=degrees, norm_src=degrees)]


def backward(d_output, X, W, row_pointers, column_index, degrees, part_pointers, part2Node, partSize, dimWorker,
             warpPerBlock):
    """[d_input, d_weight] (YiTu_GNN_kernel.cu:422-475): d' = A_hat^T d_output; d' W^T; X^T d'."""
    ops.require_cuda(d_output, "d_output")
    ops.require_cuda(X, "X")
    ops.require_cuda(W, "W")
    ops.require_cuda(degrees, "degrees")
    _graph_inputs(row_pointers, column_index, part_pointers, part2Node)
    g = _prepared(row_pointers, column_index, X.size(0))
    d_prime = _aggregate(g, d_output, True, mode=W_NODE, norm_dst=degrees, norm_src=degrees)
    return [torch.mm(d_prime, W.transpose(0, 1)), torch.mm(X.transpose(0, 1), d_prime)]


def forward_gin(input, weight, row_pointers, column_index, epsilon, part_pointers, part2Node, partSize, dimWorker,
                warpPerBlock):
    """[output, agg]: agg = epsilon * (A X); output = agg W (YiTu_GNN_kernel.cu:563-694)."""
    ops.require_cuda(input, "input")
    ops.require_cuda(weight, "weight")
    _graph_inputs(row_pointers, column_index, part_pointers, part2Node)
    g = _prepared(row_pointers, column_index, input.size(0))
    agg = ops.spmm(g, input, mode=W_NONE, alpha=float(epsilon))
    return [torch.mm(agg, weight), agg]


def backward_gin(d_output, X, W, row_pointers, column_index, epsilon, part_pointers, part2Node, partSize, dimWorker,
                 warpPerBlock):
    """[d_input, d_weight] (YiTu_GNN_kernel.cu:701-823); X is the aggregate saved by forward_gin."""
    ops.require_cuda(d_output, "d_output")
    ops.require_cuda(X, "X")
    ops.require_cuda(W, "W")
    _graph_inputs(row_pointers, column_index, part_pointers, part2Node)
    d_weight = torch.mm(X.transpose(0, 1), d_output)
    d_input_prime = torch.mm(d_output, W.transpose(0, 1))
    g = _prepared(row_pointers, column_index, X.size(0))
    d_input = _aggregate(g, d_input_prime, True, mode=W_NONE, alpha=float(epsilon))
    return [d_input, d_weight]


def build_part(partSize, indptr):
    """[partPtr, part2Node] as float32 CPU tensors, bit-identical to the reference
    (ccsrc/kernel/YiTu_GNN.cpp:203-245), from a CPU int32 row-pointer tensor."""
    if indptr.is_cuda or indptr.dtype != torch.int32 or indptr.dim() != 1:
        raise RuntimeError("build_part expects a 1-D CPU int32 row-pointer tensor")
    indptr = indptr.contiguous()
    L = lib()
    n = indptr.numel() - 1
    parts = L.yitu_build_part_count_host(int(partSize), C.c_void_p(indptr.data_ptr()), n)
    if parts < 0:
        raise RuntimeError("build_part: bad partSize")
    part_ptr = torch.zeros(parts + 1, dtype=torch.float32)
    part2node = torch.zeros(parts, dtype=torch.float32)
    check(L.yitu_build_part_host(int(partSize), C.c_void_p(indptr.data_ptr()), n, C.c_void_p(part_ptr.data_ptr()),
                                 C.c_void_p(part2node.data_ptr())))
    return [part_ptr, part2node]
