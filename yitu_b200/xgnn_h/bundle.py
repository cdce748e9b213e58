"""GEMMBundleFunction — interface of YiTu_GNN/YiTu_H/xgnn_h/bundle.py:6-26: two bias-free linears that share their
input, evaluated as one batched GEMM (graph_ext.b2gemm); the two bias arguments are accepted and unused, as there."""
from torch import autograd

from .. import graph_ext


class GEMMBundleFunction(autograd.Function):
    """(x, w_1, w_2, b_1, b_2) -> (x w_1^T, x w_2^T)."""

    @staticmethod
    def forward(ctx, x, w_1, w_2, b_1, b_2):
        ctx.save_for_backward(x, w_1, w_2)
        outputs = graph_ext.b2gemm(x, w_1, w_2)
        return outputs[0], outputs[1]

    @staticmethod
    def backward(ctx, grad_1, grad_2):
        x, w_1, w_2 = ctx.saved_tensors
        grads = graph_ext.b2gemm_backward(x, w_1, w_2, grad_1.contiguous(), grad_2.contiguous())
        return grads[0], grads[1], grads[2], None, None
