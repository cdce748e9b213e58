"""GEMMBundleFunction — interface of YiTu_GNN/YiTu_H/xgnn_h/bundle.py:6-26 (two linears sharing an input)."""
from torch import autograd

from .. import graph_ext


class GEMMBundleFunction(autograd.Function):
    @staticmethod
    def forward(ctx, x, w_1, w_2, b_1, b_2):
        y_1, y_2 = graph_ext.b2gemm(x, w_1, w_2)
        ctx.save_for_backward(x, w_1, w_2)
        return y_1, y_2

    @staticmethod
    def backward(ctx, grad_1, grad_2):
        x, w_1, w_2 = ctx.saved_tensors
        dx, dw_1, dw_2 = graph_ext.b2gemm_backward(x, w_1, w_2, grad_1.contiguous(), grad_2.contiguous())
        return dx, dw_1, dw_2, None, None
