"""GCNConv over the B200 kernels: interface of YiTu_GNN/nn/GCNConv.py:13-76.

`inputInfo` is the reference's InputInfo object (YiTu_GNN/utils/input_info.py:25-56); the fields read are
row_pointers, column_index, degrees, partPtr, part2Node, partSize, dimWorker, warpPerBlock.
"""
import math

import torch

from .. import YiTu_GNN_kernel


class GNNAFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, weight, inputInfo):
        ctx.save_for_backward(X, weight)
        ctx.inputInfo = inputInfo
        return YiTu_GNN_kernel.forward(
            X, weight, inputInfo.row_pointers, inputInfo.column_index, inputInfo.degrees, inputInfo.partPtr,
            inputInfo.part2Node, inputInfo.partSize, inputInfo.dimWorker, inputInfo.warpPerBlock)[0]

    @staticmethod
    def backward(ctx, d_output):
        X, weight = ctx.saved_tensors
        info = ctx.inputInfo
        d_input, d_weight = YiTu_GNN_kernel.backward(
            d_output.contiguous(), X, weight, info.row_pointers, info.column_index, info.degrees, info.partPtr,
            info.part2Node, info.partSize, info.dimWorker, info.warpPerBlock)
        return d_input, d_weight, None


class GCNConv(torch.nn.Module):
    """out = A_hat (X W) with A_hat[i,j] = degrees[i]*degrees[j]; weights ~ U(+-1/sqrt(output_dim))."""

    def __init__(self, input_dim, output_dim):
        super().__init__()
        self.weights = torch.nn.Parameter(torch.randn(input_dim, output_dim))
        self.reset_parameters()

    def reset_parameters(self):
        bound = 1.0 / math.sqrt(self.weights.size(1))
        self.weights.data.uniform_(-bound, bound)

    def forward(self, X, inputInfo):
        return GNNAFunction.apply(X, self.weights, inputInfo)
