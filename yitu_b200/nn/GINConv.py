"""GINConv over the B200 kernels: interface of YiTu_GNN/nn/GINConv.py:7-77 (aggregate, scale by epsilon,
then the dense update; the attribute keeps the reference's spelling `eplison`)."""
import math

import torch

from .. import YiTu_GNN_kernel


class GNNAFunction_GIN(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, weight, inputInfo, eplison):
        X_prime, X_agg = YiTu_GNN_kernel.forward_gin(
            X, weight, inputInfo.row_pointers, inputInfo.column_index, eplison, inputInfo.partPtr,
            inputInfo.part2Node, inputInfo.partSize, inputInfo.dimWorker, inputInfo.warpPerBlock)
        ctx.save_for_backward(X_agg, weight)
        ctx.inputInfo = inputInfo
        ctx.eplison = eplison
        return X_prime

    @staticmethod
    def backward(ctx, d_output):
        X_agg, weight = ctx.saved_tensors
        info = ctx.inputInfo
        d_input, d_weight = YiTu_GNN_kernel.backward_gin(
            d_output.contiguous(), X_agg, weight, info.row_pointers, info.column_index, ctx.eplison, info.partPtr,
            info.part2Node, info.partSize, info.dimWorker, info.warpPerBlock)
        return d_input, d_weight, None, None


class GINConv(torch.nn.Module):
    def __init__(self, input_dim, output_dim):
        super().__init__()
        self.weights = torch.nn.Parameter(torch.randn(input_dim, output_dim))
        self.eplison = 0.5
        self.reset_parameters()

    def reset_parameters(self):
        bound = 1.0 / math.sqrt(self.weights.size(1))
        self.weights.data.uniform_(-bound, bound)

    def forward(self, X, inputInfo):
        return GNNAFunction_GIN.apply(X, self.weights, inputInfo, self.eplison)
