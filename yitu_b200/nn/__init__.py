"""Layers over the custom aggregation kernels: GCNConv / GINConv of YiTu_GNN/nn (YiTu_GNN/nn/__init__.py:1-10) and the
YiTu_H layers GCNLayer / GATLayer / HeteroGraphConv (YiTu_GNN/YiTu_H/test/common/model.py)."""
from .GCNConv import GCNConv, GNNAFunction
from .GINConv import GINConv, GNNAFunction_GIN
from .layers import GATLayer, GCNLayer, HeteroGraphConv, StitchedRGATConv, StitchedRGCNConv, aggregate

__all__ = ["GCNConv", "GNNAFunction", "GINConv", "GNNAFunction_GIN", "GATLayer", "GCNLayer", "HeteroGraphConv",
           "StitchedRGCNConv", "StitchedRGATConv", "aggregate"]
