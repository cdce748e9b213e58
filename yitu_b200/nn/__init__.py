"""Layers of YiTu_GNN/nn that sit on the custom aggregation kernels (YiTu_GNN/nn/__init__.py:1-10)."""
from .GCNConv import GCNConv, GNNAFunction
from .GINConv import GINConv, GNNAFunction_GIN

__all__ = ["GCNConv", "GNNAFunction", "GINConv", "GNNAFunction_GIN"]
