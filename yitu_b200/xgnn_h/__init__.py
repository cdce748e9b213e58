"""Operator level of YiTu_H's xgnn_h package (YiTu_GNN/YiTu_H/xgnn_h/{block,sparse,bundle}.py) over the
B200 kernels, plus `mp`: the message-passing DSL (xgnn_h/mp.py) executing directly on those operators.  The tracing
compiler of the reference (ast / ir / optimizer / stitcher / executor) is not rebuilt; `mp` picks the same fused
operators by the shape of the expression at the point of reduction."""
from . import block, bundle, mp, sparse
from .block import Block, stitch_csr

__all__ = ["block", "bundle", "mp", "sparse", "Block", "stitch_csr"]
