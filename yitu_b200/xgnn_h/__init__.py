"""Operator level of YiTu_H's xgnn_h package (YiTu_GNN/YiTu_H/xgnn_h/{block,sparse,bundle}.py) over the
B200 kernels.  The tracing compiler above it (mp / ast / optimizer / stitcher / executor) is not rebuilt; it
lowers to exactly these operators."""
from . import block, bundle, sparse
from .block import Block, stitch_csr

__all__ = ["block", "bundle", "sparse", "Block", "stitch_csr"]
