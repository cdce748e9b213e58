"""yitu_b200 — B200-native (sm_100a) message-passing kernels behind the operator API of CGCL-codes/YiTu.

    yitu_b200.YiTu_GNN_kernel   drop-in for the extension module of ccsrc/kernel (GCN / GIN / SAG)
    yitu_b200.graph_ext         drop-in for the extension module of YiTu_H/src (SpMM / SDDMM / fused GAT)
    yitu_b200.nn                GCNConv, GINConv (YiTu_GNN/nn)
    yitu_b200.xgnn_h            Block, stitch_csr, sparse.gspmm / fused_gsddmm / fused_gat, bundle
    yitu_b200.rabbit            drop-in for the reordering extension of ccsrc/reorder (reorder)
    yitu_b200.distributed       row-partitioned multi-GPU SpMM
    yitu_b200.graphs            seeded synthetic graphs

The compute lives in libyitu_b200.so (C ABI in include/yitu_b200.h); build it with `python -m yitu_b200.build`.
"""
__version__ = "0.1.0"


def install_as_reference_modules():
    """Register the drop-in modules under the names the reference's Python code imports
    (`from YiTu_GNN import YiTu_GNN_kernel`, `from YiTu_GNN import rabbit`, `import graph_ext`), so its wrappers
    run unmodified."""
    import sys
    import types

    from . import YiTu_GNN_kernel, graph_ext, rabbit
    sys.modules["graph_ext"] = graph_ext
    pkg = sys.modules.get("YiTu_GNN")
    if pkg is None:
        pkg = types.ModuleType("YiTu_GNN")
        pkg.__path__ = []
        sys.modules["YiTu_GNN"] = pkg
    pkg.YiTu_GNN_kernel = YiTu_GNN_kernel
    sys.modules["YiTu_GNN.YiTu_GNN_kernel"] = YiTu_GNN_kernel
    pkg.rabbit = rabbit
    sys.modules["YiTu_GNN.rabbit"] = rabbit
