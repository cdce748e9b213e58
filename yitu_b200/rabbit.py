"""Drop-in for the reference extension module `rabbit` (ccsrc/reorder/reorder.cpp:235-294, imported as
`from YiTu_GNN import rabbit` by YiTu_GNN/data/dataset.py:9,164): `reorder(edge_index)` returns the edge list with
node ids renumbered so that communities occupy contiguous id ranges.

The renumbering runs on the GPU (yitu_reorder_communities: Rabbit Order's merge criterion as synchronous rounds);
the reference runs the asynchronous Rabbit Order on the host cores, so the two permutations differ while both are
community orders.  `reorder_ids` and `avg_edge_span` are additions.
"""
import ctypes as C

import torch

from ._lib import check, lib

DEFAULT_MAX_LEVELS = 32


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _stream(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _device_edges(edge_index):
    if not isinstance(edge_index, torch.Tensor) or edge_index.dim() != 2 or edge_index.size(0) != 2:
        raise RuntimeError("edge_index must be a [2, E] tensor")
    if edge_index.dtype != torch.int32:
        raise RuntimeError("edge_index must be an IntTensor (int32), got %s" % edge_index.dtype)
    if not edge_index.is_contiguous():
        raise RuntimeError("edge_index must be contiguous")
    if edge_index.is_cuda:
        return edge_index
    if not torch.cuda.is_available():
        raise RuntimeError("rabbit.reorder runs on the GPU: no CUDA device is available")
    return edge_index.cuda()


def reorder_ids(edge_index, n_nodes=None, max_levels=DEFAULT_MAX_LEVELS):
    """(new_id int32 [n_nodes] on the GPU, levels built, communities at the coarsest level)."""
    ei = _device_edges(edge_index)
    n_edges = ei.size(1)
    if n_nodes is None:
        n_nodes = int(ei.max()) + 1 if n_edges else 0
    L = lib()
    dev = ei.device
    new_id = torch.empty(n_nodes, dtype=torch.int32, device=dev)
    n_levels, n_top = C.c_int32(0), C.c_int64(0)
    with torch.cuda.device(dev):
        ws_bytes = L.yitu_reorder_workspace_bytes(n_nodes, n_edges, max_levels)
        if ws_bytes < 0:
            raise RuntimeError("reorder: sizes out of range (n_nodes=%d, n_edges=%d)" % (n_nodes, n_edges))
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        check(L.yitu_reorder_communities(n_nodes, n_edges, _ptr(ei[0]), _ptr(ei[1]), max_levels, _ptr(new_id),
                                         C.byref(n_levels), C.byref(n_top), _ptr(ws), ws_bytes, _stream(dev)))
    return new_id, n_levels.value, n_top.value


def relabel(edge_index, new_id):
    """edge_index with both rows mapped through new_id (GPU tensors)."""
    out = torch.empty_like(edge_index)
    with torch.cuda.device(edge_index.device):
        check(lib().yitu_relabel_edges(edge_index.size(1), _ptr(edge_index[0]), _ptr(edge_index[1]), _ptr(new_id),
                                       _ptr(out[0]), _ptr(out[1]), _stream(edge_index.device)))
    return out


def reorder(edge_index, max_levels=DEFAULT_MAX_LEVELS):
    """The reference's entry point: IntTensor [2, E] in, renumbered IntTensor [2, E] out, on the device the input
    lives on (the reference takes and returns CPU tensors)."""
    ei = _device_edges(edge_index)
    new_id, _, _ = reorder_ids(ei, None, max_levels)
    out = relabel(ei, new_id)
    return out if edge_index.is_cuda else out.cpu()


def avg_edge_span(edge_index):
    """mean |src - dst|, the reference's avg_edgeSpan (YiTu_GNN/data/dataset.py:109)."""
    ei = _device_edges(edge_index)
    if ei.size(1) == 0:
        return 0.0
    total = torch.zeros(1, dtype=torch.int64, device=ei.device)
    with torch.cuda.device(ei.device):
        check(lib().yitu_edge_span_sum(ei.size(1), _ptr(ei[0]), _ptr(ei[1]), _ptr(total), _stream(ei.device)))
    return int(total) / ei.size(1)


def should_reorder(edge_index, n_nodes):
    """The reference decider's rule (YiTu_GNN/utils/input_info.py:131-140): sqrt(avg span) > sqrt(n) / 100."""
    return avg_edge_span(edge_index) ** 0.5 > n_nodes ** 0.5 / 100
