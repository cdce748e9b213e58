"""Block (CSR holder) and stitch_csr — interface of YiTu_GNN/YiTu_H/xgnn_h/block.py:5-67."""
import ctypes as C
from typing import List

import torch

from .._lib import check, lib


class Block:
    """size = [n_dst, n_src]; adj_sparse = [indptr int32, indices int32]; optional right_norm = 1/in_degree."""

    def __init__(self, size: list, adj: list, right_norm=None, stitched=None):
        self.size = size
        self.adj_sparse = adj
        self.right_norm = right_norm
        # True when the column ids carry a relation id in their top 8 bits (stitch_csr sets it); None = not known
        # yet, found out once by is_stitched()
        self.stitched = stitched

    def is_stitched(self):
        """Whether any column id carries a segment id (bits 24..31).  stitch_csr marks its result; for a Block built
        from raw tensors the ids are inspected once (one device read) and the answer is kept."""
        if self.stitched is None:
            ix = self.adj_sparse[1]
            self.stitched = bool(ix.numel()) and bool((ix >> 24).ne(0).any())
        return self.stitched

    def to(self, device):
        self.adj_sparse = [self.adj_sparse[0].to(device), self.adj_sparse[1].to(device)]
        if self.right_norm is not None:
            self.right_norm = self.right_norm.to(device)
        return self

    def num_edges(self):
        assert self.adj_sparse[1].dim() == 1
        return self.adj_sparse[1].numel()

    def num_src_nodes(self):
        return self.size[1]

    def num_dst_nodes(self):
        assert self.adj_sparse[0].dim() == 1
        assert self.size[0] == self.adj_sparse[0].size(0) - 1
        return self.size[0]


def stitch_csr(block_list: List[Block]):
    """Pack up to 16 blocks with equal row counts into one segmented CSR: row r = row r of every block in
    turn, index = (block id << 24) + column + columns of the blocks before.  Same result as the reference's
    per-edge Python loop, computed by the library's host routine (result on the CPU, like there) or, when the block tables are CUDA
    tensors, by its device kernels (result on that GPU)."""
    rows = [blk.size[0] for blk in block_list]
    assert len(rows) <= 16
    assert min(rows) == max(rows)
    n_rows = rows[0]
    if all(blk.adj_sparse[0].is_cuda and blk.adj_sparse[1].is_cuda for blk in block_list):
        # tables already on a GPU: stitch there (the result stays on that device)
        from .. import ops
        try:
            ip, ix = ops.stitch_csr_device([blk.adj_sparse[0].to(torch.int32).contiguous() for blk in block_list],
                                           [blk.adj_sparse[1].to(torch.int32).contiguous() for blk in block_list],
                                           [blk.size[1] for blk in block_list])
        except RuntimeError as e:  # the reference asserts
            raise AssertionError(str(e))
        return Block(size=[n_rows, sum(blk.size[1] for blk in block_list)], adj=[ip, ix], stitched=len(block_list) > 1)
    ips = [blk.adj_sparse[0].to("cpu", torch.int32).contiguous() for blk in block_list]
    ids = [blk.adj_sparse[1].to("cpu", torch.int32).contiguous() for blk in block_list]
    n_cols = torch.tensor([blk.size[1] for blk in block_list], dtype=torch.int64)
    out_ip = torch.zeros(n_rows + 1, dtype=torch.int32)
    out_id = torch.zeros(sum(i.numel() for i in ids), dtype=torch.int32)
    PP = C.c_void_p * len(block_list)
    try:
        check(lib().yitu_stitch_csr_host(len(block_list), n_rows, PP(*[t.data_ptr() for t in ips]),
                                         PP(*[t.data_ptr() for t in ids]), C.c_void_p(n_cols.data_ptr()),
                                         C.c_void_p(out_ip.data_ptr()), C.c_void_p(out_id.data_ptr())))
    except RuntimeError as e:  # the reference asserts
        raise AssertionError(str(e))
    return Block(size=[n_rows, int(n_cols.sum())], adj=[out_ip, out_id], stitched=len(block_list) > 1)
