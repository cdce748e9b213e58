"""Graph preparation on the device through the C ABI: edge list -> CSR (sort, dedup, self-loops), degree vectors,
device stitch_csr — bit-exact against scipy / the host routine / the CPU checker."""
import numpy as np
import pytest
import scipy.sparse as sp
import torch

from conftest import random_csr

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n_src,n_dst,n_edges,loops", [(1000, 1000, 20000, True), (700, 1300, 9000, False),
                                                       (5, 5, 0, True), (3, 4, 0, False), (65536, 65536, 1 << 20, False)])
@pytest.mark.parametrize("ptr", [torch.int32, torch.int64])
def test_coo_to_csr_matches_scipy(n_src, n_dst, n_edges, loops, ptr):
    from yitu_b200 import graphs, ops
    src, dst = graphs.rmat_edges(3, n_src, n_dst, n_edges) if n_edges else (torch.zeros(0, dtype=torch.int64),) * 2
    indptr, indices = ops.coo_to_csr(src.int().cuda(), dst.int().cuda(), n_src, n_dst, self_loops=loops, ptr_dtype=ptr)
    s, d = src.numpy(), dst.numpy()
    if loops:
        s, d = np.concatenate([s, np.arange(n_dst)]), np.concatenate([d, np.arange(n_dst)])
    m = sp.coo_matrix((np.ones(len(s)), (d, s)), shape=(n_dst, n_src)).tocsr()  # duplicates are summed: same pattern
    m.sort_indices()
    assert indptr.dtype == ptr
    assert np.array_equal(indptr.cpu().numpy().astype(np.int64), m.indptr.astype(np.int64))
    assert np.array_equal(indices.cpu().numpy(), m.indices)
    # and the torch-level generator path gives the same tables
    if n_edges:
        ip2, ix2 = graphs.csr_by_destination(src, dst, n_src, n_dst, self_loops=loops, ptr_dtype=ptr)
        assert torch.equal(ip2, indptr.cpu()) and torch.equal(ix2, indices.cpu())


def test_degree_norms():
    from yitu_b200 import ops
    rng = np.random.default_rng(1)
    indptr, _ = random_csr(rng, 500, 300, density=0.05, hubs=2, hub_deg=250)
    deg = np.maximum(np.diff(indptr), 1).astype(np.float32)
    for dt in (torch.int32, torch.int64):
        ip = torch.from_numpy(indptr).to(dt).cuda()
        # the reference: torch.sqrt(FloatTensor(max(deg, 1)))  (YiTu_GNN/data/dataset.py:131-133)
        assert torch.equal(ops.degree_norm(ip, ops.DEG_SQRT).cpu(), torch.sqrt(torch.from_numpy(deg)))
        np.testing.assert_allclose(ops.degree_norm(ip, ops.DEG_RSQRT).cpu().numpy(), 1 / np.sqrt(deg), rtol=1e-6)
        np.testing.assert_allclose(ops.degree_norm(ip, ops.DEG_INV).cpu().numpy(), 1 / deg, rtol=1e-6)


def test_device_stitch_matches_host(oracle):
    from yitu_b200.xgnn_h import Block, stitch_csr
    rng = np.random.default_rng(2)
    n_dst = 257
    blocks = []
    for b in range(5):
        ip, ix = random_csr(rng, n_dst, 40 + 17 * b, density=0.1, hubs=1, hub_deg=30)
        blocks.append((ip, ix, 40 + 17 * b))
    host = stitch_csr([Block([n_dst, c], [torch.from_numpy(a), torch.from_numpy(b)]) for a, b, c in blocks])
    dev = stitch_csr([Block([n_dst, c], [torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()]) for a, b, c in blocks])
    assert dev.adj_sparse[0].is_cuda and dev.size == host.size
    assert torch.equal(dev.adj_sparse[0].cpu(), host.adj_sparse[0]) and torch.equal(dev.adj_sparse[1].cpu(), host.adj_sparse[1])
    o_ip, o_ix, _ = oracle.stitch_csr(blocks)
    assert np.array_equal(dev.adj_sparse[0].cpu().numpy(), o_ip) and np.array_equal(dev.adj_sparse[1].cpu().numpy(), o_ix)
    big = Block([1, (1 << 24) + 5], [torch.tensor([0, 1], dtype=torch.int32).cuda(),
                                     torch.tensor([(1 << 24) + 3], dtype=torch.int32).cuda()])
    with pytest.raises(AssertionError):
        stitch_csr([big])
