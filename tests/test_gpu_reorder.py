"""Community reordering on the GPU: the permutation must equal the CPU restatement bit for bit (integer arithmetic
throughout), the drop-in `rabbit.reorder` must return the relabelled edge list, and aggregation over the reordered
graph must be the same function up to the renumbering."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from test_reorder_cpu import planted_graph

pytestmark = pytest.mark.gpu


def _edges(src, dst):
    return torch.from_numpy(np.stack([src, dst]).astype(np.int32)).cuda()


def _cases():
    rng = np.random.default_rng(0)
    n = 4000
    yield "random", n, rng.integers(0, n, 30000), rng.integers(0, n, 30000)
    src, dst, _ = planted_graph(rng, 1 << 13, 64, 10, 0.9)
    yield "planted", 1 << 13, src, dst
    # duplicates, self-loops, isolated nodes (ids above 3000 never appear)
    s = rng.integers(0, 3000, 20000)
    d = np.where(rng.random(20000) < 0.1, s, rng.integers(0, 3000, 20000))
    yield "duplicates_selfloops_isolated", 3500, np.concatenate([s, s[:5000]]), np.concatenate([d, d[:5000]])
    # a hub joined to everything plus a ring
    ring = np.arange(2000)
    yield "hub_and_ring", 2001, np.concatenate([ring, np.full(2000, 2000)]), np.concatenate([(ring + 1) % 2000, ring])
    yield "single_edge", 10, np.array([3]), np.array([7])


@pytest.mark.parametrize("name,n,src,dst", list(_cases()), ids=[c[0] for c in _cases()])
def test_reorder_bit_exact_against_cpu_restatement(oracle, name, n, src, dst):
    from yitu_b200 import rabbit
    ref, ref_levels, ref_top = oracle.reorder_communities(n, src, dst)
    got, levels, top = rabbit.reorder_ids(_edges(src, dst), n)
    assert (levels, top) == (ref_levels, ref_top)
    assert np.array_equal(got.cpu().numpy(), ref)


@pytest.mark.parametrize("max_levels", [1, 2, 5])
def test_reorder_level_cap(oracle, max_levels):
    from yitu_b200 import rabbit
    rng = np.random.default_rng(5)
    n = 2000
    src, dst = rng.integers(0, n, 16000), rng.integers(0, n, 16000)
    ref, ref_levels, _ = oracle.reorder_communities(n, src, dst, max_levels=max_levels)
    got, levels, _ = rabbit.reorder_ids(_edges(src, dst), n, max_levels=max_levels)
    assert levels == ref_levels == max_levels
    assert np.array_equal(got.cpu().numpy(), ref)


def test_reorder_empty_and_loops_only():
    from yitu_b200 import rabbit
    empty = torch.zeros((2, 0), dtype=torch.int32, device="cuda")
    ids, levels, top = rabbit.reorder_ids(empty, 7)
    assert ids.tolist() == list(range(7)) and levels == 0 and top == 7
    loops = torch.tensor([[1, 2, 2], [1, 2, 2]], dtype=torch.int32, device="cuda")
    ids, levels, _ = rabbit.reorder_ids(loops, 4)
    assert ids.tolist() == [0, 1, 2, 3] and levels == 0
    assert rabbit.reorder(empty).shape == (2, 0)


def test_rabbit_reorder_matches_reference_interface(oracle):
    """rabbit.reorder(IntTensor [2,E]) -> IntTensor [2,E] of renumbered edges, CPU in / CPU out as the reference
    (ccsrc/reorder/reorder.cpp:235-290); CUDA in / CUDA out as well."""
    from yitu_b200 import rabbit
    rng = np.random.default_rng(6)
    src, dst, _ = planted_graph(rng, 4096, 64, 8, 0.9)
    n = int(max(src.max(), dst.max())) + 1
    ref, _, _ = oracle.reorder_communities(n, src, dst)
    ei = torch.from_numpy(np.stack([src, dst]).astype(np.int32))
    out = rabbit.reorder(ei)
    assert not out.is_cuda and out.dtype == torch.int32 and out.shape == ei.shape
    assert np.array_equal(out.numpy(), np.stack([ref[src], ref[dst]]))
    out_gpu = rabbit.reorder(ei.cuda())
    assert out_gpu.is_cuda and torch.equal(out_gpu.cpu(), out)
    with pytest.raises(RuntimeError):
        rabbit.reorder(ei.long())
    with pytest.raises(RuntimeError):
        rabbit.reorder(ei[0])
    with pytest.raises(RuntimeError):  # ids beyond n_nodes are refused, not read out of bounds
        rabbit.reorder_ids(ei.cuda(), n - 5)


def test_edge_span_and_decider_rule():
    from yitu_b200 import rabbit
    rng = np.random.default_rng(7)
    src, dst, _ = planted_graph(rng, 1 << 14, 128, 8, 0.95)
    ei = _edges(src, dst)
    span = rabbit.avg_edge_span(ei)
    assert span == pytest.approx(np.abs(src.astype(np.int64) - dst).mean(), rel=1e-12)
    assert rabbit.should_reorder(ei, 1 << 14)
    after = rabbit.reorder(ei)
    assert rabbit.avg_edge_span(after) < 0.3 * span


def test_aggregation_commutes_with_the_renumbering(oracle):
    """SpMM over the reordered graph, on features permuted the same way, is the original result permuted."""
    from yitu_b200 import ops, rabbit
    rng = np.random.default_rng(8)
    n, d = 1 << 12, 64
    src, dst, _ = planted_graph(rng, n, 64, 8, 0.9)
    ei = _edges(src, dst)
    new_id, _, _ = rabbit.reorder_ids(ei, n)
    x = torch.randn(n, d, device="cuda")
    ip, ix = ops.coo_to_csr(ei[0], ei[1], n, n, self_loops=True)
    y = ops.spmm(ops.PreparedGraph(ip, ix, n), x)
    ei2 = rabbit.relabel(ei, new_id)
    ip2, ix2 = ops.coo_to_csr(ei2[0].contiguous(), ei2[1].contiguous(), n, n, self_loops=True)
    x2 = torch.empty_like(x)
    x2[new_id.long()] = x
    y2 = ops.spmm(ops.PreparedGraph(ip2, ix2, n), x2)
    assert_close(y2[new_id.long()].cpu().numpy(), y.cpu().numpy(), what="spmm after reordering")
