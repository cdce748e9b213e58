"""Host logic of the executing message-passing DSL without a GPU: expression recording, pattern detection (what would
be sent to the fused kernels), the errors for expressions no kernel evaluates, and the deferral of reductions on the
graphs of a HeteroGraph (what would be stitched)."""
import numpy as np
import pytest
import torch
from torch import nn

from conftest import random_csr


def _graph(indptr, indices, n_src):
    from yitu_b200.xgnn_h import mp
    return mp.Graph.from_csr(torch.from_numpy(indptr), torch.from_numpy(indices), n_src)


def test_expressions_are_recorded_and_patterns_detected():
    from yitu_b200.xgnn_h import mp
    rng = np.random.default_rng(0)
    indptr, indices = random_csr(rng, 30, 40, density=0.2)
    g = _graph(indptr, indices, 40)
    assert g.num_dst_nodes() == 30 and g.num_src_nodes() == 40 and g.num_edges() == len(indices)
    assert g.right_norm().shape == (30, 1)
    g.src_node['q'] = torch.randn(30, 2)
    g.dst_node['k'] = torch.randn(40, 2)
    g.src_node['u'] = torch.randn(40, 2, 4)
    assert g.num_features() == 4
    g.message_func(mp.Fn.u_add_v('k', 'q', 'e'))
    assert isinstance(g.edge['e'], mp.EdgeExpr) and g.edge['e'].op == 'u_add_v'
    g.edge['c'] = nn.LeakyReLU(0.2)(g.edge['e'])
    assert g.edge['c'].op == 'leaky_relu' and g.edge['c'].args['slope'] == pytest.approx(0.2)
    g.message_func(mp.Fn.edge_softmax('c', 'attn'))
    key, query = g.edge['attn'].is_gat_attention()
    assert key is g.dst_node['k'] and query is g.src_node['q']
    g.edge['c2'] = nn.LeakyReLU(0.1)(g.edge['e'])       # another slope: not the fused kernel's pattern
    g.message_func(mp.Fn.edge_softmax('c2', 'attn2'))
    assert g.edge['attn2'].is_gat_attention() is None
    g.message_func(mp.Fn.edge_softmax('e', 'attn3'))     # no activation at all
    assert g.edge['attn3'].is_gat_attention() is None
    with pytest.raises(RuntimeError):
        g.message_func({'func': 'v_sub_u', 'u': 'k', 'v': 'q', 'out': 'z'})
    assert mp.Fn.u_mul_e('u', 'attn', 'm') == {'func': 'u_mul_e', 'u': 'u', 'e': 'attn', 'out': 'm'}


def test_expressions_without_a_kernel_raise_and_name_themselves():
    """No fallback: an expression that no kernel evaluates is a RuntimeError naming the expression."""
    from yitu_b200.xgnn_h import mp
    rng = np.random.default_rng(1)
    indptr, indices = random_csr(rng, 25, 35, density=0.25)
    g = _graph(indptr, indices, 35)
    g.src_node['q'], g.dst_node['k'], g.src_node['u'] = torch.randn(25, 3), torch.randn(35, 3), torch.randn(35, 3, 5)
    g.message_func(mp.Fn.u_add_v('k', 'q', 'e'))
    g.edge['c'] = nn.LeakyReLU(0.05)(g.edge['e'])           # not the slope the kernels fix
    g.message_func(mp.Fn.edge_softmax('c', 'attn'))
    with pytest.raises(RuntimeError, match=r"edge_softmax\(e=leaky_relu\(e=u_add_v"):
        g.edge['attn'].materialize()
    with pytest.raises(RuntimeError, match="no kernel evaluates"):
        torch.exp(g.edge['e'])                                # a bare per-edge sum has no kernel either
    g.message_func(mp.Fn.u_mul_e('u', 'attn', 'm'))
    with pytest.raises(RuntimeError, match="no kernel evaluates"):
        g.reduce_func(mp.Fn.aggregate_sum('m', 'v'))
    with pytest.raises(RuntimeError, match=r"aggregate_sum\(u_add_v"):
        g.reduce_func(mp.Fn.aggregate_sum('e', 'v'))


class _DslGCN(nn.Module):
    """The DSL calls of the reference's GCNLayer (YiTu_GNN/YiTu_H/test/common/model.py:15-30)."""

    def __init__(self, fin, fout):
        super().__init__()
        self.fc = nn.Linear(fin, fout)

    def forward(self, graph, norm, x):
        from yitu_b200.xgnn_h import mp
        h = self.fc(x[0] if isinstance(x, (list, tuple)) else x)
        graph.src_node['u'] = h.view(size=[-1, 1, h.size(-1)])
        graph.message_func(mp.Fn.copy_u('u', 'm'))
        graph.reduce_func(mp.Fn.aggregate_sum('m', 'v'))
        return torch.multiply(norm, torch.squeeze(graph.dst_node['v'], dim=1))


def test_reductions_of_a_hetero_graph_are_deferred_and_joined_per_destination_type():
    """Recording only (no kernel runs on the CPU): on graphs of a HeteroGraph reduce_func returns a deferred result;
    squeeze, the norm multiplication, the sum over the relations of a destination type and the division by their
    number are absorbed, so that one stitched pass can compute them."""
    from yitu_b200.nn import HeteroGraphConv
    from yitu_b200.xgnn_h import Block, mp
    rng = np.random.default_rng(3)
    sizes = {"a": 30, "b": 20}
    rels = {("a", "aa", "a"): random_csr(rng, 30, 30, 0.2), ("b", "ba", "a"): random_csr(rng, 30, 20, 0.2),
            ("a", "ab", "b"): random_csr(rng, 20, 30, 0.2)}
    h = mp.HeteroGraph.from_blocks({k: Block([sizes[k[2]], sizes[k[0]]], [torch.from_numpy(ip), torch.from_numpy(ix)])
                                    for k, (ip, ix) in rels.items()})
    assert all(g.hetero is h and g.relation == k for k, g in h)
    conv = HeteroGraphConv({k[1]: _DslGCN(6, 4) for k in rels})
    xs = {t: torch.randn(n, 6) for t, n in sizes.items()}
    norms = {str(k): torch.rand(sizes[k[2]], 1) for k in rels}
    out = conv(h, xs, norms)
    assert set(out) == {"a", "b"}
    da, db = out["a"], out["b"]
    assert isinstance(da, mp.DeferredAgg) and isinstance(db, mp.DeferredAgg)
    assert len(da.terms) == 2 and da.post == ("squeeze1",) and da.alpha == pytest.approx(0.5)
    assert [t.graph.relation for t in da.terms] == [("a", "aa", "a"), ("b", "ba", "a")]
    assert all(t.kind == "sum" and t.scale is not None and t.scale.shape == (30,) for t in da.terms)
    assert torch.equal(da.terms[1].scale, norms[str(("b", "ba", "a"))].reshape(-1))
    assert len(db.terms) == 1 and db.alpha == 1.0 and tuple(db.shape) == (20, 4) and tuple(da.shape) == (30, 4)
    # results of different destination types cannot be joined
    h.stitch = False   # eager mode would call the kernels at once: on the CPU that fails loudly, it does not defer
    with pytest.raises(Exception):
        conv(h, xs, norms)
