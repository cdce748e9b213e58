"""Host logic of the executing message-passing DSL without a GPU: expression recording, pattern detection (what would
be sent to the fused kernels) and the generic edge-by-edge evaluation, which is plain torch and runs on the CPU."""
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
    assert torch.is_tensor(torch.exp(g.edge['e']))        # any other torch function forces the value
    with pytest.raises(RuntimeError):
        g.message_func({'func': 'v_sub_u', 'u': 'k', 'v': 'q', 'out': 'z'})
    assert mp.Fn.u_mul_e('u', 'attn', 'm') == {'func': 'u_mul_e', 'u': 'u', 'e': 'attn', 'out': 'm'}


@pytest.mark.parametrize("slope", [0.05, None])
def test_generic_evaluation_matches_dense_attention(slope):
    """Slopes other than the kernels' 0.2 are evaluated edge by edge with torch: same mathematics as dense softmax."""
    from yitu_b200.xgnn_h import mp
    rng = np.random.default_rng(1)
    n_dst, n_src, H, F = 25, 35, 3, 5
    indptr, indices = random_csr(rng, n_dst, n_src, density=0.25, empty_rows=False)
    g = _graph(indptr, indices, n_src)
    q = torch.randn(n_dst, H, dtype=torch.float64, requires_grad=True)
    k = torch.randn(n_src, H, dtype=torch.float64)
    x = torch.randn(n_src, H, F, dtype=torch.float64)
    g.src_node['q'], g.dst_node['k'], g.src_node['u'] = q, k, x
    g.message_func(mp.Fn.u_add_v('k', 'q', 'e'))
    g.edge['c'] = nn.LeakyReLU(slope)(g.edge['e']) if slope is not None else g.edge['e']
    g.message_func(mp.Fn.edge_softmax('c', 'attn'))
    # the attention, multiplied edge by edge and summed per destination, without any CUDA operator
    attn = g.edge['attn'].materialize()
    rows, cols = g._edge_endpoints()
    out = torch.zeros(n_dst, H, F, dtype=torch.float64).index_add_(0, rows, x[cols] * attn.unsqueeze(-1))
    a = torch.zeros(n_dst, n_src, dtype=torch.float64)
    a[np.repeat(np.arange(n_dst), np.diff(indptr)), indices] = 1.0
    s = q[:, None, :] + k[None, :, :]
    if slope is not None:
        s = torch.nn.functional.leaky_relu(s, slope)
    w = torch.softmax(s.masked_fill(a[:, :, None] == 0, float('-inf')), dim=1)
    ref = torch.einsum('dsh,shf->dhf', w, x)
    assert torch.allclose(out, ref, atol=1e-12)
    out.sum().backward()          # the generic path is differentiable through torch
    assert q.grad is not None and torch.isfinite(q.grad).all()


def test_generic_sum_of_two_dimensional_messages():
    from yitu_b200.xgnn_h import mp
    rng = np.random.default_rng(2)
    indptr, indices = random_csr(rng, 20, 30, density=0.2)
    g = _graph(indptr, indices, 30)
    x = torch.randn(30, 7)
    g.src_node['x'] = x
    g.message_func(mp.Fn.copy_u('x', 'm'))
    g.reduce_func(mp.Fn.aggregate_sum('m', 'y'))
    a = torch.zeros(20, 30)
    a[np.repeat(np.arange(20), np.diff(indptr)), indices] = 1.0
    assert torch.allclose(g.dst_node['y'], a @ x, atol=1e-5)
