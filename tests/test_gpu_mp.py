"""The executing message-passing DSL (yitu_b200.xgnn_h.mp): layers written against the reference's DSL calls
(Fn.copy_u / u_add_v / edge_softmax / u_mul_e / aggregate_sum on a Graph) must give the results and gradients of the
operator-level layers and of dense float64 algebra, through the fused kernels and through the generic fallbacks."""
import numpy as np
import pytest
import torch
from torch import nn

from conftest import random_csr

pytestmark = pytest.mark.gpu


def _graph(indptr, indices, n_src):
    from yitu_b200.xgnn_h import mp
    return mp.Graph.from_csr(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(), n_src)


def _dense(indptr, indices, n_src):
    n_dst = len(indptr) - 1
    a = torch.zeros(n_dst, n_src, dtype=torch.float64)
    a[np.repeat(np.arange(n_dst), np.diff(indptr)), indices] = 1.0
    return a.cuda()


def _close(a, b, tol=2e-5):
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).abs().max()) <= tol * (float(b.abs().max()) + 1e-30)


class DslGCN(nn.Module):
    """Sum aggregation of a linear map, scaled per destination: the DSL calls of a GCN layer."""

    def __init__(self, fin, fout):
        super().__init__()
        self.fc = nn.Linear(fin, fout)

    def forward(self, graph, norm, x):
        from yitu_b200.xgnn_h import mp
        h = self.fc(x)
        graph.src_node['u'] = h.view(-1, 1, h.size(-1))
        graph.message_func(mp.Fn.copy_u('u', 'm'))
        graph.reduce_func(mp.Fn.aggregate_sum('m', 'v'))
        return norm * graph.dst_node['v'].squeeze(1)


class DslGAT(nn.Module):
    """Attention aggregation through the DSL; slope selects the LeakyReLU between score and softmax."""

    def __init__(self, fin, fout, heads, slope=0.2):
        super().__init__()
        self.heads, self.fout = heads, fout
        self.linear_q = nn.Linear(heads * fout, heads)
        self.linear_k = nn.Linear(heads * fout, heads)
        self.linear_v = nn.Linear(fin, heads * fout)
        self.act = nn.LeakyReLU(negative_slope=slope) if slope is not None else None

    def forward(self, graph, x_src, x_dst=None):
        from yitu_b200.xgnn_h import mp
        h_src = self.linear_v(x_src)
        h_dst = h_src if x_dst is None else self.linear_v(x_dst)
        graph.src_node['q'] = self.linear_q(h_dst)
        graph.dst_node['k'] = self.linear_k(h_src)
        graph.src_node['u'] = h_src.view(-1, self.heads, self.fout)
        graph.message_func(mp.Fn.u_add_v('k', 'q', 'e'))
        graph.edge['coeff'] = self.act(graph.edge['e']) if self.act is not None else graph.edge['e']
        graph.message_func(mp.Fn.edge_softmax('coeff', 'attn'))
        graph.message_func(mp.Fn.u_mul_e('u', 'attn', 'm'))
        graph.reduce_func(mp.Fn.aggregate_sum('m', 'v'))
        return torch.mean(graph.dst_node['v'], dim=1)


def _dense_gat(layer, a, x_src, x_dst, slope):
    """float64 dense statement of DslGAT."""
    p = {k: v.detach().double() for k, v in layer.named_parameters()}
    h_src = x_src.double() @ p['linear_v.weight'].t() + p['linear_v.bias']
    h_dst = x_dst.double() @ p['linear_v.weight'].t() + p['linear_v.bias']
    q = h_dst @ p['linear_q.weight'].t() + p['linear_q.bias']       # [n_dst, H]
    k = h_src @ p['linear_k.weight'].t() + p['linear_k.bias']       # [n_src, H]
    s = q[:, None, :] + k[None, :, :]                                # [n_dst, n_src, H]
    if slope is not None:
        s = torch.nn.functional.leaky_relu(s, slope)
    s = s.masked_fill(a[:, :, None] == 0, float('-inf'))
    w = torch.softmax(s, dim=1)
    w = torch.nan_to_num(w, nan=0.0)
    v = h_src.view(-1, layer.heads, layer.fout)
    return torch.einsum('dsh,shf->dhf', w, v).mean(1)


def test_dsl_gcn_matches_operator_layer_and_dense():
    from yitu_b200.nn import GCNLayer
    rng = np.random.default_rng(0)
    n = 300
    indptr, indices = random_csr(rng, n, n, density=0.04, empty_rows=False)
    g = _graph(indptr, indices, n)
    a = _dense(indptr, indices, n)
    dsl, op = DslGCN(16, 12).cuda(), GCNLayer(16, 12).cuda()
    op.load_state_dict(dsl.state_dict())
    x = torch.randn(n, 16, device="cuda", requires_grad=True)
    y = dsl(g, g.right_norm(), x)
    y.sum().backward()
    gx = x.grad.clone()
    x.grad = None
    y2 = op(g, g.right_norm(), x)
    y2.sum().backward()
    assert _close(y, y2) and _close(gx, x.grad)
    w, b = dsl.fc.weight.detach().double(), dsl.fc.bias.detach().double()
    assert _close(y, g.right_norm().double() * (a @ (x.detach().double() @ w.t() + b)))


@pytest.mark.parametrize("slope", [0.2, 0.05, None])
def test_dsl_gat_fused_and_generic_paths_match_dense(slope):
    """slope 0.2 takes the fused kernel; other slopes and no activation take the generic edge evaluation."""
    rng = np.random.default_rng(1)
    n, H, Fo = 200, 4, 8
    indptr, indices = random_csr(rng, n, n, density=0.06, empty_rows=False)
    g = _graph(indptr, indices, n)
    a = _dense(indptr, indices, n)
    layer = DslGAT(10, Fo, H, slope).cuda()
    x = torch.randn(n, 10, device="cuda", requires_grad=True)
    y = layer(g, x)
    y.sum().backward()
    xd = x.detach().double().requires_grad_()
    yd = _dense_gat(layer, a, xd, xd, slope)
    assert _close(y, yd, 5e-5)
    yd.sum().backward()
    assert _close(x.grad, xd.grad, 1e-4)


def test_dsl_gat_matches_operator_layer_with_gradients():
    from yitu_b200.nn import GATLayer
    rng = np.random.default_rng(2)
    n, H, Fo = 260, 8, 32
    indptr, indices = random_csr(rng, n, n, density=0.05, empty_rows=False)
    g = _graph(indptr, indices, n)
    dsl, op = DslGAT(20, Fo, H).cuda(), GATLayer(20, Fo, H).cuda()
    op.load_state_dict(dsl.state_dict())
    x = torch.randn(n, 20, device="cuda", requires_grad=True)
    w_out = torch.randn(n, Fo, device="cuda")
    (dsl(g, x) * w_out).sum().backward()
    got = [x.grad.clone()] + [p.grad.clone() for p in dsl.parameters()]
    x.grad = None
    (op(g, x) * w_out).sum().backward()
    ref = [x.grad.clone()] + [p.grad.clone() for p in op.parameters()]
    for u, v in zip(got, ref):
        assert _close(u, v, 5e-5)


def test_dsl_bipartite_block_and_edge_values():
    from yitu_b200 import graph_ext
    rng = np.random.default_rng(3)
    n_dst, n_src, H, Fo = 120, 210, 2, 16
    indptr, indices = random_csr(rng, n_dst, n_src, density=0.05, empty_rows=False)
    g = _graph(indptr, indices, n_src)
    a = _dense(indptr, indices, n_src)
    layer = DslGAT(12, Fo, H).cuda()
    xs, xd = torch.randn(n_src, 12, device="cuda"), torch.randn(n_dst, 12, device="cuda")
    y = layer(g, xs, xd)
    assert y.shape == (n_dst, Fo)
    assert _close(y, _dense_gat(layer, a, xs, xd, 0.2), 5e-5)
    # the symbolic attention can be asked for its values: they are the sddmm operator's
    attn = g.edge['attn'].materialize()
    ref = graph_ext.sddmm_forward(g.blk.adj_sparse[0], g.blk.adj_sparse[1], g.src_node['q'].detach().unsqueeze(0).contiguous(),
                                  g.dst_node['k'].detach().contiguous())
    assert attn.shape == (len(indices), H) and _close(attn, ref)


def test_dsl_generic_reduction_and_hetero_container():
    from yitu_b200.xgnn_h import Block, mp
    rng = np.random.default_rng(4)
    n_dst, n_src = 90, 140
    indptr, indices = random_csr(rng, n_dst, n_src, density=0.08)
    g = _graph(indptr, indices, n_src)
    a = _dense(indptr, indices, n_src)
    # a two-dimensional source value goes through the edge-by-edge path
    x = torch.randn(n_src, 6, device="cuda")
    g.src_node['x'] = x
    g.message_func(mp.Fn.copy_u('x', 'm'))
    g.reduce_func(mp.Fn.aggregate_sum('m', 'y'))
    assert _close(g.dst_node['y'], a @ x.double())
    with pytest.raises(KeyError):
        g.message_func(mp.Fn.copy_u('missing', 'm'))
    with pytest.raises(RuntimeError):
        g.reduce_func({'func': 'aggregate_max', 'e': 'm', 'out': 'y'})
    blk = Block([n_dst, n_src], [torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda()])
    h = mp.HeteroGraph.from_blocks({("paper", "cites", "author"): blk, ("author", "writes", "author"): g})
    assert [k for k, _ in h] == [("paper", "cites", "author"), ("author", "writes", "author")]
    assert h.etypes == ["cites", "writes"] and h.rel2idx[("author", "writes", "author")] == 1
    assert h.nty2num["paper"] == n_src and all(isinstance(v, mp.Graph) for _, v in h)
