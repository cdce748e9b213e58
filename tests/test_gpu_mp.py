"""The executing message-passing DSL (yitu_b200.xgnn_h.mp): layers written against the reference's DSL calls
(Fn.copy_u / u_add_v / edge_softmax / u_mul_e / aggregate_sum on a Graph) must give the results and gradients of the
operator-level layers and of dense float64 algebra; expressions without a kernel raise; the reference's own hetero
models run unchanged and reach one stitched aggregation per destination type."""
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
def test_dsl_gat_fused_path_matches_dense_and_other_slopes_raise(slope):
    """slope 0.2 takes the fused kernel; other slopes and no activation have no kernel and say so."""
    rng = np.random.default_rng(1)
    n, H, Fo = 200, 4, 8
    indptr, indices = random_csr(rng, n, n, density=0.06, empty_rows=False)
    g = _graph(indptr, indices, n)
    a = _dense(indptr, indices, n)
    layer = DslGAT(10, Fo, H, slope).cuda()
    x = torch.randn(n, 10, device="cuda", requires_grad=True)
    if slope != 0.2:
        with pytest.raises(RuntimeError, match="no kernel evaluates"):
            layer(g, x)
        return
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
    # a two-dimensional source value is a one-head aggregation
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


def _hetero_case(rng, dev):
    """Three node types, six relations; type "a" is reached by three of them, "b" by two, "c" by one."""
    from yitu_b200.xgnn_h import Block, mp
    sizes = {"a": 150, "b": 90, "c": 60}
    keys = [("a", "aa", "a"), ("b", "ba", "a"), ("c", "ca", "a"), ("a", "ab", "b"), ("c", "cb", "b"), ("a", "ac", "c")]
    blocks, norms, dense = {}, {}, {}
    for k in keys:
        ip, ix = random_csr(rng, sizes[k[2]], sizes[k[0]], density=0.08)
        deg = np.maximum(np.diff(ip), 1).astype(np.float32)
        blocks[k] = Block([sizes[k[2]], sizes[k[0]]], [torch.from_numpy(ip).to(dev), torch.from_numpy(ix).to(dev)],
                          right_norm=torch.from_numpy(1.0 / deg).to(dev).unsqueeze(-1))
        norms[str(k)] = blocks[k].right_norm
        dense[k] = _dense(ip, ix, sizes[k[0]])
    return sizes, keys, mp.HeteroGraph.from_blocks(blocks, nty2num=sizes), norms, dense


def _count_aggregations(monkeypatch):
    """Counts calls of the aggregation kernels' entry points (SpMM, edge softmax, fused GAT)."""
    from yitu_b200 import ops
    calls = {"spmm": 0, "edge_softmax_fwd": 0, "gat_fwd": 0}
    for name in list(calls):
        real = getattr(ops, name)

        def counted(*a, _real=real, _name=name, **kw):
            calls[_name] += 1
            return _real(*a, **kw)
        monkeypatch.setattr(ops, name, counted)
    return calls


@pytest.fixture()
def reference_models():
    """The reference's own layer / model file (staged by `make -C oracle ref_py`), imported over THIS package's
    executing DSL: its `from xgnn_h import mp` resolves to yitu_b200.xgnn_h."""
    import importlib
    import os
    import sys
    import yitu_b200.xgnn_h as our_xgnn_h
    staged = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "py")
    if not os.path.exists(os.path.join(staged, "reference_model.py")):
        pytest.skip("the reference's model file is not staged (make -C oracle ref_py)")
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "xgnn_h" or k.startswith("xgnn_h.")}
    sys.modules["xgnn_h"] = our_xgnn_h
    sys.path.insert(0, staged)
    try:
        yield importlib.import_module("reference_model")
    finally:
        sys.path.remove(staged)
        for k in ("xgnn_h", "reference_model"):
            sys.modules.pop(k, None)
        sys.modules.update(saved)


def test_reference_rgcn_model_is_stitched_automatically(reference_models, monkeypatch):
    """RGCNModel of the reference (HeteroGraphConv over GCNLayers, test/common/model.py:137-171,197-240), unmodified:
    each layer must run ONE aggregation per destination type over the stitched relations, keep every relation's own
    norm, and agree with the one-kernel-per-relation evaluation and with dense float64 algebra."""
    dev = torch.device("cuda")
    rng = np.random.default_rng(11)
    sizes, keys, h, norms, dense = _hetero_case(rng, dev)
    torch.manual_seed(0)
    model = reference_models.RGCNModel(h, 12, 16, 5).to(dev).eval()
    xs = {t: torch.arange(n, device=dev) for t, n in sizes.items()}
    calls = _count_aggregations(monkeypatch)
    out = model(h, norms, xs)
    y = {t: torch.as_tensor(v + 0.0) for t, v in out.items()}     # first real use computes the deferred results
    assert set(y) == {"a", "b", "c"} and y["a"].shape == (150, 5) and y["b"].shape == (90, 5)
    assert calls["spmm"] == 6, "two layers x three destination types: one aggregation each, got %r" % calls
    (y["a"].sum() + y["b"].sum()).backward()
    grads = [p.grad.clone() for p in model.parameters() if p.grad is not None]
    model.zero_grad()
    h.stitch = False
    calls2 = _count_aggregations(monkeypatch)
    out2 = model(h, norms, xs)
    assert calls2["spmm"] == 12, "unstitched: one aggregation per relation and layer"
    for t in y:
        assert _close(y[t], out2[t])
    (out2["a"].sum() + out2["b"].sum()).backward()
    for g1, g2 in zip(grads, [p.grad for p in model.parameters() if p.grad is not None]):
        assert _close(g1, g2, 1e-4)
    # dense float64 statement of the first layer for destination type "a": mean over relations of norm_r * (A_r (x W_r^T + b_r))
    em = {t: model.em.embeds[t].weight.detach().double() for t in sizes}
    acc = 0
    for k in keys:
        if k[2] != "a":
            continue
        fc = model.i2h.convs[k[1]].fc
        acc = acc + norms[str(k)].double() * (dense[k] @ (em[k[0]] @ fc.weight.detach().double().t() + fc.bias.detach().double()))
    h.stitch = True
    first = model.i2h(h, {t: model.em.embeds[t].weight for t in sizes}, norms)
    assert _close(first["a"] + 0.0, acc / 3)


def test_reference_rgat_model_is_stitched_automatically(reference_models, monkeypatch):
    """RGATModel of the reference (HeteroGraphConv over GATLayers, model.py:61-106,243-285), unmodified: per layer and
    destination type one segmented edge softmax and one SpMM over the stitched relations."""
    dev = torch.device("cuda")
    rng = np.random.default_rng(12)
    sizes, keys, h, norms, dense = _hetero_case(rng, dev)
    torch.manual_seed(1)
    model = reference_models.RGATModel(h, 12, 8, 4, n_heads=4).to(dev).eval()
    xs = {t: torch.arange(n, device=dev) for t, n in sizes.items()}
    calls = _count_aggregations(monkeypatch)
    out = model(h, xs)
    y = {t: v + 0.0 for t, v in out.items()}
    # types "a" and "b": segmented softmax + SpMM over the stitched relations; type "c" has one relation: fused kernel
    assert calls["edge_softmax_fwd"] == 4 and calls["spmm"] == 4 and calls["gat_fwd"] == 2, calls
    (y["a"].sum() + y["b"].sum()).backward()
    grads = [p.grad.clone() for p in model.parameters() if p.grad is not None]
    model.zero_grad()
    h.stitch = False
    out2 = model(h, xs)
    for t in y:
        assert _close(y[t], out2[t], 5e-5)
    (out2["a"].sum() + out2["b"].sum()).backward()
    grads2 = [p.grad for p in model.parameters() if p.grad is not None]
    top = max(float(g.abs().max()) for g in grads2)
    for g1, g2 in zip(grads, grads2):
        # gradients that are zero by symmetry (a shift of all scores of a row leaves the softmax unchanged, so the
        # bias of linear_q gets none) hold rounding noise only: measured against the largest gradient instead
        assert float((g1 - g2).abs().max()) <= 2e-4 * max(float(g2.abs().max()), 1e-3 * top)


def test_stitched_graph_with_the_attention_pattern_takes_the_two_operator_route(monkeypatch):
    """A Graph over a stitched block (relation ids in the top index bits) must not reach the fused GAT kernels, which
    would take the packed ids for column numbers: the attention pattern runs as segmented softmax + SpMM."""
    from yitu_b200.xgnn_h import Block, mp, stitch_csr
    dev = torch.device("cuda")
    rng = np.random.default_rng(13)
    blocks = []
    for n_src in (40, 70):
        ip, ix = random_csr(rng, 50, n_src, density=0.1, empty_rows=False)
        blocks.append(Block([50, n_src], [torch.from_numpy(ip).to(dev), torch.from_numpy(ix).to(dev)]))
    g = mp.Graph(stitch_csr(blocks))
    H, Fo = 2, 8
    g.src_node['q'] = torch.randn(50, H, device=dev)
    g.dst_node['k'] = torch.randn(110, H, device=dev)
    g.src_node['u'] = torch.randn(110, H, Fo, device=dev)
    g.message_func(mp.Fn.u_add_v('k', 'q', 'e'))
    g.edge['c'] = nn.LeakyReLU(0.2)(g.edge['e'])
    g.message_func(mp.Fn.edge_softmax('c', 'attn'))
    g.message_func(mp.Fn.u_mul_e('u', 'attn', 'm'))
    calls = _count_aggregations(monkeypatch)
    g.reduce_func(mp.Fn.aggregate_sum('m', 'v'))
    assert calls["gat_fwd"] == 0 and calls["edge_softmax_fwd"] == 1 and calls["spmm"] == 1
    assert g.dst_node['v'].shape == (50, H, Fo) and torch.isfinite(g.dst_node['v']).all()
