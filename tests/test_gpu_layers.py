"""Layer-level parity on the GPU: GCNConv/GINConv (YiTu_GNN/nn) and the YiTu_H layers (GCNLayer, GATLayer,
HeteroGraphConv, and its stitched one-pass form) against dense float64 torch algebra, outputs and gradients."""
import numpy as np
import pytest
import torch
from torch import nn

from conftest import random_csr

pytestmark = pytest.mark.gpu


def _dense(indptr, indices, n_src):
    n_dst = len(indptr) - 1
    a = torch.zeros(n_dst, n_src, dtype=torch.float64)
    a[np.repeat(np.arange(n_dst), np.diff(indptr)), indices] = 1.0
    return a.cuda()


def _block(indptr, indices, n_src):
    from yitu_b200.xgnn_h import Block
    return Block([len(indptr) - 1, n_src], [torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda()])


def _close(a, b, tol=2e-5):
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).abs().max()) <= tol * (float(b.abs().max()) + 1e-30)


class _Info:
    pass


def test_gcnconv_and_ginconv_autograd():
    from yitu_b200 import YiTu_GNN_kernel as K
    from yitu_b200.nn import GCNConv, GINConv
    rng = np.random.default_rng(0)
    n = 400
    dense = rng.random((n, n)) < 0.03
    dense = dense | dense.T
    np.fill_diagonal(dense, True)
    indptr = np.concatenate([[0], np.cumsum(dense.sum(1))]).astype(np.int32)
    indices = np.nonzero(dense)[1].astype(np.int32)
    info = _Info()
    info.row_pointers, info.column_index = torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda()
    deg = torch.from_numpy(np.diff(indptr).astype(np.float32))
    info.degrees = (1.0 / torch.sqrt(deg)).cuda()
    pp, p2n = K.build_part(32, torch.from_numpy(indptr))
    info.partPtr, info.part2Node = pp.int().cuda(), p2n.int().cuda()
    info.partSize, info.dimWorker, info.warpPerBlock = 32, 32, 2
    a = torch.from_numpy(dense.astype(np.float64)).cuda()
    nd = info.degrees.double()
    a_hat = nd[:, None] * a * nd[None, :]
    x = torch.randn(n, 24, device="cuda", requires_grad=True)
    w_out = torch.randn(n, 10, device="cuda")
    for layer, ref in ((GCNConv(24, 10).cuda(), lambda xx, ww: a_hat @ (xx @ ww)),
                       (GINConv(24, 10).cuda(), lambda xx, ww: (0.5 * (a @ xx)) @ ww)):
        y = layer(x, info)
        (y * w_out).sum().backward()
        gx, gw = x.grad.clone(), layer.weights.grad.clone()
        x.grad = None
        xd = x.detach().double().requires_grad_()
        wd = layer.weights.detach().double().requires_grad_()
        yd = ref(xd, wd)
        (yd * w_out.double()).sum().backward()
        assert _close(y, yd) and _close(gx, xd.grad) and _close(gw, wd.grad, 5e-5)


def test_gat_layer_matches_dense():
    from yitu_b200.nn import GATLayer
    rng = np.random.default_rng(1)
    n, H, F = 300, 4, 16
    indptr, indices = random_csr(rng, n, n, density=0.05, empty_rows=False)
    blk = _block(indptr, indices, n)
    layer = GATLayer(20, F, H).cuda()
    x = torch.randn(n, 20, device="cuda", requires_grad=True)
    y = layer(blk, x)
    y.sum().backward()
    gx = x.grad.clone()
    grads = {k: p.grad.clone() for k, p in layer.named_parameters()}
    # dense float64 restatement of model.py:75-106
    ld = GATLayer(20, F, H).cuda().double()
    ld.load_state_dict({k: v.double() for k, v in layer.state_dict().items()})
    xd = x.detach().double().requires_grad_()
    h = ld.linear_v(xd)
    q, k = ld.linear_q(h), ld.linear_k(h)
    a = _dense(indptr, indices, n)
    e = nn.functional.leaky_relu(q.unsqueeze(1) + k.unsqueeze(0), 0.2)
    e = torch.where(a.unsqueeze(-1) > 0, e, torch.full_like(e, -1e300)).permute(2, 0, 1)
    attn = torch.softmax(e, dim=-1) * a.unsqueeze(0)
    yd = torch.bmm(attn, h.view(n, H, F).transpose(0, 1)).transpose(0, 1).mean(dim=1)
    yd.sum().backward()
    assert _close(y, yd, 5e-5) and _close(gx, xd.grad, 1e-4)
    for kname, p in ld.named_parameters():
        assert _close(grads[kname], p.grad, 2e-4), kname


def test_hetero_conv_and_stitched_form_agree():
    from yitu_b200.nn import GCNLayer, HeteroGraphConv, StitchedRGCNConv
    rng = np.random.default_rng(2)
    n_dst, d_in, d_out = 250, 12, 64
    sizes = {"a": 90, "b": 140, "c": 60}
    hgraph, norms, xs, dense = {}, {}, {}, {}
    for name, n_src in sizes.items():
        indptr, indices = random_csr(rng, n_dst, n_src, density=0.08)
        hgraph[(name, "rel_" + name, "dst")] = _block(indptr, indices, n_src)
        deg = np.maximum(np.diff(indptr), 1).astype(np.float32)  # 1/in_degree; empty rows contribute 0 anyway
        norms[str((name, "rel_" + name, "dst"))] = torch.from_numpy(1.0 / deg).cuda().unsqueeze(-1)
        xs[name] = torch.randn(n_src, d_in, device="cuda", requires_grad=True)
        dense[name] = _dense(indptr, indices, n_src)
    xs["dst"] = torch.zeros(n_dst, d_in, device="cuda")
    conv = HeteroGraphConv({"rel_" + n: GCNLayer(d_in, d_out) for n in sizes}).cuda()
    y = conv(hgraph, xs, norms)["dst"]
    w_out = torch.randn(n_dst, d_out, device="cuda")
    (y * w_out).sum().backward()
    g1 = {n: xs[n].grad.clone() for n in sizes}
    gw1 = {n: conv.convs["rel_" + n].fc.weight.grad.clone() for n in sizes}

    stitched = StitchedRGCNConv([("rel_" + n, hgraph[(n, "rel_" + n, "dst")]) for n in sizes], d_in, d_out).cuda()
    for n in sizes:
        stitched.fcs["rel_" + n].load_state_dict(conv.convs["rel_" + n].fc.state_dict())
        xs[n].grad = None
    y2 = stitched({"rel_" + n: xs[n] for n in sizes})
    (y2 * w_out).sum().backward()
    assert _close(y2, y, 3e-5)
    for n in sizes:
        assert _close(xs[n].grad, g1[n], 5e-5)
        assert _close(stitched.fcs["rel_" + n].weight.grad, gw1[n], 1e-4)

    # dense float64: mean over relations of (1/in_degree) * A_r (x_r W_r^T + b_r)
    ref = 0
    for n in sizes:
        fc = conv.convs["rel_" + n].fc
        h = xs[n].detach().double() @ fc.weight.detach().double().T + fc.bias.detach().double()
        ref = ref + norms[str((n, "rel_" + n, "dst"))].double() * (dense[n] @ h)
    assert _close(y, ref / 3, 3e-5)
    summed = StitchedRGCNConv([("rel_" + n, hgraph[(n, "rel_" + n, "dst")]) for n in sizes], d_in, d_out,
                              reduce="sum").cuda()
    summed.load_state_dict(stitched.state_dict())
    assert _close(summed({"rel_" + n: xs[n] for n in sizes}), ref, 3e-5)


def test_hetero_gat_and_stitched_form_agree():
    """HeteroGraphConv over one GATLayer per relation against the stitched form (segmented softmax + one SpMM)."""
    from yitu_b200.nn import GATLayer, HeteroGraphConv, StitchedRGATConv
    rng = np.random.default_rng(5)
    n_dst, d_in, H, F = 180, 10, 4, 8
    sizes = {"a": 70, "b": 120, "c": 50}
    hgraph, xs = {}, {}
    for name, n_src in sizes.items():
        indptr, indices = random_csr(rng, n_dst, n_src, density=0.1, empty_rows=False)
        hgraph[(name, "rel_" + name, "dst")] = _block(indptr, indices, n_src)
        xs[name] = torch.randn(n_src, d_in, device="cuda", requires_grad=True)
    xs["dst"] = torch.randn(n_dst, d_in, device="cuda", requires_grad=True)
    conv = HeteroGraphConv({"rel_" + n: GATLayer(d_in, F, H) for n in sizes}).cuda()
    y = conv(hgraph, xs)["dst"]
    w_out = torch.randn(n_dst, F, device="cuda")
    (y * w_out).sum().backward()
    g1 = {n: xs[n].grad.clone() for n in xs}
    gw1 = {n: conv.convs["rel_" + n].linear_q.weight.grad.clone() for n in sizes}
    for n in xs:
        xs[n].grad = None
    stitched = StitchedRGATConv([("rel_" + n, hgraph[(n, "rel_" + n, "dst")]) for n in sizes], d_in, F, H).cuda()
    for n in sizes:
        stitched.layers["rel_" + n].load_state_dict(conv.convs["rel_" + n].state_dict())
    y2 = stitched({"rel_" + n: xs[n] for n in sizes}, xs["dst"])
    (y2 * w_out).sum().backward()
    assert y2.shape == (n_dst, F) and _close(y2, y, 3e-5)
    for n in xs:
        assert _close(xs[n].grad, g1[n], 1e-4)
    for n in sizes:
        assert _close(stitched.layers["rel_" + n].linear_q.weight.grad, gw1[n], 2e-4)


def test_two_layer_gcn_replays_from_a_cuda_graph():
    """The operators take the current stream and allocate only through torch, so a whole forward pass can be captured
    once and replayed (the small 2-layer GCN configuration is launch-bound when run eagerly)."""
    from yitu_b200 import YiTu_GNN_kernel as K, graphs
    from yitu_b200.nn import GCNConv
    n = 16384
    indptr, indices, norm = graphs.gcn_small()
    info = _Info()
    info.row_pointers, info.column_index, info.degrees = indptr.cuda(), indices.cuda(), norm.cuda()
    pp, p2n = K.build_part(32, indptr)
    info.partPtr, info.part2Node = pp.int().cuda(), p2n.int().cuda()
    info.partSize, info.dimWorker, info.warpPerBlock = 32, 32, 2
    l1, l2 = GCNConv(128, 64).cuda(), GCNConv(64, 16).cuda()
    x = graphs.randn_features(0, n, 128, device="cuda")

    def forward():
        with torch.no_grad():
            return l2(torch.relu(l1(x, info)), info)

    eager = forward()  # also builds the cached graph schedule, which synchronises and must precede the capture
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            forward()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = forward()
    x.copy_(graphs.randn_features(5, n, 128, device="cuda"))  # new input in the captured buffer
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(captured, forward()), "replay must reproduce the eager result for the new input"
    assert not torch.equal(captured, eager)


def test_fused_gat_forward_and_backward_replay_from_a_cuda_graph():
    """The fused GAT forward and its one-pass backward (hub schedules included) are plain stream work once the cached
    graph structures exist: capture both, replay on new inputs, compare with eager execution."""
    from yitu_b200 import ops
    rng = np.random.default_rng(9)
    n, H, F = 3000, 8, 32
    a = rng.random((n, n)) < 0.004
    a[5, rng.choice(n, size=1500, replace=False)] = True     # a hub row and a hub column: both schedules non-empty
    a[rng.choice(n, size=1500, replace=False), 7] = True
    indptr = np.concatenate([[0], np.cumsum(a.sum(1))]).astype(np.int32)
    indices = np.nonzero(a)[1].astype(np.int32)
    g = ops.PreparedGraph(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(), n)
    q, k = torch.randn(n, H, device="cuda"), torch.randn(n, H, device="cuda")
    x, grad = torch.randn(n, H, F, device="cuda"), torch.randn(n, H, F, device="cuda")

    def step():
        out, rmax, rsum = ops.gat_fwd(g, q, k, x)
        return (out,) + tuple(ops.gat_bwd(g, q, k, x, out, rmax, rsum, grad))

    step()  # builds the transposed graph and both hub schedules (synchronises): before the capture
    assert g.plan() is not None and g.t_prepared().plan() is not None
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    x.copy_(torch.randn(n, H, F, device="cuda"))
    q.copy_(torch.randn(n, H, device="cuda"))
    graph.replay()
    torch.cuda.synchronize()
    for got, ref in zip(captured, step()):
        assert torch.equal(got, ref)


def test_full_size_hetero_rgcn_sampled_rows_against_float64():
    """The heterogeneous benchmark configuration at full size (4 node types of 1 000 000 / 500 000 / 250 000 / 100 000
    nodes, 8 bipartite R-MAT relations x 4 M sampled edges, 64 features): per destination type ONE pass over the
    stitched relations gives sum_r mean_{edges of relation r}(x_r W_r^T + b_r) - the layer mathematics of
    YiTu_GNN/YiTu_H/test/common/model.py:15-30,142-171 with the sum instead of the division by the relation count.
    Sampled destination rows, among them the longest of every type, against float64 formed from the UNSTITCHED
    relation blocks."""
    from conftest import record_error
    from yitu_b200 import graphs
    from yitu_b200.nn.layers import StitchedRGCNConv
    from yitu_b200.xgnn_h import Block
    dev = torch.device("cuda", 0)
    sizes = graphs.HETERO_TYPES
    rels = graphs.hetero_rgcn(device=dev)
    by_dst = {}
    for i, r in enumerate(rels):
        by_dst.setdefault(r[1], []).append(i)
    assert sorted(by_dst) == [0, 1, 2, 3] and all(len(v) == 2 for v in by_dst.values())
    gen = torch.Generator().manual_seed(5)
    for dt, ids in sorted(by_dst.items()):
        torch.manual_seed(100 + dt)
        relations = [("r%d" % i, Block([sizes[dt], sizes[rels[i][0]]], [rels[i][2], rels[i][3]])) for i in ids]
        layer = StitchedRGCNConv(relations, 64, 64, reduce="sum").to(dev)
        xs = {"r%d" % i: graphs.randn_features(20 + i, sizes[rels[i][0]], 64, device=dev) for i in ids}
        with torch.no_grad():
            out = layer(xs)
        assert out.shape == (sizes[dt], 64)
        deg_total = sum((rels[i][2][1:] - rels[i][2][:-1]) for i in ids)
        rows = torch.cat([torch.topk(deg_total, 4).indices.cpu(), torch.randint(0, sizes[dt], (60,), generator=gen)]).tolist()
        truth = torch.zeros(len(rows), 64, dtype=torch.float64, device=dev)
        for i in ids:
            fc = layer.fcs["r%d" % i]
            w, b_ = fc.weight.detach().double(), fc.bias.detach().double()
            ip, ix = rels[i][2], rels[i][3]
            for j, r in enumerate(rows):
                b0, e0 = int(ip[r]), int(ip[r + 1])
                if e0 > b0:
                    h = xs["r%d" % i][ix[b0:e0].long()].double() @ w.t() + b_
                    truth[j] += h.mean(0)
        err = (out[torch.tensor(rows, device=dev)].double() - truth).abs()
        scale = float(truth.abs().max())
        # 2e-5: a dense fp32 GEMM precedes the aggregation (same bar as the other layer tests)
        assert float((err - 2e-5 * (truth.abs() + scale)).max()) <= 0, "type %d off by %g" % (dt, float(err.max()))
        big = truth.abs() >= 0.01 * scale
        record_error("full-size-hetero-rgcn", float(err.max()) / scale, float((err[big] / truth.abs()[big]).max()))
        del layer, xs, out
        torch.cuda.empty_cache()
