"""Fused layer epilogues on the GPU: row scale + bias + activation in the SpMM, the mean over heads (+ activation)
in the fused GAT kernel and its backward over the [n_dst,F] gradient, the one-pass epilogue gradient, and the
layers that use them — against the CPU oracle with the same epilogue applied in float64, and against the unfused
operator compositions."""
import numpy as np
import pytest
import torch

from conftest import assert_close, random_csr

pytestmark = pytest.mark.gpu


def _act64(v, name):
    if name == "relu":
        return np.maximum(v, 0.0)
    if name == "elu":
        return np.where(v > 0, v, np.expm1(np.minimum(v, 0.0)))
    return v


def _graph(indptr, indices, n_cols, mask=0):
    from yitu_b200 import ops
    return ops.PreparedGraph(torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda(), n_cols, mask)


@pytest.mark.parametrize("D", [8, 32, 64, 100, 128, 256, 512])
@pytest.mark.parametrize("act", [None, "relu", "elu"])
def test_spmm_epilogue_matches_oracle(oracle, D, act):
    from yitu_b200 import ops
    rng = np.random.default_rng(D)
    n_rows, n_cols = 700, 900
    indptr, indices = random_csr(rng, n_rows, n_cols, density=0.02, hubs=3, hub_deg=800)
    x = rng.standard_normal((n_cols, D)).astype(np.float32)
    vals = rng.random(len(indices)).astype(np.float32)
    scale = (rng.random(n_rows) + 0.5).astype(np.float32)
    bias = rng.standard_normal(D).astype(np.float32)
    ref = oracle.spmm(indptr, indices, x, wmode=oracle.W_EDGE, values=vals).astype(np.float64)
    ref = _act64(0.5 * scale[:, None].astype(np.float64) * ref + bias.astype(np.float64), act)
    g = _graph(indptr, indices, n_cols)
    for chunk in (ops.DEFAULT_CHUNK_EDGES, 0):  # hub rows through the chunk reduction, and through the row kernel
        got = ops.spmm(g, torch.from_numpy(x).cuda(), mode=ops.W_EDGE, edge_values=torch.from_numpy(vals).cuda(),
                       row_scale=torch.from_numpy(scale).cuda(), alpha=0.5, bias=torch.from_numpy(bias).cuda(),
                       activation=act, chunk_edges=chunk)
        assert_close(got.cpu().numpy(), ref, what="spmm epilogue D=%d act=%s chunk=%d" % (D, act, chunk))


def test_spmm_epilogue_accumulate_then_activation(oracle):
    from yitu_b200 import ops
    rng = np.random.default_rng(3)
    indptr, indices = random_csr(rng, 300, 300, density=0.04)
    x = rng.standard_normal((300, 64)).astype(np.float32)
    prev = rng.standard_normal((300, 64)).astype(np.float32)
    bias = rng.standard_normal(64).astype(np.float32)
    ref = np.maximum(prev.astype(np.float64) + oracle.spmm(indptr, indices, x) + bias, 0.0)
    out = torch.from_numpy(prev.copy()).cuda()
    ops.spmm(_graph(indptr, indices, 300), torch.from_numpy(x).cuda(), out=out, accumulate=True,
             bias=torch.from_numpy(bias).cuda(), activation="relu")
    assert_close(out.cpu().numpy(), ref, what="accumulate + bias + relu")


def test_spmm_rejects_bad_epilogue_arguments():
    from yitu_b200 import ops
    rng = np.random.default_rng(4)
    indptr, indices = random_csr(rng, 50, 50, density=0.1)
    g = _graph(indptr, indices, 50)
    x = torch.randn(50, 16, device="cuda")
    with pytest.raises(RuntimeError):
        ops.spmm(g, x, activation="gelu")
    with pytest.raises(RuntimeError):
        ops.spmm(g, x, bias=torch.zeros(8, device="cuda"))
    with pytest.raises(RuntimeError):  # shared rows only make sense with per-head edge values
        ops.spmm(g, x, n_heads=2, x_shared_heads=True)


@pytest.mark.parametrize("H,F", [(8, 32), (4, 16), (2, 64), (3, 20), (1, 8)])
def test_spmm_shared_heads_equals_expanded_rows(H, F):
    from yitu_b200 import ops
    rng = np.random.default_rng(H * 100 + F)
    n_rows, n_cols = 500, 400
    indptr, indices = random_csr(rng, n_rows, n_cols, density=0.03, hubs=2, hub_deg=390)
    g = _graph(indptr, indices, n_cols)
    xs = torch.randn(n_cols, F, device="cuda")
    vals = torch.rand(len(indices), H, device="cuda")
    full = ops.spmm(g, xs.unsqueeze(1).expand(-1, H, -1).contiguous(), n_heads=H, mode=ops.W_EDGE_HEAD,
                    edge_values=vals, alpha=0.25)
    shared = ops.spmm(g, xs, n_heads=H, mode=ops.W_EDGE_HEAD, edge_values=vals, alpha=0.25, x_shared_heads=True)
    assert shared.shape == (n_rows, H, F)
    assert torch.equal(full, shared)  # same products in the same order


@pytest.mark.parametrize("shape", [(1000, 256), (333, 7), (0, 16), (5, 4)])
@pytest.mark.parametrize("act", [None, "relu", "elu"])
def test_epilogue_grad_matches_torch(shape, act):
    from yitu_b200 import ops
    torch.manual_seed(shape[0] + shape[1])
    pre = torch.randn(*shape, device="cuda", dtype=torch.float64, requires_grad=True)
    scale = torch.rand(shape[0], device="cuda") + 0.5
    gy = torch.randn(*shape, device="cuda")
    y64 = {"relu": torch.relu, "elu": torch.nn.functional.elu, None: lambda t: t}[act](pre)
    (y64 * gy.double()).sum().backward()
    ref = pre.grad * scale.double()[:, None]
    got = ops.epilogue_grad(y64.detach().float(), gy, scale, act)
    assert got.shape == gy.shape
    if shape[0]:
        assert float((got.double() - ref).abs().max()) <= 1e-6 * (float(ref.abs().max()) + 1.0)


@pytest.mark.parametrize("H,F", [(8, 32), (4, 16), (2, 64), (3, 20), (1, 128), (16, 32)])
@pytest.mark.parametrize("act", [None, "elu"])
def test_gat_head_mean_forward_matches_oracle(oracle, H, F, act):
    from yitu_b200 import ops
    rng = np.random.default_rng(H + F)
    n = 600
    indptr, indices = random_csr(rng, n, n, density=0.03, hubs=2, hub_deg=500)
    q = rng.standard_normal((n, H)).astype(np.float32)
    k = rng.standard_normal((n, H)).astype(np.float32)
    x = rng.standard_normal((n, H, F)).astype(np.float32)
    ref_full, _ = oracle.gat_forward(indptr, indices, q, k, x)
    ref = _act64(ref_full.astype(np.float64).mean(axis=1), act)
    g = _graph(indptr, indices, n)
    out, rmax, rsum, heads = ops.gat_fwd(g, torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(),
                                         torch.from_numpy(x).cuda(), head_mean=True, activation=act)
    assert out.shape == (n, F) and heads.shape == (n, H, F)
    assert_close(heads.cpu().numpy(), ref_full, what="per-head result kept for the backward")
    assert_close(out.cpu().numpy(), ref, what="gat head mean H=%d F=%d act=%s" % (H, F, act))
    full, rmax2, rsum2 = ops.gat_fwd(g, torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(),
                                     torch.from_numpy(x).cuda())
    assert torch.equal(rmax, rmax2) and torch.equal(rsum, rsum2)
    assert_close(full.cpu().numpy(), ref_full, what="per-head output unchanged")


@pytest.mark.parametrize("act", ["relu", "elu"])
def test_gat_forward_activation_without_head_mean(oracle, act):
    from yitu_b200 import ops
    rng = np.random.default_rng(9)
    n, H, F = 300, 4, 16
    indptr, indices = random_csr(rng, n, n, density=0.05)
    q = rng.standard_normal((n, H)).astype(np.float32)
    k = rng.standard_normal((n, H)).astype(np.float32)
    x = rng.standard_normal((n, H, F)).astype(np.float32)
    ref, _ = oracle.gat_forward(indptr, indices, q, k, x)
    out, _, _ = ops.gat_fwd(_graph(indptr, indices, n), torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(),
                            torch.from_numpy(x).cuda(), activation=act)
    assert_close(out.cpu().numpy(), _act64(ref.astype(np.float64), act), what="gat activation %s" % act)


@pytest.mark.parametrize("H,F", [(8, 32), (4, 16), (2, 64), (3, 20), (16, 32)])
def test_gat_head_mean_backward_matches_oracle(oracle, H, F):
    from yitu_b200 import ops
    rng = np.random.default_rng(10 * H + F)
    n = 500
    indptr, indices = random_csr(rng, n, n, density=0.03, hubs=2, hub_deg=450)
    q = rng.standard_normal((n, H)).astype(np.float32)
    k = rng.standard_normal((n, H)).astype(np.float32)
    x = rng.standard_normal((n, H, F)).astype(np.float32)
    g_mean = rng.standard_normal((n, F)).astype(np.float32)
    # gradient of mean over heads: every head receives g / H
    g_full = np.repeat(g_mean[:, None, :], H, axis=1) / np.float32(H)
    _, attn = oracle.gat_forward(indptr, indices, q, k, x)
    ref_q, ref_k, ref_x = oracle.gat_backward(indptr, indices, q, k, x, attn, g_full.astype(np.float32))
    gr = _graph(indptr, indices, n)
    tq, tk, tx = (torch.from_numpy(a).cuda() for a in (q, k, x))
    out, rmax, rsum, heads = ops.gat_fwd(gr, tq, tk, tx, head_mean=True)
    gq, gk, gx = ops.gat_bwd(gr, tq, tk, tx, out, rmax, rsum, torch.from_numpy(g_mean).cuda(), head_mean=True,
                             out_heads=heads)
    assert_close(gq.cpu().numpy(), np.asarray(ref_q).reshape(gq.shape), rtol=2e-5, what="grad_query")
    assert_close(gk.cpu().numpy(), ref_k, rtol=2e-5, what="grad_key")
    assert_close(gx.cpu().numpy(), ref_x, rtol=2e-5, what="grad_x")
    with pytest.raises(RuntimeError):  # the per-head gradient shape is refused in head-mean mode
        ops.gat_bwd(gr, tq, tk, tx, out, rmax, rsum, torch.from_numpy(g_full).cuda(), head_mean=True, out_heads=heads)
    with pytest.raises(RuntimeError):  # and so is a head-mean backward without the per-head forward result
        ops.gat_bwd(gr, tq, tk, tx, out, rmax, rsum, torch.from_numpy(g_mean).cuda(), head_mean=True)


def _block(indptr, indices, n_src):
    from yitu_b200.xgnn_h import Block
    return Block([len(indptr) - 1, n_src], [torch.from_numpy(indptr).cuda(), torch.from_numpy(indices).cuda()])


def _dense(indptr, indices, n_src):
    n_dst = len(indptr) - 1
    a = torch.zeros(n_dst, n_src, dtype=torch.float64)
    a[np.repeat(np.arange(n_dst), np.diff(indptr)), indices] = 1.0
    return a.cuda()


def _close(a, b, tol=2e-5):
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).abs().max()) <= tol * (float(b.abs().max()) + 1e-30)


@pytest.mark.parametrize("act", [None, "relu", "elu"])
@pytest.mark.parametrize("with_bias", [False, True])
def test_aggregate_epilogue_autograd_matches_dense(act, with_bias):
    from yitu_b200.nn.layers import aggregate
    rng = np.random.default_rng(20)
    n_dst, n_src, D = 260, 310, 24
    indptr, indices = random_csr(rng, n_dst, n_src, density=0.05)
    blk = _block(indptr, indices, n_src)
    a = _dense(indptr, indices, n_src)
    x = torch.randn(n_src, D, device="cuda", requires_grad=True)
    scale = torch.rand(n_dst, device="cuda") + 0.5
    bias = torch.randn(D, device="cuda", requires_grad=True) if with_bias else None
    w_out = torch.randn(n_dst, D, device="cuda")
    y = aggregate(blk, x, row_scale=scale, bias=bias, activation=act)
    (y * w_out).sum().backward()
    xd = x.detach().double().requires_grad_()
    bd = bias.detach().double().requires_grad_() if with_bias else None
    pre = scale.double()[:, None] * (a @ xd)
    if with_bias:
        pre = pre + bd
    yd = {"relu": torch.relu, "elu": torch.nn.functional.elu, None: lambda t: t}[act](pre)
    (yd * w_out.double()).sum().backward()
    assert _close(y, yd) and _close(x.grad, xd.grad)
    if with_bias:
        assert _close(bias.grad, bd.grad)


def test_gcn_layer_fuses_norm_and_activation():
    from yitu_b200.nn import GCNLayer
    rng = np.random.default_rng(21)
    n = 350
    indptr, indices = random_csr(rng, n, n, density=0.04, empty_rows=False)
    blk = _block(indptr, indices, n)
    a = _dense(indptr, indices, n)
    norm = (1.0 / torch.from_numpy(np.diff(indptr).astype(np.float32))).cuda().view(n, 1)
    layer = GCNLayer(20, 12, activation="relu").cuda()
    x = torch.randn(n, 20, device="cuda", requires_grad=True)
    y = layer(blk, norm, x)
    y.sum().backward()
    xd = x.detach().double().requires_grad_()
    wd, bd = layer.fc.weight.detach().double().requires_grad_(), layer.fc.bias.detach().double().requires_grad_()
    yd = torch.relu(norm.double() * (a @ (xd @ wd.t() + bd)))
    yd.sum().backward()
    assert _close(y, yd) and _close(x.grad, xd.grad)
    assert _close(layer.fc.weight.grad, wd.grad, 5e-5) and _close(layer.fc.bias.grad, bd.grad, 5e-5)


@pytest.mark.parametrize("act", [None, "elu"])
def test_gat_layer_head_mean_matches_unfused_composition(act):
    from yitu_b200.nn import GATLayer
    from yitu_b200.xgnn_h import sparse
    rng = np.random.default_rng(22)
    n, H, F = 320, 4, 16
    indptr, indices = random_csr(rng, n, n, density=0.05, empty_rows=False)
    blk = _block(indptr, indices, n)
    layer = GATLayer(20, F, H, activation=act).cuda()
    x = torch.randn(n, 20, device="cuda", requires_grad=True)
    w_out = torch.randn(n, F, device="cuda")
    y = layer(blk, x)
    (y * w_out).sum().backward()
    got = [x.grad.clone()] + [p.grad.clone() for p in layer.parameters()]
    x.grad = None
    layer.zero_grad()
    # the reference's formulation: attention tensor, aggregation, torch.mean, activation as separate operators
    h = layer.linear_v(x)
    q, k = layer.linear_q(h), layer.linear_k(h)
    out = sparse.gspmm(blk, sparse.fused_gsddmm(blk, q, k), h.view(-1, H, F))
    y2 = sparse._TORCH_ACT[act](torch.mean(out, dim=1))
    (y2 * w_out).sum().backward()
    ref = [x.grad.clone()] + [p.grad.clone() for p in layer.parameters()]
    assert _close(y, y2)
    for a, b in zip(got, ref):
        assert _close(a, b, 5e-5)


def test_head_mean_inference_skips_the_per_head_write():
    from yitu_b200 import ops
    from yitu_b200.xgnn_h import sparse
    rng = np.random.default_rng(23)
    n, H, F = 300, 4, 16
    indptr, indices = random_csr(rng, n, n, density=0.05)
    blk = _block(indptr, indices, n)
    q, k, x = torch.randn(n, H, device="cuda"), torch.randn(n, H, device="cuda"), torch.randn(n, H, F, device="cuda")
    y_train = sparse.fused_gat(blk, q.clone().requires_grad_(), k, x, head_mean=True, activation="elu")
    with torch.no_grad():
        y_eval = sparse.fused_gat(blk, q, k, x, head_mean=True, activation="elu")
    assert torch.equal(y_train.detach(), y_eval)
    g = ops.prepared(blk.adj_sparse[0], blk.adj_sparse[1], n, 0)
    assert ops.gat_fwd(g, q, k, x, head_mean=True, keep_heads=False)[3] is None
