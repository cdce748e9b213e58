"""SpMM parity on the GPU: the C ABI (through yitu_b200.ops / YiTu_GNN_kernel) against the CPU checker."""
import numpy as np
import pytest
import torch

from conftest import assert_close, random_csr

pytestmark = pytest.mark.gpu


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


@pytest.mark.parametrize("D", [1, 3, 16, 20, 32, 48, 64, 100, 128, 200, 256, 512, 640])
@pytest.mark.parametrize("mode", ["none", "node", "edge"])
@pytest.mark.parametrize("kernel", ["auto", "rows", "stream"])
def test_spmm_modes_and_widths(oracle, monkeypatch, D, mode, kernel):
    from yitu_b200 import ops
    if kernel != "auto" and not 64 < D <= 256:
        pytest.skip("one kernel form for this width")
    monkeypatch.setenv("YITU_SPMM_STREAM", {"auto": "1", "rows": "0", "stream": "2"}[kernel])
    rng = np.random.default_rng(D * 7 + len(mode))
    n_rows, n_cols = 211, 173
    indptr, indices = random_csr(rng, n_rows, n_cols, density=0.05, hubs=3, hub_deg=150)
    x = rng.standard_normal((n_cols, D)).astype(np.float32)
    nd = rng.uniform(0.1, 1.0, n_rows).astype(np.float32)
    ns = rng.uniform(0.1, 1.0, n_cols).astype(np.float32)
    vals = rng.standard_normal(indices.shape[0]).astype(np.float32)
    rs = rng.uniform(0.5, 2.0, n_rows).astype(np.float32)
    kw_o = dict(wmode={"none": oracle.W_NONE, "node": oracle.W_NODE, "edge": oracle.W_EDGE}[mode])
    kw_g = dict(mode={"none": ops.W_NONE, "node": ops.W_NODE, "edge": ops.W_EDGE}[mode])
    if mode == "node":
        kw_o.update(norm_dst=nd, norm_src=ns)
        kw_g.update(norm_dst=_dev(nd), norm_src=_dev(ns))
    if mode == "edge":
        kw_o.update(values=vals)
        kw_g.update(edge_values=_dev(vals))
    ref = oracle.spmm(indptr, indices, x, row_scale=rs, alpha=0.5, **kw_o)
    for chunk in (0, 32, 512):  # no hub plan / every hub row split / default
        for ptr_dtype in (torch.int32, torch.int64):
            g = ops.PreparedGraph(_dev(indptr, ptr_dtype), _dev(indices), n_cols)
            got = ops.spmm(g, _dev(x), row_scale=_dev(rs), alpha=0.5, chunk_edges=chunk, **kw_g)
            assert_close(got.cpu().numpy(), ref, what="spmm D=%d %s chunk=%d" % (D, mode, chunk))


def test_spmm_accumulate_and_determinism(oracle):
    from yitu_b200 import ops
    rng = np.random.default_rng(5)
    indptr, indices = random_csr(rng, 300, 300, density=0.1, hubs=2, hub_deg=280)
    x = rng.standard_normal((300, 64)).astype(np.float32)
    base = rng.standard_normal((300, 64)).astype(np.float32)
    g = ops.PreparedGraph(_dev(indptr), _dev(indices), 300)
    out = _dev(base).clone()
    ops.spmm(g, _dev(x), out=out, accumulate=True, alpha=2.0, chunk_edges=64)
    ref = oracle.spmm(indptr, indices, x, alpha=2.0, out=base)
    assert_close(out.cpu().numpy(), ref, what="accumulate")
    a = ops.spmm(g, _dev(x), chunk_edges=64)
    b = ops.spmm(g, _dev(x), chunk_edges=64)
    assert torch.equal(a, b), "hub-split SpMM must be run-to-run identical (no float atomics)"


def test_empty_graph_and_empty_rows(oracle):
    from yitu_b200 import ops
    indptr = np.zeros(6, dtype=np.int32)
    indices = np.zeros(0, dtype=np.int32)
    g = ops.PreparedGraph(_dev(indptr), _dev(indices), 4)
    out = ops.spmm(g, torch.randn(4, 32, device="cuda"))
    assert out.shape == (5, 32) and float(out.abs().max()) == 0.0
    g0 = ops.PreparedGraph(_dev(np.zeros(1, dtype=np.int32)), _dev(indices), 4)
    assert ops.spmm(g0, torch.randn(4, 8, device="cuda")).shape == (0, 8)


def _csr_from_degrees(rng, degs, n_cols):
    rows = [np.sort(rng.choice(n_cols, size=int(k), replace=False)).astype(np.int32) for k in degs]
    indptr = np.zeros(len(degs) + 1, dtype=np.int64)
    indptr[1:] = np.cumsum([len(r) for r in rows])
    indices = np.concatenate(rows) if rows else np.zeros(0, dtype=np.int32)
    return indptr, indices.astype(np.int32)


STREAM_PATTERNS = {
    # runs of empty rows at the start, in the middle and at the end of 16-row batches
    "empty_runs": [0] * 5 + [3, 0, 0, 7, 1] + [0] * 20 + [40, 0, 33, 0, 0, 0] + [2] * 9 + [0] * 18,
    # rows that end exactly on 32-edge tile borders and on borders of the 4/8/16-edge gather groups
    "tile_borders": [32, 32, 64, 16, 16, 8, 8, 8, 8, 4, 4, 96, 1, 31, 33, 63, 65],
    # hub rows (above the 64-edge chunk limit used below) inside batches, adjacent to each other and at the ends
    "hubs_inside": [70, 3, 0, 200, 130, 5, 1] + [2] * 12 + [300] + [1] * 30 + [65, 64, 66],
    "single_row": [5],
    "only_empty": [0] * 37,
    "one_long_row_no_plan": [1000],
}


@pytest.mark.parametrize("pattern", sorted(STREAM_PATTERNS))
@pytest.mark.parametrize("D", [96, 128, 136, 256])
def test_stream_kernel_row_patterns(oracle, monkeypatch, pattern, D):
    """The edge-stream SpMM (warp = batch of consecutive rows walked as one edge stream) on row patterns that put
    every bookkeeping branch to work: empty rows anywhere in a batch, rows ending on tile / group borders, hub rows
    stepped over inside a batch, accumulate mode with and without an epilogue, every batch size and unroll."""
    from yitu_b200 import ops
    rng = np.random.default_rng(len(pattern) * 131 + D)
    n_cols = 1100
    degs = STREAM_PATTERNS[pattern]
    indptr, indices = _csr_from_degrees(rng, degs, n_cols)
    n_rows = len(degs)
    x = rng.standard_normal((n_cols, D)).astype(np.float32)
    vals = rng.standard_normal(indices.shape[0]).astype(np.float32)
    nd = rng.uniform(0.1, 1.0, n_rows).astype(np.float32)
    ns = rng.uniform(0.1, 1.0, n_cols).astype(np.float32)
    base = rng.standard_normal((n_rows, D)).astype(np.float32)
    bias = rng.standard_normal(D).astype(np.float32)
    chunk = 0 if pattern == "one_long_row_no_plan" else 64
    ref_edge = oracle.spmm(indptr, indices, x, wmode=oracle.W_EDGE, values=vals)
    ref_node = oracle.spmm(indptr, indices, x, wmode=oracle.W_NODE, norm_dst=nd, norm_src=ns)
    ref_acc = oracle.spmm(indptr, indices, x, alpha=0.5, out=base)
    ref_acc_epi = np.maximum(oracle.spmm(indptr, indices, x, out=base) + bias, 0)
    monkeypatch.setenv("YITU_SPMM_STREAM", "2")  # this kernel whatever the average row length
    for rows, eu in ((16, None), (8, None), (31, None), (16, 16 if D <= 128 else 8)):
        monkeypatch.setenv("YITU_SPMM_STREAM_ROWS", str(rows))
        if eu is None:
            monkeypatch.delenv("YITU_SPMM_STREAM_EU", raising=False)
        else:
            monkeypatch.setenv("YITU_SPMM_STREAM_EU", str(eu))
        for ptr_dtype in (torch.int32, torch.int64):
            g = ops.PreparedGraph(_dev(indptr, ptr_dtype), _dev(indices), n_cols)
            tag = "stream %s D=%d rows=%d eu=%s" % (pattern, D, rows, eu)
            got = ops.spmm(g, _dev(x), mode=ops.W_EDGE, edge_values=_dev(vals), chunk_edges=chunk)
            assert_close(got.cpu().numpy(), ref_edge, what=tag + " edge")
            got = ops.spmm(g, _dev(x), mode=ops.W_NODE, norm_dst=_dev(nd), norm_src=_dev(ns), chunk_edges=chunk)
            assert_close(got.cpu().numpy(), ref_node, what=tag + " node")
            out = _dev(base).clone()
            ops.spmm(g, _dev(x), out=out, accumulate=True, alpha=0.5, chunk_edges=chunk)
            assert_close(out.cpu().numpy(), ref_acc, what=tag + " accumulate")
            out = _dev(base).clone()
            ops.spmm(g, _dev(x), out=out, accumulate=True, bias=_dev(bias), activation="relu", chunk_edges=chunk)
            assert_close(out.cpu().numpy(), ref_acc_epi, what=tag + " accumulate+epilogue")
    # the default dispatch: hub chunks on the warp-per-row kernel, every other row on the edge-stream kernel
    monkeypatch.setenv("YITU_SPMM_STREAM", "1")
    monkeypatch.delenv("YITU_SPMM_STREAM_ROWS", raising=False)
    monkeypatch.delenv("YITU_SPMM_STREAM_EU", raising=False)
    g = ops.PreparedGraph(_dev(indptr, torch.int64), _dev(indices), n_cols)
    got = ops.spmm(g, _dev(x), mode=ops.W_NODE, norm_dst=_dev(nd), norm_src=_dev(ns), chunk_edges=chunk)
    assert_close(got.cpu().numpy(), ref_node, what="split %s D=%d node" % (pattern, D))
    out = _dev(base).clone()
    ops.spmm(g, _dev(x), out=out, accumulate=True, bias=_dev(bias), activation="relu", chunk_edges=chunk)
    assert_close(out.cpu().numpy(), ref_acc_epi, what="split %s D=%d accumulate+epilogue" % (pattern, D))
    # the warp-per-row kernel on the same inputs gives the same sums up to the order of the additions
    monkeypatch.setenv("YITU_SPMM_STREAM", "0")
    g = ops.PreparedGraph(_dev(indptr, torch.int32), _dev(indices), n_cols)
    got = ops.spmm(g, _dev(x), mode=ops.W_EDGE, edge_values=_dev(vals), chunk_edges=chunk)
    assert_close(got.cpu().numpy(), ref_edge, what="rows-kernel %s D=%d" % (pattern, D))


def test_kernel_module_matches_oracle_on_gcn_graph(oracle):
    """2-layer GCN forward of the small benchmark configuration, plus the other YiTu_GNN_kernel entry points."""
    from yitu_b200 import YiTu_GNN_kernel as K, graphs
    n = 16384
    indptr, indices, norm = graphs.gcn_small()
    x = graphs.randn_features(0, n, 128)
    w1 = graphs.glorot_uniform(11, 128, 64)
    w2 = graphs.glorot_uniform(12, 64, 16)
    ip, ix, nm = indptr.cuda(), indices.cuda(), norm.cuda()
    pp, p2n = K.build_part(32, indptr)
    pp, p2n = pp.int().cuda(), p2n.int().cuda()
    args = (ip, ix, nm, pp, p2n, 32, 32, 2)
    h1 = K.forward(x.cuda(), w1.cuda(), *args)[0]
    out = K.forward(torch.relu(h1), w2.cuda(), *args)[0]
    r1 = oracle.gcn_forward(x.numpy(), w1.numpy(), indptr.numpy(), indices.numpy(), norm.numpy())
    r2 = oracle.gcn_forward(np.maximum(r1, 0), w2.numpy(), indptr.numpy(), indices.numpy(), norm.numpy())
    assert_close(h1.cpu().numpy(), r1, what="gcn layer 1")
    assert_close(out.cpu().numpy(), r2, rtol=2e-5, what="gcn layer 2")

    # backward: true transpose by default; the reference's forward-CSR variant behind the flag
    d_out = graphs.randn_features(3, n, 64)
    d_in, d_w = K.backward(d_out.cuda(), x.cuda(), w1.cuda(), *args)
    rd_in, rd_w = oracle.gcn_backward(d_out.numpy(), x.numpy(), w1.numpy(), indptr.numpy(), indices.numpy(),
                                      norm.numpy(), transpose=True)
    assert_close(d_in.cpu().numpy(), rd_in, rtol=2e-5, what="gcn d_input")
    assert_close(d_w.cpu().numpy(), rd_w, rtol=2e-5, what="gcn d_weight")
    K.BACKWARD_USES_FORWARD_CSR = True
    try:
        d_in2, _ = K.backward(d_out.cuda(), x.cuda(), w1.cuda(), *args)
    finally:
        K.BACKWARD_USES_FORWARD_CSR = False
    rd_in2, _ = oracle.gcn_backward(d_out.numpy(), x.numpy(), w1.numpy(), indptr.numpy(), indices.numpy(),
                                    norm.numpy(), transpose=False)
    assert_close(d_in2.cpu().numpy(), rd_in2, rtol=2e-5, what="gcn d_input (forward CSR)")

    # SAG and GIN
    xs = x[:, :64].contiguous()
    sag = K.SAG(xs.cuda(), *args)
    assert_close(sag.cpu().numpy(), oracle.spmm(indptr.numpy(), indices.numpy(), xs.numpy()), what="SAG")
    wg = graphs.glorot_uniform(13, 64, 32)
    gargs = (ip, ix, 0.5, pp, p2n, 32, 32, 2)
    o_gin, agg = K.forward_gin(xs.cuda(), wg.cuda(), *gargs)
    r_gin, r_agg = oracle.gin_forward(xs.numpy(), wg.numpy(), indptr.numpy(), indices.numpy(), 0.5)
    assert_close(agg.cpu().numpy(), r_agg, what="gin agg")
    assert_close(o_gin.cpu().numpy(), r_gin, rtol=2e-5, what="gin out")
    dg = graphs.randn_features(4, n, 32)
    di, dw = K.backward_gin(dg.cuda(), agg, wg.cuda(), *gargs)
    rdi, rdw = oracle.gin_backward(dg.numpy(), r_agg, wg.numpy(), indptr.numpy(), indices.numpy(), 0.5)
    assert_close(di.cpu().numpy(), rdi, rtol=2e-5, what="gin d_input")
    assert_close(dw.cpu().numpy(), rdw, rtol=2e-5, what="gin d_weight")


def test_input_contract():
    from yitu_b200 import YiTu_GNN_kernel as K
    x = torch.randn(4, 8)
    ip = torch.tensor([0, 1, 2, 3, 4], dtype=torch.int32).cuda()
    ix = torch.tensor([0, 1, 2, 3], dtype=torch.int32).cuda()
    d = torch.ones(4).cuda()
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        K.SAG(x, ip, ix, d, ip, ix, 32, 32, 2)
    with pytest.raises(RuntimeError, match="contiguous"):
        K.SAG(torch.randn(8, 4).cuda().t(), ip, ix, d, ip, ix, 32, 32, 2)


def test_graph_tables_bit_exact(oracle):
    from yitu_b200 import ops
    rng = np.random.default_rng(17)
    indptr, indices = random_csr(rng, 1500, 900, density=0.03, hubs=4, hub_deg=700)
    for ptr_dtype in (torch.int32, torch.int64):
        g = ops.PreparedGraph(_dev(indptr, ptr_dtype), _dev(indices), 900)
        t_ip, t_rows, t_perm = g.transpose()
        r_ip, r_rows, r_perm = oracle.csr_transpose(indptr, indices, 900)
        assert np.array_equal(t_ip.cpu().numpy().astype(np.int64), r_ip)
        assert np.array_equal(t_rows.cpu().numpy(), r_rows)
        assert np.array_equal(t_perm.cpu().numpy(), r_perm)
        for parts in (1, 2, 3, 8):
            b = ops.partition_rows(g, parts).cpu().numpy()
            assert np.array_equal(b, oracle.partition_rows(indptr, parts))
        plan = g.plan(64)
        deg = np.diff(indptr)
        exp_rows, exp_begin = [], []
        for r in np.nonzero(deg > 64)[0]:
            for j in range((deg[r] + 63) // 64):
                exp_rows.append(r)
                exp_begin.append(indptr[r] + 64 * j)
        assert plan[0].n_chunks == len(exp_rows)
        assert np.array_equal(plan[1].cpu().numpy(), np.asarray(exp_rows, dtype=np.int32))
        assert np.array_equal(plan[2].cpu().numpy(), np.asarray(exp_begin, dtype=np.int64))


def test_full_size_properties():
    """Benchmark-size graph (2^21 nodes, 2^26 sampled edges, 256 features): properties that need no CPU pass.
    unweighted A*1 = in-degree; linearity in x; hub-split and unsplit schedules agree."""
    from yitu_b200 import graphs, ops
    n = 1 << 21
    indptr, indices, values = graphs.spmm_rmat(device="cuda", n=n, e=1 << 26)
    g = ops.PreparedGraph(indptr, indices, n)
    deg = (indptr[1:] - indptr[:-1]).float()
    ones = torch.ones(n, 4, device="cuda")
    out = ops.spmm(g, ones)
    assert torch.equal(out[:, 0], deg), "A*1 must equal the in-degree exactly (integers < 2^24)"
    x1 = graphs.randn_features(1, n, 256, device="cuda")
    y1 = ops.spmm(g, x1, mode=ops.W_EDGE, edge_values=values)
    y1b = ops.spmm(g, x1, mode=ops.W_EDGE, edge_values=values, chunk_edges=0)
    scale = float(y1.abs().max())
    assert float((y1 - y1b).abs().max()) <= 2e-5 * scale
    y2 = ops.spmm(g, x1 * 2.0, mode=ops.W_EDGE, edge_values=values)
    assert torch.equal(y2, y1 * 2.0), "scaling x by 2 is exact in binary floating point"
    # transposed product: <A x, y> == <x, A^T y> within reduction tolerance (float64 dots)
    gt = g.t_prepared()
    t_perm = g.transpose()[2]
    yv = graphs.randn_features(2, n, 256, device="cuda")
    aty = ops.spmm(gt, yv, mode=ops.W_EDGE, edge_values=values, edge_perm=t_perm)
    lhs = float((y1.double() * yv.double()).sum())
    rhs = float((x1.double() * aty.double()).sum())
    assert abs(lhs - rhs) <= 1e-5 * max(abs(lhs), abs(rhs), 1.0) + 1e-2


def _rows_truth_f64(indptr, indices, values, x, rows):
    """float64 aggregation of a few destination rows, straight from the definition."""
    out = []
    for r in rows.tolist():
        b, e = int(indptr[r]), int(indptr[r + 1])
        cols = indices[b:e].long()
        w = values[b:e].double() if values is not None else torch.ones(e - b, dtype=torch.float64, device=x.device)
        out.append((w[:, None] * x[cols].double()).sum(0))
    return torch.stack(out)


def test_full_size_sampled_rows_against_float64():
    """Benchmark-size SpMM (2^21 nodes, 63.5 M edges, 256 features): 300 sampled destination rows, among them the
    longest hub rows, forward and transposed, against float64 sums at the 1e-5 bar."""
    from yitu_b200 import graphs, ops
    n = 1 << 21
    indptr, indices, values = graphs.spmm_rmat(device="cuda", n=n, e=1 << 26)
    g = ops.PreparedGraph(indptr, indices, n)
    x = graphs.randn_features(1, n, 256, device="cuda")
    y = ops.spmm(g, x, mode=ops.W_EDGE, edge_values=values)
    deg = indptr[1:] - indptr[:-1]
    gen = torch.Generator(device="cpu").manual_seed(0)
    rows = torch.cat([torch.topk(deg, 20).indices.cpu(), torch.randint(0, n, (280,), generator=gen)])
    truth = _rows_truth_f64(indptr, indices, values, x, rows)
    scale = float(truth.abs().max())
    err = (y[rows.cuda()].double() - truth).abs()
    assert float((err - 1e-5 * (truth.abs() + scale)).max()) <= 0, "forward rows off by %g" % float(err.max())
    # transposed product over the CSC built on the device
    gt = g.t_prepared()
    t_indptr, t_rows, t_perm = g.transpose()
    yt = ops.spmm(gt, x, mode=ops.W_EDGE, edge_values=values, edge_perm=t_perm)
    out_deg = t_indptr[1:] - t_indptr[:-1]
    cols = torch.cat([torch.topk(out_deg, 20).indices.cpu(), torch.randint(0, n, (280,), generator=gen)])
    truth_t = _rows_truth_f64(t_indptr, t_rows, values[t_perm.long()], x, cols)
    scale_t = float(truth_t.abs().max())
    err_t = (yt[cols.cuda()].double() - truth_t).abs()
    assert float((err_t - 1e-5 * (truth_t.abs() + scale_t)).max()) <= 0, "transposed rows off by %g" % float(err_t.max())


def test_partitioned_config_on_one_gpu_sampled_rows_against_float64():
    """The 8-GPU configuration's graph on one GPU: R-MAT 2^24 nodes, 2^29 sampled edges, int64 row pointers,
    weights 1/in-degree, 128 features (2^31 feature elements: element offsets use all 32 bits).  Sampled destination
    rows in float64 - the longest rows, rows whose sources lie at the very end of the feature matrix, and random
    ones - plus the exact identities A*1 = in-degree and (A/deg)*1 = 1."""
    from yitu_b200 import graphs, ops
    n, d = 1 << 24, 128
    indptr, indices, values = graphs.spmm_partitioned(device="cuda", n=n, e=1 << 29)
    assert indptr.dtype == torch.int64
    g = ops.PreparedGraph(indptr, indices, n)
    deg = indptr[1:] - indptr[:-1]
    ones = torch.ones(n, 4, device="cuda")
    assert torch.equal(ops.spmm(g, ones)[:, 0], deg.float()), "A*1 must equal the in-degree exactly"
    del ones
    x = graphs.randn_features(1, n, d, device="cuda")
    y = ops.spmm(g, x, mode=ops.W_EDGE, edge_values=values)
    gen = torch.Generator(device="cpu").manual_seed(0)
    # destination rows of the edges whose source id is largest (the last rows of x, offsets just below 2^31)
    far = torch.topk(indices.long(), 64).indices
    far_rows = (torch.searchsorted(indptr, far, right=True) - 1).cpu()
    assert int(indices.max()) * d + d > (1 << 30), "the sample must reach the upper half of the offset range"
    rows = torch.cat([torch.topk(deg, 16).indices.cpu(), far_rows, torch.randint(0, n, (240,), generator=gen)]).unique()
    truth = _rows_truth_f64(indptr, indices, values, x, rows)
    scale = float(truth.abs().max())
    err = (y[rows.cuda()].double() - truth).abs()
    assert float((err - 1e-5 * (truth.abs() + scale)).max()) <= 0, "rows off by %g" % float(err.max())
    from conftest import record_error
    big = truth.abs() >= 0.01 * scale
    record_error("partitioned-config-1gpu", float(err.max()) / scale, float((err[big] / truth.abs()[big]).max()))
