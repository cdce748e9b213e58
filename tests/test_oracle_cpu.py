"""Pins of the CPU checker (no GPU): the golden vectors produced by the reference's own CPU code, scipy, and the
dense-math identities of the reference's kernel tests (YiTu_GNN/YiTu_H/test/test_kernel.py:25-359) evaluated in
float64 torch autograd."""
import json
import os

import numpy as np
import pytest
import scipy.sparse as sp
import torch

from conftest import assert_close, random_csr

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _golden(name):
    with open(os.path.join(GOLDEN, name + ".json")) as f:
        return json.load(f)


def test_build_part_matches_reference_outputs(oracle):
    for case in _golden("build_part"):
        pp, p2n = oracle.build_part(case["part_size"], np.asarray(case["indptr"], dtype=np.int32))
        assert pp.dtype == np.float32 and p2n.dtype == np.float32
        assert pp.tolist() == case["part_ptr"], case
        assert p2n.tolist() == case["part2node"], case


def test_build_part_known_answer(oracle):
    pp, p2n = oracle.build_part(2, [0, 3, 3, 8, 9])
    assert pp.tolist() == [0, 2, 3, 5, 7, 8, 9] and p2n.tolist() == [0, 0, 2, 2, 2, 3]
    pp, _ = oracle.build_part(2, [0, 3, 3, 8, 8])  # last node empty: the reference leaves the terminal pointer 0
    assert pp.tolist() == [0, 2, 3, 5, 7, 0]


def test_stitch_csr_matches_reference_outputs(oracle):
    for case in _golden("stitch_csr"):
        blocks = [(np.asarray(b["indptr"], dtype=np.int32), np.asarray(b["indices"], dtype=np.int32), b["n_cols"])
                  for b in case["blocks"]]
        ip, ix, n_cols = oracle.stitch_csr(blocks)
        assert ip.tolist() == case["indptr"] and ix.tolist() == case["indices"]
        assert [case["n_rows"], n_cols] == case["size"]


def test_csr_convention_matches_reference_to_csr(oracle):
    """Rows = destinations, ascending columns: what convert.to_csr and scipy give the reference."""
    for case in _golden("to_csr"):
        dense = np.asarray(case["dense"])
        m = sp.csr_matrix(dense)
        m.sort_indices()
        assert m.indptr.tolist() == case["indptr"] and m.indices.tolist() == case["indices"]
        t_ip, t_rows, t_perm = oracle.csr_transpose(m.indptr, m.indices, dense.shape[1])
        mt = sp.csr_matrix(dense.T)
        mt.sort_indices()
        assert t_ip.tolist() == mt.indptr.tolist() and t_rows.tolist() == mt.indices.tolist()
        assert np.array_equal(np.asarray(case["indices"])[t_perm], np.repeat(np.arange(dense.shape[1]), np.diff(t_ip)))


@pytest.mark.parametrize("mode", ["none", "node", "edge"])
def test_spmm_against_scipy(oracle, mode):
    rng = np.random.default_rng(1)
    indptr, indices = random_csr(rng, 300, 257, density=0.05, hubs=2, hub_deg=200)
    x = rng.standard_normal((257, 48)).astype(np.float32)
    nd = rng.uniform(0.2, 1, 300).astype(np.float32)
    ns = rng.uniform(0.2, 1, 257).astype(np.float32)
    vals = rng.standard_normal(indices.shape[0]).astype(np.float32)
    rows = np.repeat(np.arange(300), np.diff(indptr))
    if mode == "none":
        w = np.ones(indices.shape[0])
        got = oracle.spmm(indptr, indices, x)
    elif mode == "node":
        w = (nd[rows] * ns[indices]).astype(np.float64)
        got = oracle.spmm(indptr, indices, x, wmode=oracle.W_NODE, norm_dst=nd, norm_src=ns)
    else:
        w = vals.astype(np.float64)
        got = oracle.spmm(indptr, indices, x, wmode=oracle.W_EDGE, values=vals)
    a = sp.csr_matrix((w, indices, indptr), shape=(300, 257))
    assert_close(got, a @ x.astype(np.float64), rtol=1e-6, what="oracle spmm vs scipy")
    g = rng.standard_normal((300, 48)).astype(np.float32)
    kw = {} if mode == "none" else (dict(wmode=oracle.W_NODE, norm_dst=nd, norm_src=ns) if mode == "node"
                                    else dict(wmode=oracle.W_EDGE, values=vals))
    assert_close(oracle.spmm_transpose(indptr, indices, 257, g, **kw), a.T @ g.astype(np.float64), rtol=1e-6,
                 what="oracle transposed spmm vs scipy")


def test_gcn_forward_small_config(oracle):
    """2-layer GCN forward of the small benchmark configuration against scipy in float64."""
    from yitu_b200 import graphs
    n = 2048
    indptr, indices, norm = graphs.gcn_small(n=n, e=32768)
    x = graphs.randn_features(0, n, 128).numpy()
    w1, w2 = graphs.glorot_uniform(1, 128, 64).numpy(), graphs.glorot_uniform(2, 64, 16).numpy()
    ip, ix, nm = indptr.numpy(), indices.numpy(), norm.numpy()
    h = oracle.gcn_forward(x, w1, ip, ix, nm)
    out = oracle.gcn_forward(np.maximum(h, 0), w2, ip, ix, nm)
    rows = np.repeat(np.arange(n), np.diff(ip))
    a = sp.csr_matrix(((nm[rows] * nm[ix]).astype(np.float64), ix, ip), shape=(n, n))
    h_ref = a @ (x.astype(np.float64) @ w1.astype(np.float64))
    out_ref = a @ (np.maximum(h_ref, 0) @ w2.astype(np.float64))
    assert_close(h, h_ref, rtol=1e-6, what="layer 1")
    assert_close(out, out_ref, rtol=2e-6, what="layer 2")
    # self-loops present and symmetric normalisation: diagonal weight = 1/deg
    assert np.all(np.diff(ip) >= 1)


def _dense_attention(indptr, indices, q, k, n_src):
    """softmax over in-edges of LeakyReLU(q_i + k_j), dense float64 torch (test_kernel.py:131-152)."""
    n_dst, H = q.shape
    adj = torch.zeros(n_dst, n_src, dtype=torch.float64)
    rows = np.repeat(np.arange(n_dst), np.diff(indptr))
    adj[rows, indices] = 1.0
    e = torch.nn.functional.leaky_relu(q.unsqueeze(1) + k.unsqueeze(0), 0.2)
    e = torch.where(adj.unsqueeze(-1) > 0, e, torch.full_like(e, -1e300)).permute(2, 0, 1)
    return torch.softmax(e, dim=-1) * adj.unsqueeze(0), rows


@pytest.mark.parametrize("seed", range(3))
def test_reference_identity_gsddmm_gspmm(oracle, seed):
    """fused_gsddmm + gspmm == masked dense softmax + bmm, outputs and gradients (check_gsddmm / check_gspmm)."""
    rng = np.random.default_rng(seed)
    n_dst, n_src, H, F = int(rng.integers(2, 60)), int(rng.integers(2, 60)), int(rng.integers(1, 6)), int(rng.integers(1, 20))
    indptr, indices = random_csr(rng, n_dst, n_src, density=0.2, empty_rows=False)
    q = torch.tensor(rng.standard_normal((n_dst, H)).astype(np.float32), dtype=torch.float64, requires_grad=True)
    k = torch.tensor(rng.standard_normal((n_src, H)).astype(np.float32), dtype=torch.float64, requires_grad=True)
    x = torch.tensor(rng.standard_normal((n_src, H, F)).astype(np.float32), dtype=torch.float64, requires_grad=True)
    g = rng.standard_normal((n_dst, H, F)).astype(np.float32)
    attn_d, rows = _dense_attention(indptr, indices, q, k, n_src)
    y = torch.bmm(attn_d, x.transpose(0, 1)).transpose(0, 1)
    (y * torch.tensor(g, dtype=torch.float64)).sum().backward()

    qn, kn, xn = (t.detach().numpy().astype(np.float32) for t in (q, k, x))
    out, attn = oracle.gat_forward(indptr, indices, qn, kn, xn)
    assert_close(out, y.detach().numpy(), rtol=2e-6, what="gat out")
    assert_close(attn, attn_d.detach().numpy()[:, rows, indices].T, rtol=2e-6, what="attn")
    gq, gk, gx = oracle.gat_backward(indptr, indices, qn, kn, xn, attn, g)
    assert_close(gq, q.grad.numpy(), rtol=5e-6, what="grad q")
    assert_close(gk, k.grad.numpy(), rtol=5e-6, what="grad k")
    assert_close(gx, x.grad.numpy(), rtol=5e-6, what="grad x")
    # edge-value gradient of gspmm alone (check_gspmm): d/d values of sum(out * g)
    ga, _ = oracle.spmm_backward(attn, indptr, indices, xn, g)
    ref_ga = np.einsum("ehf,ehf->eh", g[rows].astype(np.float64), xn[indices].astype(np.float64))
    assert_close(ga, ref_ga, rtol=2e-6, what="grad values")


def test_reference_identity_stitch(oracle):
    """Sum over relations of (sddmm, spmm) equals the stitched (sddmm, spmm) (check_stitch)."""
    rng = np.random.default_rng(5)
    n_dst, H, F = 40, 3, 7
    blocks, qs, ks, xs = [], [], [], []
    for b in range(3):
        n_src = 20 + 9 * b
        ip, ix = random_csr(rng, n_dst, n_src, density=0.15)
        blocks.append((ip, ix, n_src))
        qs.append(rng.standard_normal((n_dst, H)).astype(np.float32))
        ks.append(rng.standard_normal((n_src, H)).astype(np.float32))
        xs.append(rng.standard_normal((n_src, H, F)).astype(np.float32))
    total = sum(oracle.gat_forward(ip, ix, q, k, x)[0].astype(np.float64)
                for (ip, ix, _), q, k, x in zip(blocks, qs, ks, xs))
    sip, six, n_cols = oracle.stitch_csr(blocks)
    attn = oracle.sddmm_forward(sip, six, np.stack(qs), np.concatenate(ks))
    out = oracle.spmm(sip, six, np.concatenate(xs), n_heads=H, wmode=oracle.W_EDGE_HEAD, values=attn,
                      index_mask=0xFFFFFF)
    assert_close(out, total, rtol=2e-6, what="stitched vs per-relation")
    # per-(row, segment) weights sum to one wherever the segment has edges
    seg = (six.astype(np.uint32) >> 24).astype(np.int64)
    rows = np.repeat(np.arange(n_dst), np.diff(sip))
    sums = np.zeros((n_dst, 3, H))
    np.add.at(sums, (rows, seg), attn)
    present = np.zeros((n_dst, 3), dtype=bool)
    present[rows, seg] = True
    assert np.allclose(sums[present], 1.0, atol=1e-6)


def test_partition_rows(oracle):
    rng = np.random.default_rng(8)
    indptr, _ = random_csr(rng, 500, 300, density=0.05, hubs=3, hub_deg=250)
    nnz = int(indptr[-1])
    for parts in (1, 2, 3, 8, 16):
        b = oracle.partition_rows(indptr, parts)
        targets = [-(-p * nnz // parts) for p in range(parts)]
        expect = np.searchsorted(indptr, targets, side="left")
        expect[0] = 0
        assert b.tolist() == expect.tolist() + [500]
        assert np.all(np.diff(b) >= 0)
    assert oracle.partition_rows(indptr.astype(np.int64), 8).tolist() == oracle.partition_rows(indptr, 8).tolist()
