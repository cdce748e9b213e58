"""The reference's own CUDA kernels (YiTu_GNN/YiTu_H/src, compiled unmodified for sm_100a into oracle/_ref by
`make -C oracle ref_gpu`) run on the GPU against the CPU checker and against this library, on seeded inputs inside
the reference's launch limits (at most 65535 destination rows, spmm_cuda.cu:57).  This pins the checker's
floating-point restatement to the reference itself.  Skipped where the reference build is absent."""
import glob
import importlib
import os
import sys

import numpy as np
import pytest
import torch

from conftest import assert_close, random_csr

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


@pytest.fixture(scope="module")
def ref_ext():
    if not glob.glob(os.path.join(REF_DIR, "graph_ext_ref*.so")):
        pytest.skip("reference graph_ext not built (make -C oracle ref_gpu)")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module("graph_ext_ref")


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("H,F,seed", [(1, 64, 0), (8, 32, 1), (3, 5, 2), (4, 16, 3), (16, 8, 4), (2, 100, 5)])
def test_reference_spmm_kernels(oracle, ref_ext, H, F, seed):
    from yitu_b200 import graph_ext
    rng = np.random.default_rng(seed)
    n_dst, n_src = 301, 257
    indptr, indices = random_csr(rng, n_dst, n_src, density=0.05, hubs=2, hub_deg=200)
    vals = rng.standard_normal((indices.shape[0], H)).astype(np.float32)
    x = rng.standard_normal((n_src, H, F)).astype(np.float32)
    g = rng.standard_normal((n_dst, H, F)).astype(np.float32)
    ip, ix, dv, dx, dg = _dev(indptr), _dev(indices), _dev(vals), _dev(x), _dev(g)
    ref_out = ref_ext.spmm_forward(dv, ip, ix, dx)
    ref_ga, ref_gx = ref_ext.spmm_backward(dv, ip, ix, dx, dg)
    torch.cuda.synchronize()
    o_out = oracle.spmm(indptr, indices, x, n_heads=H, wmode=oracle.W_EDGE_HEAD, values=vals, index_mask=0xFFFFFF)
    o_ga, o_gx = oracle.spmm_backward(vals, indptr, indices, x, g)
    # the reference accumulates in fp32 (serially forward, by atomics backward): 2e-5 covers its own rounding
    assert_close(ref_out.cpu().numpy(), o_out, rtol=2e-5, what="reference spmm_forward vs checker")
    assert_close(ref_ga.cpu().numpy(), o_ga, rtol=2e-5, what="reference grad_a vs checker")
    assert_close(ref_gx.cpu().numpy(), o_gx, rtol=2e-5, what="reference grad_x vs checker")
    out = graph_ext.spmm_forward(dv, ip, ix, dx)
    ga, gx = graph_ext.spmm_backward(dv, ip, ix, dx, dg)
    assert_close(out.cpu().numpy(), ref_out.cpu().numpy(), rtol=2e-5, what="spmm_forward vs reference kernel")
    assert_close(ga.cpu().numpy(), ref_ga.cpu().numpy(), rtol=2e-5, what="grad_a vs reference kernel")
    assert_close(gx.cpu().numpy(), ref_gx.cpu().numpy(), rtol=2e-5, what="grad_x vs reference kernel")


@pytest.mark.parametrize("H,B,seed", [(1, 1, 0), (8, 1, 1), (5, 1, 2), (16, 1, 3), (4, 3, 4), (8, 2, 5)])
def test_reference_sddmm_kernels(oracle, ref_ext, H, B, seed):
    from yitu_b200 import graph_ext
    rng = np.random.default_rng(100 + seed)
    n_dst = 211
    blocks = []
    for b in range(B):
        ip, ix = random_csr(rng, n_dst, 90 + 20 * b, density=0.08, hubs=1, hub_deg=70)
        blocks.append((ip, ix, 90 + 20 * b))
    indptr, indices, n_src = blocks[0] if B == 1 else oracle.stitch_csr(blocks)
    q = rng.standard_normal((B, n_dst, H)).astype(np.float32)
    k = rng.standard_normal((n_src, H)).astype(np.float32)
    g = rng.standard_normal((indices.shape[0], H)).astype(np.float32)
    ip, ix, dq, dk, dg = _dev(indptr), _dev(indices), _dev(q), _dev(k), _dev(g)
    ref_attn = ref_ext.sddmm_forward(ip, ix, dq, dk)
    ref_gq, ref_gk = ref_ext.sddmm_backward(ip, ix, dq, dk, ref_attn, dg)
    torch.cuda.synchronize()
    o_attn = oracle.sddmm_forward(indptr, indices, q, k)
    o_gq, o_gk = oracle.sddmm_backward(indptr, indices, q, k, ref_attn.cpu().numpy(), g)
    assert_close(ref_attn.cpu().numpy(), o_attn, rtol=2e-5, what="reference sddmm_forward vs checker")
    assert_close(ref_gq.cpu().numpy(), o_gq, rtol=2e-5, what="reference grad_query vs checker")
    assert_close(ref_gk.cpu().numpy(), o_gk, rtol=2e-5, what="reference grad_key vs checker")
    attn = graph_ext.sddmm_forward(ip, ix, dq, dk)
    gq, gk = graph_ext.sddmm_backward(ip, ix, dq, dk, ref_attn, dg)
    assert_close(attn.cpu().numpy(), ref_attn.cpu().numpy(), rtol=2e-5, what="sddmm_forward vs reference kernel")
    assert_close(gq.cpu().numpy(), ref_gq.cpu().numpy(), rtol=2e-5, what="grad_query vs reference kernel")
    assert_close(gk.cpu().numpy(), ref_gk.cpu().numpy(), rtol=2e-5, what="grad_key vs reference kernel")


@pytest.fixture(scope="module")
def ref_ccsrc():
    if not glob.glob(os.path.join(REF_DIR, "yitu_gnn_kernel_ref*.so")):
        pytest.skip("reference YiTu_GNN_kernel not built (make -C oracle ref_gpu_ccsrc)")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module("yitu_gnn_kernel_ref")


def _symmetric_graph(rng, n, density):
    dense = rng.random((n, n)) < density
    dense = dense | dense.T
    np.fill_diagonal(dense, True)
    indptr = np.concatenate([[0], np.cumsum(dense.sum(1))]).astype(np.int32)
    indices = np.nonzero(dense)[1].astype(np.int32)
    return indptr, indices


@pytest.mark.parametrize("n,d_in,d_out,seed", [(300, 48, 16, 0), (777, 64, 64, 1), (1500, 20, 7, 2)])
def test_reference_ccsrc_kernels(oracle, ref_ccsrc, n, d_in, d_out, seed):
    """GCN forward/backward, GIN forward/backward and SAG of the reference extension on a symmetric graph (the only
    kind on which its backward is the gradient), against the CPU checker and against the drop-in module."""
    from yitu_b200 import YiTu_GNN_kernel as K
    rng = np.random.default_rng(200 + seed)
    indptr, indices = _symmetric_graph(rng, n, 0.02)
    deg = np.diff(indptr).astype(np.float32)
    norm = (1.0 / np.sqrt(deg)).astype(np.float32)
    x = rng.standard_normal((n, d_in)).astype(np.float32)
    w = (rng.standard_normal((d_in, d_out)) * 0.2).astype(np.float32)
    g = rng.standard_normal((n, d_out)).astype(np.float32)
    pp, p2n = ref_ccsrc.build_part(32, torch.from_numpy(indptr))
    mine_pp, mine_p2n = K.build_part(32, torch.from_numpy(indptr))
    assert torch.equal(pp, mine_pp) and torch.equal(p2n, mine_p2n)
    graph = (_dev(indptr), _dev(indices), _dev(norm), pp.int().cuda(), p2n.int().cuda(), 32, 32, 2)
    dx, dw, dg = _dev(x), _dev(w), _dev(g)

    ref_out = ref_ccsrc.forward(dx, dw, *graph)[0]
    ref_din, ref_dw = ref_ccsrc.backward(dg, dx, dw, *graph)
    torch.cuda.synchronize()
    o_out = oracle.gcn_forward(x, w, indptr, indices, norm)
    o_din, o_dw = oracle.gcn_backward(g, x, w, indptr, indices, norm, transpose=False)
    assert_close(ref_out.cpu().numpy(), o_out, rtol=2e-5, what="reference GCN forward vs checker")
    assert_close(ref_din.cpu().numpy(), o_din, rtol=3e-5, what="reference GCN d_input vs checker")
    assert_close(ref_dw.cpu().numpy(), o_dw, rtol=3e-5, what="reference GCN d_weight vs checker")
    out = K.forward(dx, dw, *graph)[0]
    din, dwt = K.backward(dg, dx, dw, *graph)
    assert_close(out.cpu().numpy(), ref_out.cpu().numpy(), rtol=2e-5, what="GCN forward vs reference kernel")
    assert_close(din.cpu().numpy(), ref_din.cpu().numpy(), rtol=3e-5, what="GCN d_input vs reference kernel")
    assert_close(dwt.cpu().numpy(), ref_dw.cpu().numpy(), rtol=3e-5, what="GCN d_weight vs reference kernel")

    ref_sag = ref_ccsrc.SAG(dx, *graph)
    assert_close(ref_sag.cpu().numpy(), oracle.spmm(indptr, indices, x), rtol=2e-5, what="reference SAG vs checker")
    assert_close(K.SAG(dx, *graph).cpu().numpy(), ref_sag.cpu().numpy(), rtol=2e-5, what="SAG vs reference kernel")

    gin_graph = (graph[0], graph[1], 0.5) + graph[3:]
    ref_o, ref_agg = ref_ccsrc.forward_gin(dx, dw, *gin_graph)
    o_o, o_agg = oracle.gin_forward(x, w, indptr, indices, 0.5)
    assert_close(ref_agg.cpu().numpy(), o_agg, rtol=2e-5, what="reference GIN aggregate vs checker")
    assert_close(ref_o.cpu().numpy(), o_o, rtol=3e-5, what="reference GIN output vs checker")
    mine_o, mine_agg = K.forward_gin(dx, dw, *gin_graph)
    assert_close(mine_agg.cpu().numpy(), ref_agg.cpu().numpy(), rtol=2e-5, what="GIN aggregate vs reference kernel")
    ref_gi, ref_gw = ref_ccsrc.backward_gin(dg, ref_agg, dw, *gin_graph)
    mine_gi, mine_gw = K.backward_gin(dg, ref_agg, dw, *gin_graph)
    assert_close(mine_gi.cpu().numpy(), ref_gi.cpu().numpy(), rtol=3e-5, what="GIN d_input vs reference kernel")
    assert_close(mine_gw.cpu().numpy(), ref_gw.cpu().numpy(), rtol=3e-5, what="GIN d_weight vs reference kernel")
