"""yitu_spmm_csr_f32_static: the SpMM entry point for callers that cannot allocate device memory (fixed
memory budgets, plugins that only receive buffers, loops that must not touch the allocator).  Its hub-row
partial sums live in a 16 MiB array inside the library.  Checked here through the C ABI against the regular
entry point on two consecutive calls (the array is shared and keeps the previous call's contents), and for
its size limit.  This file sorts last on purpose: a run that stops at the first failure has by then run
every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(ops, lib_mod, g, x, out, values, plan):
    a = lib_mod.SpmmArgs()
    a.graph = g.csr
    a.n_heads, a.n_feats = 1, x.size(1)
    a.weight_mode, a.accumulate = lib_mod.W_EDGE, 0
    a.edge_values = C.c_void_p(values.data_ptr())
    a.alpha = 1.0
    a.x, a.x_stride = C.c_void_p(x.data_ptr()), x.size(1)
    a.out, a.out_stride = C.c_void_p(out.data_ptr()), x.size(1)
    if plan is not None:
        a.plan = C.pointer(plan[0])
    return a


def test_static_scratch_spmm_matches_regular_entry_point():
    from yitu_b200 import _lib, graphs, ops
    L = _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n, d = 1 << 15, 128
    indptr, indices, values = graphs.spmm_rmat(device=dev, n=n, e=1 << 20, seed=9)
    g = ops.PreparedGraph(indptr, indices, n)
    plan = g.plan(64)
    assert plan is not None and plan[0].n_chunks > 100, "the test graph must have split hub rows"
    assert plan[0].n_chunks * d * 4 <= L.yitu_static_scratch_bytes()
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    for seed in (1, 2):  # two calls in a row: the second finds the first call's partial sums in the array
        x = graphs.randn_features(seed, n, d, device=dev)
        ref = torch.empty(n, d, device=dev)
        scratch = torch.empty(plan[0].n_chunks * d, device=dev)
        a = _args(ops, _lib, g, x, ref, values, plan)
        a.scratch, a.scratch_bytes = C.c_void_p(scratch.data_ptr()), scratch.numel() * 4
        _lib.check(L.yitu_spmm_csr_f32(C.byref(a), stream))
        got = torch.full((n, d), float("nan"), device=dev)
        b = _args(ops, _lib, g, x, got, values, plan)
        _lib.check(L.yitu_spmm_csr_f32_static(C.byref(b), stream))
        torch.cuda.synchronize()
        ref_np, got_np = ref.cpu().numpy(), got.cpu().numpy()
        scale = np.abs(ref_np).max()
        assert np.isfinite(got_np).all()
        assert np.abs(got_np - ref_np).max() <= 1e-5 * scale  # same kernels, same order: expected identical
        assert torch.equal(got, ref)


def test_static_scratch_rejects_oversized_schedule():
    from yitu_b200 import _lib, graphs, ops
    L = _lib.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n, d = 1 << 15, 512
    indptr, indices, values = graphs.spmm_rmat(device=dev, n=n, e=1 << 21, seed=10)
    g = ops.PreparedGraph(indptr, indices, n)
    plan = g.plan(32)
    assert plan[0].n_chunks * d * 4 > L.yitu_static_scratch_bytes(), "schedule must exceed the built-in scratch"
    x = torch.zeros(n, d, device=dev)
    out = torch.zeros(n, d, device=dev)
    a = _args(ops, _lib, g, x, out, values, plan)
    rc = L.yitu_spmm_csr_f32_static(C.byref(a), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    assert rc == _lib.ERR_LIMIT
    assert b"built-in scratch" in L.yitu_last_error()
