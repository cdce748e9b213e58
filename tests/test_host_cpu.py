"""Host-side logic of the product without a GPU: the C-ABI library loads and exports every declared symbol, the
host tables (build_part, stitch_csr, row partition) match the reference's outputs bit for bit, the drop-in
modules enforce the reference's input contract, and the graph generator is reproducible."""
import json
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def _golden(name):
    with open(os.path.join(GOLDEN, name + ".json")) as f:
        return json.load(f)


def test_library_exports_every_declared_symbol():
    from yitu_b200 import _lib
    header = open(os.path.join(ROOT, "include", "yitu_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(yitu_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 20
    L = _lib.lib()
    for name in declared:
        assert hasattr(L, name), "libyitu_b200.so does not export %s" % name
    assert declared == set(_lib.SYMBOLS), "ctypes table and header disagree: %s" % (declared ^ set(_lib.SYMBOLS))
    assert L.yitu_version() >= 100
    assert L.yitu_status_string(0) == b"ok"
    assert L.yitu_static_scratch_bytes() == 16 << 20


def test_struct_layouts_match_the_header(tmp_path):
    """Sizes and field offsets the C compiler gives the argument structs of the header, against the ctypes
    mirrors: a moved or missing field in either place fails here."""
    import ctypes as C
    import subprocess
    from yitu_b200 import _lib
    mirrors = {"yitu_csr_t": _lib.Csr, "yitu_hub_plan_t": _lib.HubPlan, "yitu_spmm_args_t": _lib.SpmmArgs,
               "yitu_gat_args_t": _lib.GatArgs, "yitu_gat_bwd_args_t": _lib.GatBwdArgs}
    lines = []
    for cname, cls in mirrors.items():
        lines.append('printf("%s %%zu\\n", sizeof(%s));' % (cname, cname))
        for fname, _ in cls._fields_:
            lines.append('printf("%s.%s %%zu\\n", offsetof(%s, %s));' % (cname, fname, cname, fname))
    src = tmp_path / "layout.c"
    src.write_text('#include <stddef.h>\n#include <stdio.h>\n#include "yitu_b200.h"\nint main(void) {\n%s\nreturn 0; }\n'
                   % "\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    got = dict(l.split() for l in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for cname, cls in mirrors.items():
        assert int(got[cname]) == C.sizeof(cls), cname
        for fname, _ in cls._fields_:
            assert int(got["%s.%s" % (cname, fname)]) == getattr(cls, fname).offset, (cname, fname)


def test_build_part_bit_identical_to_reference():
    from yitu_b200 import YiTu_GNN_kernel as K
    for case in _golden("build_part"):
        pp, p2n = K.build_part(case["part_size"], torch.IntTensor(case["indptr"]))
        assert pp.dtype == torch.float32 and p2n.dtype == torch.float32 and not pp.is_cuda
        assert pp.tolist() == case["part_ptr"] and p2n.tolist() == case["part2node"], case
    with pytest.raises(RuntimeError):
        K.build_part(32, torch.tensor([0, 1], dtype=torch.int64))


def test_stitch_csr_bit_identical_to_reference():
    from yitu_b200.xgnn_h import Block, stitch_csr
    for case in _golden("stitch_csr"):
        blocks = [Block([case["n_rows"], b["n_cols"]], [torch.IntTensor(b["indptr"]), torch.IntTensor(b["indices"])])
                  for b in case["blocks"]]
        st = stitch_csr(blocks)
        assert st.size == case["size"]
        assert st.adj_sparse[0].dtype == torch.int32 and st.adj_sparse[1].dtype == torch.int32
        assert st.adj_sparse[0].tolist() == case["indptr"] and st.adj_sparse[1].tolist() == case["indices"]
        assert st.num_edges() == len(case["indices"]) and st.num_dst_nodes() == case["n_rows"]


def test_stitch_csr_limits():
    from yitu_b200.xgnn_h import Block, stitch_csr
    one = Block([1, 1], [torch.IntTensor([0, 1]), torch.IntTensor([0])])
    with pytest.raises(AssertionError):
        stitch_csr([one] * 17)
    with pytest.raises(AssertionError):  # unequal row counts
        stitch_csr([one, Block([2, 1], [torch.IntTensor([0, 1, 1]), torch.IntTensor([0])])])
    big = Block([1, (1 << 24) + 5], [torch.IntTensor([0, 1]), torch.IntTensor([(1 << 24) + 3])])
    with pytest.raises(AssertionError):  # column beyond 2^24, as the reference asserts
        stitch_csr([big])
    # the boundary: column 2^24 - 1 is the largest that leaves the segment tag intact.  The reference's
    # `assert col <= 2**24` lets 2^24 itself through, where it turns into column 0 of the next relation; rejected here.
    edge = Block([1, 1 << 24], [torch.IntTensor([0, 1]), torch.IntTensor([(1 << 24) - 1])])
    assert stitch_csr([edge]).adj_sparse[1].tolist() == [(1 << 24) - 1]
    with pytest.raises(AssertionError):  # shifted by the one column of the block before it: exactly 2^24
        stitch_csr([one, edge])


def test_partition_rows_host(oracle):
    from yitu_b200 import ops
    rng = np.random.default_rng(4)
    deg = rng.integers(0, 50, size=999)
    deg[::97] = 3000
    indptr = np.concatenate([[0], np.cumsum(deg)])
    for dtype in (torch.int32, torch.int64):
        for parts in (1, 2, 4, 8, 13):
            got = ops.partition_rows_host(torch.from_numpy(indptr).to(dtype), parts)
            assert got.tolist() == oracle.partition_rows(indptr.astype(np.int64), parts).tolist()


def test_operators_reject_cpu_tensors():
    """The reference's CHECK_INPUT (ccsrc/kernel/YiTu_GNN.cpp:65-69, YiTu_H/src/common.h:6-12) raises for
    non-CUDA tensors; so do the drop-in modules, before anything touches a device."""
    from yitu_b200 import YiTu_GNN_kernel as K, graph_ext
    x = torch.randn(4, 8)
    ip = torch.tensor([0, 1, 2, 3, 4], dtype=torch.int32)
    ix = torch.tensor([0, 1, 2, 3], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        K.forward(x, torch.randn(8, 2), ip, ix, torch.ones(4), ip, ix, 32, 32, 2)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        graph_ext.spmm_forward(torch.randn(4, 1), ip, ix, x.view(4, 1, 8))
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        graph_ext.sddmm_forward(ip, ix, torch.randn(1, 4, 2), torch.randn(4, 2))


def test_install_as_reference_modules():
    import sys
    import yitu_b200
    saved = {k: sys.modules.get(k) for k in ("graph_ext", "YiTu_GNN", "YiTu_GNN.YiTu_GNN_kernel", "YiTu_GNN.rabbit")}
    try:
        yitu_b200.install_as_reference_modules()
        import graph_ext
        from YiTu_GNN import YiTu_GNN_kernel
        for fn in ("spmm_forward", "spmm_backward", "sddmm_forward", "sddmm_backward", "hfused_forward",
                   "hfused_backward", "b2gemm", "b2gemm_backward"):
            assert callable(getattr(graph_ext, fn))
        for fn in ("SAG", "forward", "backward", "forward_gin", "backward_gin", "build_part"):
            assert callable(getattr(YiTu_GNN_kernel, fn))
        from YiTu_GNN import rabbit
        assert callable(rabbit.reorder)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


# ------------------------------------------------------------------------------------------- generators
def _mix64_numpy(z):
    z = z.astype(np.uint64)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def test_mixer_matches_unsigned_reference_implementation():
    from yitu_b200 import graphs
    idx = torch.arange(0, 5000, dtype=torch.int64) * 7919 - 12345
    got = graphs._mix64(idx).numpy().view(np.uint64)
    with np.errstate(over="ignore"):
        assert np.array_equal(got, _mix64_numpy(idx.numpy().view(np.uint64)))


def test_graph_generators_are_reproducible_and_canonical():
    from yitu_b200 import graphs
    a = graphs.gcn_small(n=4096, e=40000, seed=0)
    b = graphs.gcn_small(n=4096, e=40000, seed=0)
    c = graphs.gcn_small(n=4096, e=40000, seed=1)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert not torch.equal(a[1][:1000], c[1][:1000])
    indptr, indices, norm = a
    assert indptr.dtype == torch.int32 and indices.dtype == torch.int32
    ip, ix = indptr.numpy(), indices.numpy()
    for r in (0, 1, 17, 4095):
        row = ix[ip[r]:ip[r + 1]]
        assert np.all(np.diff(row) > 0), "columns must be ascending and unique within a row"
        assert r in row, "self-loop present"
    deg = np.diff(ip)
    assert np.allclose(norm.numpy(), 1.0 / np.sqrt(deg), rtol=1e-6)
    assert deg.max() > 20 * deg.mean(), "R-MAT skew expected"
    # chunked generation does not change the stream
    s1, d1 = graphs.rmat_edges(3, 1000, 700, 5000, chunk=1 << 25)
    s2, d2 = graphs.rmat_edges(3, 1000, 700, 5000, chunk=777)
    assert torch.equal(s1, s2) and torch.equal(d1, d2)
    assert int(s1.max()) < 1000 and int(d1.max()) < 700 and int(s1.min()) >= 0
    x = graphs.randn_features(5, 2000, 64)
    assert abs(float(x.mean())) < 0.02 and abs(float(x.std()) - 1.0) < 0.02
    rels = graphs.hetero_rgcn(type_sizes=(500, 300, 200, 100), e_per_rel=2000)
    assert len(rels) == 8 and {r[1] for r in rels} == {0, 1, 2, 3}
    for st, dt, ipr, ixr in rels:
        assert ipr.numel() == (500, 300, 200, 100)[dt] + 1 and int(ixr.max()) < (500, 300, 200, 100)[st]


# ------------------------------------------------------------------------------------------- properties
from hypothesis import given, settings, strategies as st


@settings(max_examples=60, deadline=None)
@given(degs=st.lists(st.integers(0, 70), min_size=0, max_size=40), part_size=st.sampled_from([1, 2, 3, 8, 32]))
def test_build_part_matches_checker_on_random_degrees(degs, part_size):
    from oracle import oracle as O
    from yitu_b200 import YiTu_GNN_kernel as K
    indptr = np.concatenate([[0], np.cumsum(degs)]).astype(np.int32)
    pp, p2n = K.build_part(part_size, torch.from_numpy(indptr))
    opp, op2n = O.build_part(part_size, indptr)
    assert pp.tolist() == opp.tolist() and p2n.tolist() == op2n.tolist()
    # group table invariants (when the last node has edges): monotone pointers that tile every row
    if len(degs) and degs[-1] > 0:
        ptr = pp.numpy().astype(np.int64)
        assert ptr[0] == 0 and ptr[-1] == indptr[-1] and np.all(np.diff(ptr) >= 1) and np.all(np.diff(ptr) <= part_size)
        assert np.array_equal(np.bincount(p2n.numpy().astype(np.int64), minlength=len(degs)),
                              -(-np.asarray(degs) // part_size))


@settings(max_examples=40, deadline=None)
@given(data=st.data())
def test_stitch_csr_matches_checker_on_random_blocks(data):
    from oracle import oracle as O
    from yitu_b200.xgnn_h import Block, stitch_csr
    n_rows = data.draw(st.integers(0, 12))
    blocks = []
    for _ in range(data.draw(st.integers(1, 5))):
        n_cols = data.draw(st.integers(1, 9))
        rows = [sorted(data.draw(st.sets(st.integers(0, n_cols - 1), max_size=n_cols))) for _ in range(n_rows)]
        indptr = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int32)
        indices = np.asarray([c for r in rows for c in r], dtype=np.int32)
        blocks.append((indptr, indices, n_cols))
    st_blk = stitch_csr([Block([n_rows, c], [torch.from_numpy(a), torch.from_numpy(b)]) for a, b, c in blocks])
    o_ip, o_ix, o_cols = O.stitch_csr(blocks)
    assert st_blk.adj_sparse[0].tolist() == o_ip.tolist() and st_blk.adj_sparse[1].tolist() == o_ix.tolist()
    assert st_blk.size == [n_rows, o_cols]
    # every stitched index decodes to (block, column) of exactly one input edge, in block order within a row
    ix = st_blk.adj_sparse[1].numpy().astype(np.int64)
    seg = ix >> 24
    ip = st_blk.adj_sparse[0].numpy()
    for r in range(n_rows):
        assert np.all(np.diff(seg[ip[r]:ip[r + 1]]) >= 0)


@settings(max_examples=60, deadline=None)
@given(degs=st.lists(st.integers(0, 500), min_size=1, max_size=60), parts=st.integers(1, 9))
def test_partition_rows_properties(degs, parts):
    from oracle import oracle as O
    from yitu_b200 import ops
    indptr = np.concatenate([[0], np.cumsum(degs)]).astype(np.int64)
    b = ops.partition_rows_host(torch.from_numpy(indptr), parts).numpy()
    assert b.tolist() == O.partition_rows(indptr, parts).tolist()
    assert b[0] == 0 and b[-1] == len(degs) and np.all(np.diff(b) >= 0)
    nnz = int(indptr[-1])
    for p in range(1, parts):
        target = -(-p * nnz // parts)
        assert indptr[b[p]] >= target and (b[p] == 0 or indptr[b[p] - 1] < target)


def test_cost_aware_partition_balances_edges_plus_rows():
    from yitu_b200.distributed import partition_bounds
    rng = np.random.default_rng(6)
    deg = np.concatenate([rng.integers(200, 400, size=50), rng.integers(0, 3, size=5000)])  # hubs first, then a long tail
    indptr = torch.from_numpy(np.concatenate([[0], np.cumsum(deg)]).astype(np.int64))
    plain = partition_bounds(indptr, 4)
    aware = partition_bounds(indptr, 4, row_cost=7)
    assert plain[0] == aware[0] == 0 and plain[-1] == aware[-1] == len(deg)
    cost = indptr.numpy() + 7 * np.arange(len(deg) + 1)
    for p in range(1, 4):
        target = -(-p * int(cost[-1]) // 4)
        assert cost[aware[p]] >= target and cost[aware[p] - 1] < target
    rows_plain = np.diff(plain)
    rows_aware = np.diff(aware)
    assert rows_aware.max() < rows_plain.max(), "weighing rows must shrink the largest shard of a skewed graph"


def test_operator_wrappers_reject_bad_tensors_before_any_launch():
    """The tensor-level wrappers hand raw pointers to the kernels; sizes, dtypes, layout and device are checked on
    the host first.  One rejection per operator, on CPU tensors: the check fires before anything is launched."""
    from yitu_b200 import ops
    ip = torch.tensor([0, 2, 3, 3, 5], dtype=torch.int32)
    ix = torch.tensor([0, 1, 2, 0, 2], dtype=torch.int32)
    g = ops.PreparedGraph(ip, ix, 3)
    x = torch.zeros(3, 8)
    xh = torch.zeros(3, 2, 4)
    with pytest.raises(RuntimeError, match="edge_values must hold 5"):
        ops.spmm(g, x, mode=ops.W_EDGE, edge_values=torch.zeros(4))
    with pytest.raises(RuntimeError, match="edge_values must hold 10"):
        ops.spmm(g, xh, n_heads=2, mode=ops.W_EDGE_HEAD, edge_values=torch.zeros(5, 1))
    with pytest.raises(RuntimeError, match="needs edge_values"):
        ops.spmm(g, x, mode=ops.W_EDGE)
    with pytest.raises(RuntimeError, match="norm_src must hold 3"):
        ops.spmm(g, x, mode=ops.W_NODE, norm_dst=torch.zeros(4), norm_src=torch.zeros(4))
    with pytest.raises(RuntimeError, match="row_scale must hold 4"):
        ops.spmm(g, x, row_scale=torch.zeros(3))
    with pytest.raises(RuntimeError, match="edge_perm must have dtype"):
        ops.spmm(g, x, mode=ops.W_EDGE, edge_values=torch.zeros(5), edge_perm=torch.zeros(5, dtype=torch.int64))
    with pytest.raises(RuntimeError, match="source nodes"):
        ops.spmm(g, torch.zeros(4, 8))
    with pytest.raises(RuntimeError, match="out must hold"):
        ops.spmm(g, x, out=torch.zeros(3, 8))
    with pytest.raises(RuntimeError, match="grad_out must have shape"):
        ops.edge_dot(g, torch.zeros(3, 2, 4), xh)
    with pytest.raises(RuntimeError, match="values must have shape"):
        ops.spmm_bwd(g, torch.zeros(5, 1), xh, torch.zeros(4, 2, 4))
    with pytest.raises(RuntimeError, match="query must have shape"):
        ops.edge_softmax_fwd(g, torch.zeros(1, 3, 2), torch.zeros(3, 2))
    with pytest.raises(RuntimeError, match="grad_attn must have shape"):
        ops.edge_softmax_bwd(g, torch.zeros(1, 4, 2), torch.zeros(3, 2), torch.zeros(5, 2), torch.zeros(4, 2))
    with pytest.raises(RuntimeError, match="key must have shape"):
        ops.gat_fwd(g, torch.zeros(4, 2), torch.zeros(4, 2), xh)
    with pytest.raises(RuntimeError, match="row_max must have shape"):
        ops.gat_bwd(g, torch.zeros(4, 2), torch.zeros(3, 2), xh, torch.zeros(4, 2, 4), torch.zeros(3, 2),
                    torch.zeros(4, 2), torch.zeros(4, 2, 4))
    if torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="the graph is on"):
            ops.spmm(g, x.cuda())


def test_prepared_graph_is_found_by_memory_not_by_tensor_object():
    """Reference-style callers pass a fresh tensor object per call (a view of the same storage): the derived
    structures must be built once.  An in-place edit of the tables leads to a new build."""
    from yitu_b200 import ops
    ip = torch.tensor([0, 2, 3, 3, 5], dtype=torch.int32)
    ix = torch.tensor([0, 1, 2, 0, 2], dtype=torch.int32)
    g1 = ops.prepared(ip, ix, 3)
    g2 = ops.prepared(ip.view(-1), ix[:], 3)          # distinct tensor objects, same memory
    g3 = ops.prepared(ip.detach(), ix.detach(), 3, 0)
    assert g1 is g2 and g1 is g3
    assert ops.prepared(ip, ix, 3, ops.STITCH_MASK) is not g1   # another mask: another entry
    assert ops.prepared(ip.clone(), ix, 3) is not g1            # other memory
    ix[0] = 1                                                    # in-place edit bumps the version counter
    assert ops.prepared(ip, ix, 3) is not g1


def test_fused_gat_route_is_closed_for_stitched_blocks():
    """A stitched block carries relation ids in the top index bits; the fused GAT kernels would read them as column
    ids.  stitch_csr marks its result, a Block built from raw packed tensors is inspected once."""
    from yitu_b200.xgnn_h import Block, stitch_csr
    a = Block([2, 3], [torch.IntTensor([0, 1, 2]), torch.IntTensor([0, 2])])
    b = Block([2, 2], [torch.IntTensor([0, 1, 1]), torch.IntTensor([1])])
    assert a.is_stitched() is False
    st = stitch_csr([a, b])
    assert st.stitched is True and st.is_stitched() is True
    assert stitch_csr([a]).is_stitched() is False
    raw = Block(st.size, [st.adj_sparse[0].clone(), st.adj_sparse[1].clone()])
    assert raw.stitched is None and raw.is_stitched() is True
