"""numpy front end of the CPU checker (oracle/yitu_oracle.c).

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by __graft_entry__.smoke() and by the
CPU-baseline / reference legs of bench.py; nothing in the yitu_b200 package may import it.

Each function cites the reference code whose arithmetic it restates; the C file carries the
loop-level citations.  Floating-point results are accumulated in float64 and rounded once.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libyitu_oracle.so")

W_NONE, W_NODE, W_EDGE, W_EDGE_HEAD, W_SEG_MEAN = 0, 1, 2, 3, 4


def build(force=False):
    """Compile the C checker next to its source (gcc + OpenMP)."""
    src = os.path.join(_HERE, "yitu_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libyitu_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.yo_build_part_count.restype = C.c_int64
        _lib.yo_stitch_csr.restype = C.c_int64
    return _lib


def set_threads(n):
    """Use n OpenMP threads from now on, whatever OMP_NUM_THREADS said when the process started."""
    lib().yo_set_threads(C.c_int(int(n)))
    return lib().yo_max_threads()


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def _ptr_arr(indptr):
    a = np.ascontiguousarray(indptr)
    if a.dtype == np.int64:
        return a, 1
    return np.ascontiguousarray(a, dtype=np.int32), 0


# ----------------------------------------------------------------------------------------------
def build_part(part_size, indptr):
    """ccsrc/kernel/YiTu_GNN.cpp:203-245 -> (partPtr float32[P+1], part2Node float32[P])."""
    indptr = _i32(indptr)
    n = indptr.shape[0] - 1
    P = lib().yo_build_part_count(C.c_int(part_size), _p(indptr), C.c_int64(n))
    part_ptr = np.zeros(P + 1, dtype=np.float32)
    part2node = np.zeros(P, dtype=np.float32)
    lib().yo_build_part(C.c_int(part_size), _p(indptr), C.c_int64(n), _p(part_ptr), _p(part2node))
    return part_ptr, part2node


def spmm(indptr, indices, x, *, n_heads=1, wmode=W_NONE, values=None, perm=None, norm_dst=None,
         norm_src=None, row_scale=None, alpha=1.0, index_mask=0, out=None):
    """out[r,h,k] = alpha*row_scale[r] * sum_i w(i,h) * x[col_i,h,k]; x is [n_src, H*F] or [n_src,H,F].

    Restates ccsrc/kernel/YiTu_GNN_kernel.cu:319-415 (W_NODE), :620-694 (W_NONE + alpha=epsilon),
    :179-257 (W_NONE) and YiTu_GNN/YiTu_H/src/spmm_cuda.cu:4-21 (W_EDGE_HEAD, index_mask=0xffffff).
    """
    ip, is64 = _ptr_arr(indptr)
    indices = _i32(indices)
    x = _f32(x)
    n_rows = ip.shape[0] - 1
    x2 = x.reshape(x.shape[0], -1)
    D = x2.shape[1]
    H = n_heads
    F = D // H
    accumulate = 0
    if out is None:
        out = np.zeros((n_rows, D), dtype=np.float32)
    else:
        accumulate = 1
        out = np.ascontiguousarray(out, dtype=np.float32).reshape(n_rows, D).copy()
    values, norm_dst, norm_src, row_scale = _f32(values), _f32(norm_dst), _f32(norm_src), _f32(row_scale)
    perm = _i32(perm)
    lib().yo_spmm(C.c_int64(n_rows), C.c_int64(H), C.c_int64(F), _p(ip), C.c_int(is64), _p(indices),
                  C.c_int32(index_mask), C.c_int(wmode), _p(values), _p(perm), _p(norm_dst), _p(norm_src),
                  _p(row_scale), C.c_float(alpha), C.c_int(accumulate), _p(x2), _p(out))
    return out.reshape((n_rows,) + x.shape[1:])


def spmm_transpose(indptr, indices, n_cols, g, *, wmode=W_NONE, values=None, norm_dst=None, norm_src=None,
                   index_mask=0):
    """out[c,:] = sum_{i: col_i=c} w_i * g[row_i,:] — the mathematics of the GCN backward aggregation
    (ccsrc/kernel/YiTu_GNN_kernel.cu:422-475 runs the forward CSR, exact only for symmetric patterns)."""
    ip, is64 = _ptr_arr(indptr)
    indices, g = _i32(indices), _f32(g)
    n_rows = ip.shape[0] - 1
    D = g.shape[1]
    out64 = np.zeros((n_cols, D), dtype=np.float64)
    out = np.zeros((n_cols, D), dtype=np.float32)
    lib().yo_spmm_transpose(C.c_int64(n_rows), C.c_int64(n_cols), C.c_int64(D), _p(ip), C.c_int(is64),
                            _p(indices), C.c_int32(index_mask), C.c_int(wmode), _p(_f32(values)),
                            _p(_f32(norm_dst)), _p(_f32(norm_src)), _p(g), _p(out64), _p(out))
    return out


def spmm_backward(values, indptr, indices, x, grad_out):
    """graph_ext.spmm_backward (YiTu_GNN/YiTu_H/src/spmm_cuda.cu:24-42) -> (grad_a [E,H], grad_x [n_src,H,F])."""
    values, x, g = _f32(values), _f32(x), _f32(grad_out)
    indptr, indices = _i32(indptr), _i32(indices)
    n_rows = indptr.shape[0] - 1
    n_src, H, F = x.shape
    grad_a = np.zeros_like(values)
    gx64 = np.zeros(x.shape, dtype=np.float64)
    grad_x = np.zeros_like(x)
    lib().yo_spmm_backward(C.c_int64(n_rows), C.c_int64(n_src), C.c_int64(H), C.c_int64(F), _p(indptr),
                           _p(indices), _p(values), _p(x), _p(g), _p(grad_a), _p(gx64), _p(grad_x))
    return grad_a, grad_x


def sddmm_forward(indptr, indices, query, key):
    """graph_ext.sddmm_forward (YiTu_GNN/YiTu_H/src/sddmm_cuda.cu:5-33): query [B,n_dst,H], key [n_src,H]."""
    indptr, indices, query, key = _i32(indptr), _i32(indices), _f32(query), _f32(key)
    n_rows = indptr.shape[0] - 1
    H = key.shape[1]
    attn = np.zeros((indices.shape[0], H), dtype=np.float32)
    lib().yo_sddmm_forward(C.c_int64(n_rows), C.c_int64(H), _p(indptr), _p(indices), _p(query), _p(key),
                           _p(attn))
    return attn


def sddmm_backward(indptr, indices, query, key, attn, grad_out):
    """graph_ext.sddmm_backward (YiTu_GNN/YiTu_H/src/sddmm_cuda.cu:36-67) -> (grad_query, grad_key)."""
    indptr, indices = _i32(indptr), _i32(indices)
    query, key, attn, g = _f32(query), _f32(key), _f32(attn), _f32(grad_out)
    n_rows = indptr.shape[0] - 1
    n_src, H = key.shape
    grad_q = np.zeros_like(query)
    gk64 = np.zeros(key.shape, dtype=np.float64)
    grad_k = np.zeros_like(key)
    lib().yo_sddmm_backward(C.c_int64(n_rows), C.c_int64(n_src), C.c_int64(H), _p(indptr), _p(indices),
                            _p(query), _p(key), _p(attn), _p(g), _p(grad_q), _p(gk64), _p(grad_k))
    return grad_q, grad_k


def stitch_csr(blocks):
    """xgnn_h/block.py:36-67.  blocks: list of (indptr, indices, n_cols) with equal row counts (<= 16)."""
    assert len(blocks) <= 16
    ips = [_i32(b[0]) for b in blocks]
    ids = [_i32(b[1]) for b in blocks]
    n_rows = ips[0].shape[0] - 1
    assert all(ip.shape[0] - 1 == n_rows for ip in ips)
    ncols = np.asarray([b[2] for b in blocks], dtype=np.int64)
    total = int(sum(i.shape[0] for i in ids))
    out_ip = np.zeros(n_rows + 1, dtype=np.int32)
    out_id = np.zeros(total, dtype=np.int32)
    PP = C.c_void_p * len(blocks)
    got = lib().yo_stitch_csr(C.c_int(len(blocks)), C.c_int64(n_rows), PP(*[i.ctypes.data for i in ips]),
                              PP(*[i.ctypes.data for i in ids]), _p(ncols), _p(out_ip), _p(out_id))
    if got < 0:
        raise AssertionError("column index exceeds 2**24")
    return out_ip, out_id, int(ncols.sum())


def csr_transpose(indptr, indices, n_cols, index_mask=0):
    """Stable CSR -> CSC: (t_indptr int64[n_cols+1], t_rows int32[nnz], t_perm int32[nnz])."""
    ip, is64 = _ptr_arr(indptr)
    indices = _i32(indices)
    n_rows = ip.shape[0] - 1
    nnz = int(ip[-1])
    t_ip = np.zeros(n_cols + 1, dtype=np.int64)
    t_rows = np.zeros(nnz, dtype=np.int32)
    t_perm = np.zeros(nnz, dtype=np.int32)
    lib().yo_csr_transpose(C.c_int64(n_rows), C.c_int64(n_cols), _p(ip), C.c_int(is64), _p(indices),
                           C.c_int32(index_mask), _p(t_ip), _p(t_rows), _p(t_perm))
    return t_ip, t_rows, t_perm


def partition_rows(indptr, n_parts):
    """Edge-balanced contiguous row ranges: int64 bounds[n_parts+1]."""
    ip, is64 = _ptr_arr(indptr)
    bounds = np.zeros(n_parts + 1, dtype=np.int64)
    lib().yo_partition_rows(C.c_int64(ip.shape[0] - 1), _p(ip), C.c_int(is64), C.c_int(n_parts), _p(bounds))
    return bounds


# ----------------------------------------------------------------------------------------------
# Layer-level compositions (float64 dense algebra around the aggregation kernels)
# ----------------------------------------------------------------------------------------------
def _mm(a, b):
    return (np.asarray(a, dtype=np.float64) @ np.asarray(b, dtype=np.float64)).astype(np.float32)


def gcn_forward(x, w, indptr, indices, degrees):
    """YiTu_GNN_kernel.forward: out = A_hat (X W), A_hat[i,j] = degrees[i]*degrees[j]
    (ccsrc/kernel/YiTu_GNN_kernel.cu:264-317)."""
    return spmm(indptr, indices, _mm(x, w), wmode=W_NODE, norm_dst=degrees, norm_src=degrees)


def gcn_backward(d_out, x, w, indptr, indices, degrees, transpose=True):
    """YiTu_GNN_kernel.backward (ccsrc/kernel/YiTu_GNN_kernel.cu:422-475): d' = A_hat^T d_out,
    d_input = d' W^T, d_weight = X^T d'.  transpose=False reproduces the reference's reuse of the
    forward CSR."""
    n = np.asarray(x).shape[0]
    if transpose:
        dp = spmm_transpose(indptr, indices, n, d_out, wmode=W_NODE, norm_dst=degrees, norm_src=degrees)
    else:
        dp = spmm(indptr, indices, d_out, wmode=W_NODE, norm_dst=degrees, norm_src=degrees)
    return _mm(dp, np.asarray(w).T), _mm(np.asarray(x).T, dp)


def gin_forward(x, w, indptr, indices, epsilon):
    """YiTu_GNN_kernel.forward_gin (ccsrc/kernel/YiTu_GNN_kernel.cu:563-618): agg = eps*(A X); out = agg W."""
    agg = spmm(indptr, indices, x, wmode=W_NONE, alpha=epsilon)
    return _mm(agg, w), agg


def gin_backward(d_out, agg, w, indptr, indices, epsilon, transpose=True):
    """YiTu_GNN_kernel.backward_gin (ccsrc/kernel/YiTu_GNN_kernel.cu:701-751); the X argument is the saved agg."""
    d_weight = _mm(np.asarray(agg).T, d_out)
    dp = _mm(d_out, np.asarray(w).T)
    if transpose:
        d_in = spmm_transpose(indptr, indices, dp.shape[0], dp) * np.float32(epsilon)
    else:
        d_in = spmm(indptr, indices, dp, wmode=W_NONE, alpha=epsilon)
    return d_in.astype(np.float32), d_weight


def gat_forward(indptr, indices, q, k, x):
    """fused_gsddmm + gspmm (xgnn_h/sparse.py:38-51,84-91): returns (out [n_dst,H,F], attn [E,H])."""
    q = np.asarray(q, dtype=np.float32)
    if q.ndim == 2:
        q = q[None]
    attn = sddmm_forward(indptr, indices, q, k)
    out = spmm(indptr, indices, x, n_heads=x.shape[1], wmode=W_EDGE_HEAD, values=attn, index_mask=0xFFFFFF)
    return out, attn


def gat_backward(indptr, indices, q, k, x, attn, grad_out):
    """Backward of gat_forward: (grad_q, grad_k, grad_x)."""
    q = np.asarray(q, dtype=np.float32)
    squeeze = q.ndim == 2
    if squeeze:
        q = q[None]
    grad_a, grad_x = spmm_backward(attn, indptr, indices, x, grad_out)
    grad_q, grad_k = sddmm_backward(indptr, indices, q, k, attn, grad_a)
    return (grad_q[0] if squeeze else grad_q), grad_k, grad_x


# ----------------------------------------------------------------------------------------------
# Locality reordering (numpy; integer arithmetic, so the device result must match bit for bit)
# ----------------------------------------------------------------------------------------------
def reorder_communities(n, src, dst, max_levels=32):
    """new_id int32[n], levels built, communities at the coarsest level.

    Community aggregation with Rabbit Order's merge criterion — join the neighbour u maximising
    w(v,u) - str(v)*str(u)/tot_wgt when that is positive (ccsrc/reorder/rabbit_order.hpp:455-470), on the
    symmetrised edge list without self-loops and with parallel edges summed (ccsrc/reorder/reorder.cpp:32-80) — run
    as synchronous rounds: candidates are the neighbours of higher rank (str, then id), ties go to the smaller id, and
    v joins u only if u itself stays in place in that round; the graph is contracted between rounds.  New ids order the
    nodes by (coarsest community, ..., finest community, old id).

    Parity unpinned against the reference: its asynchronous Rabbit Order needs Boost and libnuma (absent here) and
    its output depends on thread timing.  This restates the round-synchronous schedule the device code runs.
    """
    src = np.asarray(src, dtype=np.int64)
    dst = np.asarray(dst, dtype=np.int64)
    keep = src != dst
    keys = np.concatenate([(src[keep] << 32) | dst[keep], (dst[keep] << 32) | src[keep]])
    keys, w = np.unique(keys, return_counts=True)
    w = w.astype(np.int64)
    cu, cv = keys >> 32, keys & 0xFFFFFFFF
    strength = np.bincount(cu, weights=w, minlength=n).astype(np.int64)
    tot = int(strength.sum())
    cur = np.arange(n, dtype=np.int64)
    levels = []
    n_cur = n
    while len(levels) < max_levels and len(cu) > 0:
        gain = w * tot - strength[cu] * strength[cv]
        ok = (gain > 0) & ((strength[cv] > strength[cu]) | ((strength[cv] == strength[cu]) & (cv > cu)))
        parent = np.arange(n_cur, dtype=np.int64)
        idx = np.nonzero(ok)[0]
        if len(idx):
            order = np.lexsort((cv[idx], -gain[idx], cu[idx]))  # per cu: largest gain first, then smaller cv
            ii = idx[order]
            first = np.ones(len(ii), dtype=bool)
            first[1:] = cu[ii][1:] != cu[ii][:-1]
            parent[cu[ii][first]] = cv[ii][first]
        stays = parent == np.arange(n_cur)
        root = np.where(stays[parent], parent, np.arange(n_cur))
        is_root = root == np.arange(n_cur)
        n_next = int(is_root.sum())
        if n_next == n_cur:
            break
        label = (np.cumsum(is_root) - 1)[root]
        strength = np.bincount(label, weights=strength, minlength=n_next).astype(np.int64)
        a, b = label[cu], label[cv]
        m = a != b
        if m.any():
            keys, inv = np.unique((a[m] << 32) | b[m], return_inverse=True)
            w = np.bincount(inv, weights=w[m], minlength=len(keys)).astype(np.int64)
        else:
            keys, w = np.zeros(0, dtype=np.int64), np.zeros(0, dtype=np.int64)
        cu, cv = keys >> 32, keys & 0xFFFFFFFF
        cur = label[cur]
        levels.append(cur.copy())
        n_cur = n_next
    perm = np.arange(n, dtype=np.int64)
    for lv in levels:
        perm = perm[np.argsort(lv[perm], kind="stable")]
    new_id = np.empty(n, dtype=np.int64)
    new_id[perm] = np.arange(n)
    return new_id.astype(np.int32), len(levels), n_cur
