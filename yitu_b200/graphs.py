"""Seeded synthetic graphs in the CSR-by-destination form the YiTu kernels consume.

The reference builds its CSR on the host with scipy from an edge list and derives the degree
vector from the row pointers (YiTu_GNN/data/dataset.py:117-133).  The graphs here follow the same
conventions (row = destination, column = source, columns ascending within a row) but are produced
with integer-only torch arithmetic, so the same seed gives bit-identical arrays on the CPU and on
a GPU, and a 5e8-edge graph takes seconds on the device instead of minutes on the host.

Randomness is a counter-based 64-bit mixer applied to (seed, edge id, draw id): no generator state,
so any slice of the edge list can be produced independently.
"""
import math

import torch

_M34 = (1 << 34) - 1
_M37 = (1 << 37) - 1
_M33 = (1 << 33) - 1
_C1 = -4658895280553007687   # 0xBF58476D1CE4E5B9 as int64
_C2 = -7723592293110705685   # 0x94D049BB133111EB as int64
_GOLD = -7046029254386353131  # 0x9E3779B97F4A7C15 as int64


def _mix64(z):
    """splitmix64 finaliser on int64 tensors (logical shifts emulated with masks)."""
    z = (z ^ ((z >> 30) & _M34)) * _C1
    z = (z ^ ((z >> 27) & _M37)) * _C2
    return z ^ ((z >> 31) & _M33)


def _draw(seed, idx, stream):
    """64 pseudo-random bits per element of idx (int64 tensor) for draw number `stream`."""
    base = (int(seed) * 0x632BE59BD9B4E019 + int(stream) * 0x9E3779B97F4A7C15 + 0x1234567) & ((1 << 64) - 1)
    if base >= 1 << 63:
        base -= 1 << 64
    return _mix64(_mix64(idx * _GOLD + base))


def rmat_edges(seed, n_src, n_dst, n_edges, probs=(0.57, 0.19, 0.19, 0.05), device="cpu", chunk=1 << 25):
    """R-MAT edge list (src, dst) as int64 tensors.

    Each of the max(ceil(log2 n_src), ceil(log2 n_dst)) recursion levels picks a quadrant with
    probabilities (a, b, c, d) quantised to 16 bits: a = (src bit 0, dst bit 0), b = (0, 1), c = (1, 0),
    d = (1, 1).  When the two sides have different depths the extra levels of the deeper side use
    that side's marginal.  Ids are then rescaled from the power-of-two range to [0, n) by
    floor(id * n / 2^depth), which keeps the skew and wastes no sample.
    """
    a, b, c, d = probs
    ls = max(1, math.ceil(math.log2(max(n_src, 2))))
    ld = max(1, math.ceil(math.log2(max(n_dst, 2))))
    t_a = int(round(a * 65536))
    t_ab = int(round((a + b) * 65536))
    t_abc = int(round((a + b + c) * 65536))
    t_src1 = int(round((c + d) * 65536))   # P(src bit = 1)
    t_dst1 = int(round((b + d) * 65536))   # P(dst bit = 1)
    levels = max(ls, ld)
    srcs, dsts = [], []
    for e0 in range(0, n_edges, chunk):
        idx = torch.arange(e0, min(e0 + chunk, n_edges), dtype=torch.int64, device=device)
        src = torch.zeros_like(idx)
        dst = torch.zeros_like(idx)
        for lvl in range(levels):
            if lvl % 4 == 0:
                bits = _draw(seed, idx, lvl // 4)
            u = (bits >> (16 * (lvl % 4))) & 0xFFFF
            both = lvl < ls and lvl < ld
            if both:
                sbit = (u >= t_ab).to(torch.int64)
                dbit = (((u >= t_a) & (u < t_ab)) | (u >= t_abc)).to(torch.int64)
                src = (src << 1) | sbit
                dst = (dst << 1) | dbit
            elif lvl < ls:
                src = (src << 1) | (u < t_src1).to(torch.int64)
            else:
                dst = (dst << 1) | (u < t_dst1).to(torch.int64)
        if n_src != 1 << ls:
            src = (src * n_src) >> ls
        if n_dst != 1 << ld:
            dst = (dst * n_dst) >> ld
        srcs.append(src)
        dsts.append(dst)
    return torch.cat(srcs), torch.cat(dsts)


def uniform_edges(seed, n_src, n_dst, n_edges, device="cpu", chunk=1 << 26):
    """Erdos-Renyi style edge list: independent uniform src and dst."""
    srcs, dsts = [], []
    for e0 in range(0, n_edges, chunk):
        idx = torch.arange(e0, min(e0 + chunk, n_edges), dtype=torch.int64, device=device)
        bits = _draw(seed, idx, 0)
        srcs.append(((bits & 0xFFFFFFFF) * n_src) >> 32)
        dsts.append((((bits >> 32) & 0xFFFFFFFF) * n_dst) >> 32)
    return torch.cat(srcs), torch.cat(dsts)


def planted_community_edges(seed, n, community, n_edges, p_intra=0.9, device="cpu", shuffle=True, chunk=1 << 26):
    """Edges mostly inside blocks of `community` consecutive nodes (probability p_intra, otherwise a uniform
    destination), with node ids then passed through a pseudo-random bijection of [0, n) when shuffle is set — a graph
    that has locality to find but whose numbering hides it, as crawled real-world graphs do.  n must be a power of
    two (the bijection is an odd-multiplier / xor-shift permutation of log2(n)-bit words)."""
    assert n & (n - 1) == 0 and community <= n
    bits_n = n.bit_length() - 1
    t_intra = int(round(p_intra * 65536))
    srcs, dsts = [], []
    for e0 in range(0, n_edges, chunk):
        idx = torch.arange(e0, min(e0 + chunk, n_edges), dtype=torch.int64, device=device)
        a, b = _draw(seed, idx, 0), _draw(seed, idx, 1)
        src = ((a & 0xFFFFFFFF) * n) >> 32
        inside = ((b >> 48) & 0xFFFF) < t_intra
        local = (((a >> 32) & 0xFFFFFFFF) * community) >> 32
        anywhere = ((b & 0xFFFFFFFF) * n) >> 32
        dst = torch.where(inside, torch.div(src, community, rounding_mode="floor") * community + local, anywhere)
        srcs.append(src)
        dsts.append(dst)
    src, dst = torch.cat(srcs), torch.cat(dsts)
    if shuffle:
        def scramble(v):
            v = (v * 0x9E3779B1 + 0x7F4A7C15) & (n - 1)          # odd multiplier: a bijection modulo 2^k
            v = v ^ (v >> max(1, bits_n // 2))                     # xor-shift: a bijection
            return (v * 0x85EBCA6B + 0x165667B1) & (n - 1)
        src, dst = scramble(src), scramble(dst)
    return src, dst


def csr_by_destination(src, dst, n_src, n_dst, self_loops=False, index_dtype=torch.int32,
                       ptr_dtype=torch.int32):
    """Deduplicate (src, dst) pairs, optionally add (i, i) for every i, and return
    (indptr[n_dst+1], indices[nnz]) with rows = destinations and ascending sources within a row.
    Same result as scipy's coo->csr on the deduplicated list (YiTu_GNN/data/dataset.py:117-129)."""
    key = dst * n_src + src
    if self_loops:
        assert n_src == n_dst
        loop = torch.arange(n_dst, dtype=torch.int64, device=key.device)
        key = torch.cat([key, loop * n_src + loop])
    del src, dst
    key = torch.unique(key)  # sorted ascending
    rows = torch.div(key, n_src, rounding_mode="floor")
    cols = (key - rows * n_src).to(index_dtype)
    del key
    counts = torch.bincount(rows, minlength=n_dst)
    del rows
    indptr = torch.zeros(n_dst + 1, dtype=torch.int64, device=cols.device)
    torch.cumsum(counts, 0, out=indptr[1:])
    return indptr.to(ptr_dtype), cols


def in_degrees(indptr):
    return (indptr[1:] - indptr[:-1]).to(torch.float32)


def randn_features(seed, n, d, device="cpu", chunk_rows=1 << 20, row_begin=0):
    """N(0,1) float32 features, reproducible per (seed, row) on any device: Box-Muller over the mixer.
    Returns rows [row_begin, row_begin + n) of the conceptual matrix, so a rank can make its shard alone."""
    out = torch.empty((n, d), dtype=torch.float32, device=device)
    flat = out.view(-1)
    total = n * d
    step = chunk_rows * d
    base = row_begin * d
    for s in range(0, total, step):
        idx = torch.arange(base + s, base + min(s + step, total), dtype=torch.int64, device=device)
        bits = _draw(seed, idx, 977)
        u1 = ((bits & 0xFFFFFF).to(torch.float32) + 1.0) * (1.0 / 16777216.0)          # (0,1]
        u2 = (((bits >> 24) & 0xFFFFFF).to(torch.float32)) * (1.0 / 16777216.0)        # [0,1)
        flat[s:s + idx.numel()] = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(6.283185307179586 * u2)
    return out


def randn_rows(seed, row_ids, d):
    """Rows `row_ids` (an int64 tensor, any order, repeats allowed) of the matrix randn_features(seed, ., d) makes,
    on the device of row_ids: lets a checker produce the features of arbitrary source nodes without the matrix."""
    idx = (row_ids.to(torch.int64)[:, None] * d + torch.arange(d, dtype=torch.int64, device=row_ids.device)).reshape(-1)
    bits = _draw(seed, idx, 977)
    u1 = ((bits & 0xFFFFFF).to(torch.float32) + 1.0) * (1.0 / 16777216.0)
    u2 = (((bits >> 24) & 0xFFFFFF).to(torch.float32)) * (1.0 / 16777216.0)
    return (torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(6.283185307179586 * u2)).view(-1, d)


def uniform_values(seed, shape, lo, hi, device="cpu"):
    n = 1
    for s in shape:
        n *= s
    idx = torch.arange(n, dtype=torch.int64, device=device)
    bits = _draw(seed, idx, 1543)
    u = ((bits & 0xFFFFFF).to(torch.float32)) * (1.0 / 16777216.0)
    return (lo + (hi - lo) * u).reshape(shape)


def glorot_uniform(seed, fan_in, fan_out, device="cpu"):
    lim = math.sqrt(6.0 / (fan_in + fan_out))
    return uniform_values(seed, (fan_in, fan_out), -lim, lim, device=device)


# ----------------------------------------------------------------------------------------------
# The five benchmark workloads (scaled by `scale_log2` for tests: negative values shrink them)
# ----------------------------------------------------------------------------------------------
def gcn_small(device="cpu", n=16384, e=262144, seed=0):
    """2-layer GCN graph: R-MAT, deduplicated, plus self-loops; norm = in-degree^-1/2 of (A+I)."""
    src, dst = rmat_edges(seed, n, n, e, device=device)
    indptr, indices = csr_by_destination(src, dst, n, n, self_loops=True)
    norm = in_degrees(indptr).clamp(min=1.0).rsqrt()
    return indptr, indices, norm


def spmm_rmat(device="cpu", n=2097152, e=67108864, seed=1, ptr_dtype=torch.int32):
    """Sum-aggregation graph with per-edge symmetric-normalised float32 weights."""
    src, dst = rmat_edges(seed, n, n, e, device=device)
    indptr, indices = csr_by_destination(src, dst, n, n, ptr_dtype=ptr_dtype)
    deg_in = in_degrees(indptr).clamp(min=1.0)
    deg_out = torch.bincount(indices.long(), minlength=n).to(torch.float32).clamp(min=1.0)
    rows = torch.repeat_interleave(torch.arange(n, device=indptr.device), (indptr[1:] - indptr[:-1]).long())
    values = deg_in.rsqrt()[rows] * deg_out.rsqrt()[indices.long()]
    return indptr, indices, values


def gat_uniform(device="cpu", n=1048576, e=33554432, seed=2):
    src, dst = uniform_edges(seed, n, n, e, device=device)
    return csr_by_destination(src, dst, n, n, self_loops=True)


HETERO_TYPES = (1000000, 500000, 250000, 100000)


def hetero_relations(n_relations=8):
    """Relation r connects source type r mod 4 to destination type (r div 2) mod 4."""
    return [(r % 4, (r // 2) % 4) for r in range(n_relations)]


def hetero_rgcn(device="cpu", type_sizes=HETERO_TYPES, n_relations=8, e_per_rel=4000000, seed=3):
    """List of (src_type, dst_type, indptr, indices) bipartite R-MAT blocks."""
    rels = []
    for r, (st, dt) in enumerate(hetero_relations(n_relations)):
        src, dst = rmat_edges(seed * 1000 + r, type_sizes[st], type_sizes[dt], e_per_rel, device=device)
        indptr, indices = csr_by_destination(src, dst, type_sizes[st], type_sizes[dt])
        rels.append((st, dt, indptr, indices))
    return rels


def spmm_partitioned(device="cpu", n=16777216, e=536870912, seed=4):
    """Row-partitioned SpMM graph: int64 row pointers, int32 columns, weight = 1/in-degree(dst)."""
    src, dst = rmat_edges(seed, n, n, e, device=device)
    indptr, indices = csr_by_destination(src, dst, n, n, ptr_dtype=torch.int64)
    inv = 1.0 / in_degrees(indptr).clamp(min=1.0)
    values = torch.repeat_interleave(inv, indptr[1:] - indptr[:-1])
    return indptr, indices, values
