/*
 * yitu_b200 — C ABI of the B200 (sm_100a) message-passing kernels that replace the CUDA
 * extensions of CGCL-codes/YiTu on its GNN aggregation path:
 *
 *   YiTu_GNN.YiTu_GNN_kernel  (ccsrc/kernel/YiTu_GNN.cpp:247-258)   SAG / forward / backward /
 *                                                                   forward_gin / backward_gin / build_part
 *   graph_ext                 (YiTu_GNN/YiTu_H/src/entry.cpp:184-193) spmm_* / sddmm_* / hfused_*
 *
 * Conventions
 *   - torch-free: raw device pointers, explicit sizes, a CUDA stream per call.  Every pointer is
 *     DEVICE memory unless the parameter name ends in `_host`.
 *   - inputs are borrowed and never written; outputs and workspaces are allocated by the caller.
 *   - a graph is a CSR by destination row: indptr[n_rows+1] (int32 or int64), indices[nnz] (int32,
 *     column = source node).  With index_mask != 0 an index is "stitched": column = idx & index_mask and
 *     segment (relation) id = (uint32)idx >> 24, the packed format of xgnn_h/block.py:36-67.
 *   - every function returns YITU_OK (0) or an error code; yitu_last_error() gives the detail text of the
 *     calling thread's last failure.  Nothing here calls exit() (the reference does on a launch error,
 *     ccsrc/kernel/YiTu_GNN_kernel.cu:309-314).
 *   - no state is kept between calls and no call is tied to a thread, so forward may run on the user
 *     thread and backward on an autograd thread.
 */
#ifndef YITU_B200_H
#define YITU_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *yitu_stream_t; /* same type as cudaStream_t */

enum {
    YITU_OK = 0,
    YITU_ERR_INVALID_ARG = 1,
    YITU_ERR_CUDA = 2,
    YITU_ERR_WORKSPACE = 3,   /* workspace / scratch too small */
    YITU_ERR_UNSUPPORTED = 4, /* shape outside what this kernel was built for */
    YITU_ERR_LIMIT = 5        /* size beyond a documented fixed limit */
};

const char *yitu_status_string(int status);
const char *yitu_last_error(void);
int yitu_version(void);

/* ---------------------------------------------------------------------------------------------- graph */
typedef struct yitu_csr_t {
    int64_t n_rows;      /* destination nodes */
    int64_t n_cols;      /* source nodes */
    int64_t nnz;         /* stored edges */
    const void *indptr;  /* [n_rows+1] */
    int32_t indptr_is64; /* 0: int32 row pointers, 1: int64 */
    int32_t index_mask;  /* 0: plain column ids; 0xffffff: stitched (segment id in the top 8 bits) */
    const int32_t *indices; /* [nnz] */
} yitu_csr_t;

/* Schedule that splits rows longer than chunk_edges into chunks of chunk_edges edges, so that a hub row
 * of a power-law graph is aggregated by many warps and reduced in a fixed order (no float atomics).
 * It plays the role of the reference's neighbour-group table (ccsrc/kernel/YiTu_GNN.cpp:203-245), which
 * splits EVERY row into groups of partSize and merges them with atomics. */
typedef struct yitu_hub_plan_t {
    int32_t chunk_edges;
    int32_t reserved;
    int64_t n_chunks;
    const int32_t *chunk_row;   /* [n_chunks] row of each chunk, ascending */
    const int64_t *chunk_begin; /* [n_chunks] first edge of each chunk */
} yitu_hub_plan_t;

int64_t yitu_hub_plan_workspace_bytes(int64_t n_rows);
/* Step 1: counts the chunks (*n_chunks_host, synchronises the stream) and leaves per-row offsets in
 * `workspace`.  Step 2 (yitu_hub_plan_fill) writes the two tables from the same workspace. */
int yitu_hub_plan_count(const yitu_csr_t *g, int32_t chunk_edges, void *workspace, int64_t workspace_bytes,
                        int64_t *n_chunks_host, yitu_stream_t stream);
int yitu_hub_plan_fill(const yitu_csr_t *g, int32_t chunk_edges, const void *workspace, int64_t n_chunks,
                       int32_t *chunk_row, int64_t *chunk_begin, yitu_stream_t stream);

/* CSR -> CSC (rows = sources) plus the edge permutation, stable: within a column the edges keep their CSR
 * order (ascending destination).  t_indptr has the width of g->indptr.  Replaces nothing in the reference:
 * its backward kernels scatter with atomicAdd instead (YiTu_GNN/YiTu_H/src/spmm_cuda.cu:32-38,
 * sddmm_cuda.cu:58-63) and the ccsrc backward reuses the forward CSR (YiTu_GNN_kernel.cu:448-466). */
int64_t yitu_csr_transpose_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t nnz);
int yitu_csr_transpose(const yitu_csr_t *g, void *t_indptr, int32_t *t_rows, int32_t *t_perm, void *workspace,
                       int64_t workspace_bytes, yitu_stream_t stream);

/* Edge-balanced contiguous row partition: bounds[p] = min{ r : indptr[r] >= ceil(p*nnz/P) }, bounds[0]=0,
 * bounds[P]=n_rows (int64, device).  Reworks the node-count-balanced range partition of
 * YiTu_GNN/mmap/partition.py:12-22,165-197 (whose rebased-indptr convention the callers keep). */
int yitu_partition_rows(const yitu_csr_t *g, int32_t n_parts, int64_t *bounds, yitu_stream_t stream);
int yitu_partition_rows_host(int64_t n_rows, const void *indptr_host, int32_t indptr_is64, int32_t n_parts,
                             int64_t *bounds_host);

/* Edge list -> CSR by destination on the device: sorts (dst, src), drops duplicate pairs, optionally adds (i, i) for
 * every node, columns ascending within a row.  Same structure as the scipy coo->csr the reference runs on the host
 * (YiTu_GNN/data/dataset.py:117-129).  indices_out needs n_edges (+ n_dst with self-loops) entries; the number of stored
 * edges comes back in *nnz_host (the call synchronises the stream). */
int64_t yitu_coo_to_csr_workspace_bytes(int64_t n_edges, int64_t n_dst, int32_t add_self_loops);
int yitu_coo_to_csr(int64_t n_src, int64_t n_dst, int64_t n_edges, const int32_t *src, const int32_t *dst,
                    int32_t add_self_loops, void *indptr_out, int32_t indptr_is64, int32_t *indices_out, int64_t *nnz_host,
                    void *workspace, int64_t workspace_bytes, yitu_stream_t stream);

/* Per-node degree vector from the row pointers, d = max(in-degree, 1): mode 0 = sqrt(d), the `degrees` tensor the
 * reference's dataset passes to its GCN kernel (YiTu_GNN/data/dataset.py:131-133); mode 1 = 1/sqrt(d) (symmetric
 * normalisation); mode 2 = 1/d (right norm, xgnn_h/mp.py:165-167). */
int yitu_degree_norm_f32(int64_t n_rows, const void *indptr, int32_t indptr_is64, int32_t mode, float *out,
                         yitu_stream_t stream);

/* stitch_csr on the device: block tables are DEVICE int32 arrays, the two pointer arrays and n_cols are HOST arrays.
 * out_indices needs sum(nnz) entries; *overflow_flag (device int32) becomes 1 if a stitched column exceeds 2^24. */
int yitu_stitch_csr(int32_t n_blocks, int64_t n_rows, const int32_t *const *indptrs_host,
                    const int32_t *const *indices_host, const int64_t *n_cols_host, int32_t *out_indptr,
                    int32_t *out_indices, int32_t *overflow_flag, yitu_stream_t stream);

/* Neighbour-group table, on the host, bit-identical to build_part (ccsrc/kernel/YiTu_GNN.cpp:203-245):
 * float32 storage, and the terminal pointer is written only while the last node's groups are emitted. */
int64_t yitu_build_part_count_host(int32_t part_size, const int32_t *indptr_host, int64_t n_nodes);
int yitu_build_part_host(int32_t part_size, const int32_t *indptr_host, int64_t n_nodes, float *part_ptr_host,
                         float *part2node_host);

/* stitch_csr (YiTu_GNN/YiTu_H/xgnn_h/block.py:36-67) on the host: concatenates row r of up to 16 blocks,
 * new index = (block id << 24) + column + columns of the blocks before.  out_indices needs sum(nnz) entries.
 * Fails with YITU_ERR_LIMIT where the reference asserts (more than 16 blocks, column > 2^24). */
int yitu_stitch_csr_host(int32_t n_blocks, int64_t n_rows, const int32_t *const *indptrs_host,
                         const int32_t *const *indices_host, const int64_t *n_cols_host, int32_t *out_indptr_host,
                         int32_t *out_indices_host);

/* ------------------------------------------------------------------------------------ locality reordering */
/* new_id[v] = position of node v in an order that keeps communities contiguous: hierarchical aggregation with
 * Rabbit Order's merge criterion (largest positive modularity gain, ccsrc/reorder/rabbit_order.hpp:455-530) run
 * as synchronous data-parallel rounds on the device — the role of rabbit.reorder (ccsrc/reorder/reorder.cpp:235-290,
 * called from YiTu_GNN/data/dataset.py:149-170), which runs on the host cores there.  Deterministic: integer
 * arithmetic throughout.  The edge list is treated as undirected; self-loops and repeated edges are accepted.
 * Fewer than 2^30 edges.  Synchronises the stream (one small read-back per level).
 * n_levels_host / n_top_host (optional): levels built, communities at the coarsest level. */
int64_t yitu_reorder_workspace_bytes(int64_t n_nodes, int64_t n_edges, int32_t max_levels);
int yitu_reorder_communities(int64_t n_nodes, int64_t n_edges, const int32_t *src, const int32_t *dst,
                             int32_t max_levels, int32_t *new_id, int32_t *n_levels_host, int64_t *n_top_host,
                             void *workspace, int64_t workspace_bytes, yitu_stream_t stream);

/* out_src[i] = new_id[src[i]], out_dst[i] = new_id[dst[i]] — the edge list rabbit.reorder returns. */
int yitu_relabel_edges(int64_t n_edges, const int32_t *src, const int32_t *dst, const int32_t *new_id,
                       int32_t *out_src, int32_t *out_dst, yitu_stream_t stream);

/* *sum_device = sum_i |src[i] - dst[i]|: numerator of the reference's avg_edgeSpan (YiTu_GNN/data/dataset.py:109),
 * which its decider compares with sqrt(n)/100 to decide whether to reorder (YiTu_GNN/utils/input_info.py:131-140). */
int yitu_edge_span_sum(int64_t n_edges, const int32_t *src, const int32_t *dst, uint64_t *sum_device,
                       yitu_stream_t stream);

/* ---------------------------------------------------------------------------------------------- SpMM */
enum {
    YITU_W_NONE = 0,      /* w = 1                       SAG, GIN, gspmm(edge=None)  */
    YITU_W_NODE = 1,      /* w = norm_dst[row]*norm_src[col]   ccsrc GCN             */
    YITU_W_EDGE = 2,      /* w = values[e]                                            */
    YITU_W_EDGE_HEAD = 3  /* w = values[e*H + h]         graph_ext.spmm_forward       */
};

/* Epilogue activations fused into the aggregation kernels (the layers apply them right after the aggregation:
 * ReLU in the GCN models, ELU in the GAT models — YiTu_GNN/YiTu_H/test/common/model.py:46-49,126-129). */
enum {
    YITU_ACT_NONE = 0,
    YITU_ACT_RELU = 1,
    YITU_ACT_ELU = 2 /* v > 0 ? v : exp(v) - 1 */
};

/* out[r,h,k] = act( alpha * row_scale[r] * sum_{e in row r} w(e,h) * x[col_e,h,k]  (+ out[r,h,k] if accumulate)
 *                   + bias[h*F+k] )
 *
 * Replaces the aggregation kernels of
 *   ccsrc/kernel/YiTu_GNN_kernel.cu:179-257 (SAG), :319-415 / :477-556 (GCN fwd / bwd),
 *   :620-694 / :753-823 (GIN fwd / bwd), and YiTu_GNN/YiTu_H/src/spmm_cuda.cu:4-21 (multi-head SpMM);
 * run over the transposed graph (yitu_csr_transpose, edge_perm = t_perm) it is also the grad_x half of
 * spmm_cuda.cu:24-42.  The dense X*W of the GCN/GIN layers stays outside (a library GEMM). */
typedef struct yitu_spmm_args_t {
    yitu_csr_t graph;
    int64_t n_heads;          /* H (1 for plain SpMM) */
    int64_t n_feats;          /* F; a feature row holds H*F floats */
    int32_t weight_mode;      /* YITU_W_* */
    int32_t accumulate;       /* 0: overwrite out, 1: add to it */
    const float *edge_values; /* W_EDGE: [nnz]; W_EDGE_HEAD: [nnz,H] */
    const int32_t *edge_perm; /* optional: edge e reads edge_values[edge_perm[e]] */
    const float *norm_dst;    /* W_NODE: [n_rows] */
    const float *norm_src;    /* W_NODE: [n_cols] */
    const float *row_scale;   /* optional [n_rows] */
    float alpha;              /* scalar epilogue (GIN epsilon; 1/#relations) */
    int32_t activation;       /* YITU_ACT_*, applied last */
    const float *x;           /* [n_cols, x_stride] source features */
    int64_t x_stride;         /* floats between feature rows (>= H*F; >= F with x_shared_heads) */
    float *out;               /* [n_rows, out_stride] */
    int64_t out_stride;
    const yitu_hub_plan_t *plan; /* optional hub-row schedule (host struct, device tables) */
    float *scratch;              /* plan != NULL: >= plan->n_chunks * H*F floats */
    int64_t scratch_bytes;
    const float *bias;           /* optional [H*F], added before the activation */
    int32_t x_shared_heads;      /* W_EDGE_HEAD only: a source row holds F floats that every head reads (the gradient
                                    of a mean over heads) instead of H*F */
    int32_t reserved;
} yitu_spmm_args_t;

int yitu_spmm_csr_f32(const yitu_spmm_args_t *args, yitu_stream_t stream);

/* The same SpMM for callers that may not allocate device memory (fixed-budget memory pools, plugins that
 * are handed their buffers, latency-critical loops): the hub partial sums go to a 16 MiB array built into the
 * library instead of args->scratch, which is ignored.  No counterpart in the reference.
 *   - returns YITU_ERR_LIMIT when plan->n_chunks * H*F * 4 bytes exceed yitu_static_scratch_bytes();
 *   - every GPU that loads the library holds the array until the process exits;
 *   - all calls on a device share it: calls that overlap on the GPU race, so keep them on one stream;
 *   - the first call on each device looks up the array's address (no allocation); make it before any
 *     stream capture starts.
 * Inputs, outputs and the hub plan are still the caller's. */
int64_t yitu_static_scratch_bytes(void);
int yitu_spmm_csr_f32_static(const yitu_spmm_args_t *args, yitu_stream_t stream);

/* Backward of the fused epilogue y = act(row_scale[r] * agg + bias):
 *   grad_agg[r,d] = grad_y[r,d] * act'(y[r,d]) * row_scale[r]     (row_scale NULL = 1)
 * with act' taken from the OUTPUT y (ReLU: y > 0; ELU: y > 0 ? 1 : y + 1).  One pass; grad_agg may alias grad_y.
 * The reference runs these as separate torch element-wise kernels around the aggregation. */
int yitu_epilogue_grad_f32(int64_t n_rows, int64_t n_feats, int32_t activation, const float *y, const float *grad_y,
                           const float *row_scale, float *grad_agg, yitu_stream_t stream);

/* values[e] = 1 / (number of edges of e's row that carry e's segment id): with YITU_W_EDGE over a stitched
 * graph this turns the SpMM into "mean per relation, then sum over relations" in ONE pass and one output
 * write per destination row — the mathematics of HeteroGraphConv over GCNLayer with norm = 1/in_degree
 * (YiTu_GNN/YiTu_H/test/common/model.py:15-30,142-171; xgnn_h/mp.py:223-227).  Rows without edges of a
 * segment simply contribute nothing (the reference would form 0 * inf there). */
int yitu_segment_mean_weights_f32(const yitu_csr_t *g, float *values, yitu_stream_t stream);

/* grad_a[e,h] = sum_k g[row_e,h,k] * x[col_e,h,k] — the edge-value half of
 * YiTu_GNN/YiTu_H/src/spmm_cuda.cu:24-42, without atomics (one owner per (e,h)). */
int yitu_edge_dot_f32(const yitu_csr_t *g, int64_t n_heads, int64_t n_feats, const float *grad_out, const float *x,
                      float *grad_a, const yitu_hub_plan_t *plan, yitu_stream_t stream);

/* Both gradients of out[r,h,:] = sum_e values[e,h] * x[col_e,h,:] in ONE pass over the transposed graph
 * (YiTu_GNN/YiTu_H/src/spmm_cuda.cu:24-42, two atomicAdds per edge, head and feature there): the rows of grad_out
 * gathered for grad_x[c] = sum_e values_e * grad_out[row_e] also give grad_values[e] = <grad_out[row_e], x[c]> against
 * the source's own features.  H <= 32, H*F <= 512, F/4 a power of two <= 32; other shapes return YITU_ERR_UNSUPPORTED
 * (use yitu_edge_dot_f32 + yitu_spmm_csr_f32 over the transposed graph).  graph: sizes and index width of the forward
 * graph; edge_values / grad_values are in its edge order. */
typedef struct yitu_spmm_bwd_args_t {
    yitu_csr_t graph;
    int64_t n_heads, n_feats;
    const float *edge_values;  /* [nnz,H] */
    const float *x;            /* [n_cols,H,F] */
    const float *grad_out;     /* [n_rows,H,F] */
    const void *t_indptr;      /* transposed graph from yitu_csr_transpose */
    const int32_t *t_rows;
    const int32_t *t_perm;
    float *grad_values;        /* [nnz,H] */
    float *grad_x;             /* [n_cols,H,F] */
    const yitu_hub_plan_t *t_plan; /* optional hub schedule of the transposed graph */
    float *scratch;            /* t_plan: >= t_plan->n_chunks * H*F floats */
    int64_t scratch_bytes;
} yitu_spmm_bwd_args_t;
int yitu_spmm_bwd_f32(const yitu_spmm_bwd_args_t *args, yitu_stream_t stream);

/* ---------------------------------------------------------------------------------------------- GAT */
/* The `plan` argument of the functions below is the optional hub-row schedule of the graph they walk (the transposed
 * graph's for yitu_edge_gather_sum_f32): with it, rows longer than plan->chunk_edges are processed by a whole CTA, or
 * chunk by chunk, instead of by one warp.  NULL keeps one warp per row. */
/* attn[e,h] = softmax over {edges of the same row and segment} of LeakyReLU_slope(query[seg,row,h] + key[col,h]).
 * Replaces sddmm_forward (YiTu_GNN/YiTu_H/src/sddmm_cuda.cu:5-33,69-89).  Unlike the reference the row maximum
 * is subtracted before exponentiation (same value, no overflow).  n_segments = query.size(0) (<= 16). */
int yitu_edge_softmax_fwd_f32(const yitu_csr_t *g, int32_t n_segments, int64_t n_heads, float slope,
                              const float *query, const float *key, float *attn, const yitu_hub_plan_t *plan,
                              yitu_stream_t stream);

/* Replaces sddmm_backward (sddmm_cuda.cu:36-67,91-118): writes grad_query[seg,row,h] (every entry, zeros
 * included) and edge_grad[e,h] = d loss / d (query+key) per edge; grad_key is then the per-source sum of
 * edge_grad, taken with yitu_edge_gather_sum_f32 over the transposed graph (no atomics). */
int yitu_edge_softmax_bwd_f32(const yitu_csr_t *g, int32_t n_segments, int64_t n_heads, float slope,
                              const float *query, const float *key, const float *attn, const float *grad_attn,
                              float *grad_query, float *edge_grad, const yitu_hub_plan_t *plan, yitu_stream_t stream);

/* out[c,h] = sum_{j in column c of the transposed graph} edge_vals[t_perm[j], h] */
int yitu_edge_gather_sum_f32(int64_t n_cols, const void *t_indptr, int32_t indptr_is64, const int32_t *t_perm,
                             int64_t n_heads, const float *edge_vals, float *out, const yitu_hub_plan_t *t_plan,
                             yitu_stream_t stream);

/* Fused GAT layer core: scores, LeakyReLU, edge softmax (online maximum/sum) and the weighted aggregation in
 * one pass over each row's edges — the composition sddmm_forward + spmm_forward of the reference
 * (xgnn_h/sparse.py:38-51,84-91; layer YiTu_GNN/YiTu_H/test/common/model.py:75-106) without the [nnz,H]
 * attention tensor.  Plain (unstitched) graphs, H <= 32, F a multiple of 4, H*F <= 512; other shapes return
 * YITU_ERR_UNSUPPORTED and the caller composes the unfused ops.  The backward call needs no pass over a row to
 * normalise: with the row statistics of the forward pass and D[r,h] = <grad_out[r,h,:], out[r,h,:]>
 * (= sum_e attn_e * d attn_e) every edge's attention and score gradient follow on their own, so ONE pass over the
 * transposed graph — which gathers the rows of grad_out for grad_x anyway — also yields d attn (against the source's
 * own features), the score gradients (scattered to edge_grad, then summed per row into grad_query) and grad_key. */
typedef struct yitu_gat_args_t {
    yitu_csr_t graph;
    int64_t n_heads, n_feats;
    float slope;
    int32_t head_mean;  /* 1: out[r,k] = act(mean_h out[r,h,k]) — the layer's torch.mean(v, dim=1), model.py:106 */
    const float *query; /* [n_rows,H] */
    const float *key;   /* [n_cols,H] */
    const float *x;     /* [n_cols,H,F] */
    float *out;         /* [n_rows,H,F], or [n_rows,F] with head_mean */
    float *row_max;     /* [n_rows,H] softmax statistics */
    float *row_sum;     /* [n_rows,H] */
    int32_t activation; /* YITU_ACT_* on out (forward only; the backward call expects the gradient with respect
                           to the pre-activation values) */
    int32_t reserved;
    float *out_heads;   /* head_mean only: the per-head result [n_rows,H,F] before the mean; optional in the forward
                           call, required by the backward call (which reads it instead of `out`) */
    const yitu_hub_plan_t *plan; /* optional hub-row schedule of `graph`: rows longer than plan->chunk_edges are cut
                                    into chunks that separate warps process (power-law graphs) */
    float *scratch;     /* plan != NULL: forward needs yitu_gat_fwd_scratch_bytes(plan->n_chunks, H, F) */
    int64_t scratch_bytes;
} yitu_gat_args_t;
int64_t yitu_gat_fwd_scratch_bytes(int64_t n_chunks, int64_t n_heads, int64_t n_feats);
int yitu_gat_fwd_f32(const yitu_gat_args_t *args, yitu_stream_t stream);

typedef struct yitu_gat_bwd_args_t {
    yitu_gat_args_t fwd;       /* same tensors as the forward call (out, row_max, row_sum now inputs) */
    const float *grad_out;     /* [n_rows,H,F], or [n_rows,F] with fwd.head_mean */
    const void *t_indptr;      /* transposed graph from yitu_csr_transpose */
    const int32_t *t_rows;
    const int32_t *t_perm;
    float *grad_query;         /* [n_rows,H] */
    float *grad_key;           /* [n_cols,H] */
    float *grad_x;             /* [n_cols,H,F] */
    float *edge_attn;          /* scratch [nnz,H]; needed only when F/4 is not a power of two <= 32 (may be NULL otherwise) */
    float *edge_grad;          /* scratch [nnz,H]: the score gradient per edge, in CSR order */
    const yitu_hub_plan_t *t_plan; /* optional hub-row schedule of the transposed graph (fwd.plan is that of the graph) */
    float *scratch;            /* yitu_gat_bwd_scratch_bytes(n_rows, fwd.plan chunks or 0, t_plan chunks or 0, H, F) */
    int64_t scratch_bytes;
} yitu_gat_bwd_args_t;
int64_t yitu_gat_bwd_scratch_bytes(int64_t n_rows, int64_t n_chunks, int64_t t_n_chunks, int64_t n_heads,
                                   int64_t n_feats);
int yitu_gat_bwd_f32(const yitu_gat_bwd_args_t *args, yitu_stream_t stream);

/* ---------------------------------------------------------------------------------------------- multi-GPU */
/* dst[i, :] = row ids[i] of a feature matrix that is sharded by contiguous row ranges over several GPUs:
 * shard p holds rows [shard_bounds_host[p], shard_bounds_host[p+1]) at shard_ptrs_host[p] (a pointer this GPU
 * can dereference: its own memory, or a peer's mapped through CUDA IPC / peer access).  Rows are fetched with
 * plain 128-bit loads over NVLink — no collective, no multicast — so each needed source row crosses the link
 * once and lands in local memory, where the SpMM gathers it.  Both `_host` arrays are HOST memory
 * (n_shards <= 16, n_shards+1 bounds).  row_floats must be a multiple of 4 and all pointers 16-byte aligned.
 * Reworks the feature exchange of YiTu_GNN/distributed/communication.py:14-51,230-264. */
int yitu_halo_gather_f32(int32_t n_shards, const float *const *shard_ptrs_host, const int64_t *shard_bounds_host,
                         const int32_t *ids, int64_t n_ids, int64_t row_floats, float *dst, yitu_stream_t stream);

/* The same exchange driven by the OWNER of the rows: row ids[i] of this GPU's shard `x` (local row numbers) is
 * written to row (i - list_begin_host[d]) of destination d's buffer dst_ptrs_host[d], for the destination d with
 * list_begin_host[d] <= i < list_begin_host[d+1].  Destination pointers are peer mappings (yitu_shared_open) that
 * already point at the first row reserved for this owner.  Plain 128-bit stores over NVLink: posted writes, no
 * collective, no multicast.  Completion of the kernel on `stream` means the rows have left; the destinations must
 * still learn of it (a stream-ordered collective or event chain that follows this call).  Both `_host` arrays are
 * HOST memory (n_dests <= 16, n_dests+1 offsets).  Takes the role of the per-destination sends of
 * YiTu_GNN/distributed/communication.py:230-264. */
int yitu_halo_push_f32(int32_t n_dests, float *const *dst_ptrs_host, const int64_t *list_begin_host,
                       const int32_t *ids, const float *x, int64_t row_floats, uint64_t *work_counter,
                       int32_t n_sms, yitu_stream_t stream);
/* work_counter: 8 bytes of device memory owned by the caller, used by one push at a time (the call zeroes it on
 * `stream`; the kernel hands out its items from it).  n_sms: SMs the push occupies, one 1024-thread CTA each, which
 * nothing else shares (0 = default, 24: enough to fill one NVLink direction); a push that is paced by its
 * destination's ingress rather than by this GPU's egress needs fewer. */

/* Delivery flags between GPUs, for the owner-side push.  yitu_flags_signal stores `value` (use the step number:
 * flags only ever grow) into n 64-bit flags, typically one in each reader's memory (peer mappings), in stream order
 * - after a push on the same stream it tells those readers that the rows are in place.  yitu_flags_wait makes
 * `stream` wait until flags[i] >= value for every i in `mask` (the first 32 flags of a local array), for at most
 * timeout_ns (required, <= 10 s); on expiry it stores 1 + (index of a missing flag) into *error_flag (device int32,
 * set once, never cleared by the library) and lets the stream continue.  No counterpart in the reference, whose
 * ranks meet in collectives (YiTu_GNN/distributed/communication.py:230-264). */
int yitu_flags_signal(int32_t n, uint64_t *const *targets_host, uint64_t value, yitu_stream_t stream);
int yitu_flags_wait(const uint64_t *flags, uint32_t mask, uint64_t value, int64_t timeout_ns, int32_t *error_flag,
                    yitu_stream_t stream);

/* Feature shards that peers can read.  yitu_shared_alloc allocates `bytes` of device memory on the current
 * device (one cudaMalloc, so the pointer is an allocation base) and fills `handle_out` with its 64-byte CUDA IPC
 * handle; another PROCESS passes those bytes to yitu_shared_open, with its own GPU current, and receives a pointer
 * valid in kernels on that GPU (peer access over NVLink is enabled lazily by the driver).  yitu_shared_close
 * unmaps an opened pointer, yitu_shared_free releases an allocated one.  Host-side calls; `handle` is host memory.
 * Reworks the role of the pickled tensor exchange in YiTu_GNN/distributed/communication.py:83-162. */
int yitu_shared_alloc(int64_t bytes, void **ptr_out, unsigned char *handle_out);
int yitu_shared_open(const unsigned char *handle, void **ptr_out);
int yitu_shared_close(void *ptr);
int yitu_shared_free(void *ptr);

#ifdef __cplusplus
}
#endif
#endif /* YITU_B200_H */
