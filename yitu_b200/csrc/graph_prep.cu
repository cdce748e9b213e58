// One-time graph preparation: hub-row schedule, CSR->CSC transpose with edge permutation, edge-balanced
// row partition, per-segment mean weights (device), and the host-side tables the reference's callers
// expect (build_part, stitch_csr).  Integer work only; scans and sorts use CUB from the CUDA toolkit.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>
#include <cub/device/device_select.cuh>

#include <cstdarg>
#include <cstring>

#include "common.cuh"

namespace yitu {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

static inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// ------------------------------------------------------------------------------------------- hub plan
__global__ void hub_count_kernel(int64_t n_rows, const void *indptr, int is64, int chunk_edges, int64_t *counts) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r > n_rows) return;
    int64_t c = 0;
    if (r < n_rows) {
        const int64_t deg = load_ptr(indptr, is64, r + 1) - load_ptr(indptr, is64, r);
        if (deg > chunk_edges) c = (deg + chunk_edges - 1) / chunk_edges;
    }
    counts[r] = c;  // counts[n_rows] = 0 so that the exclusive scan leaves the total there
}

__global__ void hub_fill_kernel(int64_t n_rows, const void *indptr, int is64, int chunk_edges,
                                const int64_t *offsets, int *chunk_row, int64_t *chunk_begin) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r >= n_rows) return;
    const int64_t base = offsets[r], cnt = offsets[r + 1] - base;
    if (cnt == 0) return;
    const int64_t rb = load_ptr(indptr, is64, r);
    for (int64_t j = 0; j < cnt; ++j) {
        chunk_row[base + j] = static_cast<int>(r);
        chunk_begin[base + j] = rb + j * chunk_edges;
    }
}

static size_t scan_temp_bytes(int64_t n) {
    size_t bytes = 0;
    cub::DeviceScan::ExclusiveSum(nullptr, bytes, static_cast<int64_t *>(nullptr), static_cast<int64_t *>(nullptr),
                                  n);
    return bytes;
}

// ------------------------------------------------------------------------------------------- transpose
__global__ void edge_rows_kernel(int64_t n_rows, const void *indptr, int is64, int *rows_of_edge) {
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_rows) return;
    const int64_t b = load_ptr(indptr, is64, warp), e = load_ptr(indptr, is64, warp + 1);
    for (int64_t i = b + lane; i < e; i += 32) rows_of_edge[i] = static_cast<int>(warp);
}

__global__ void iota_mask_kernel(int64_t nnz, const int *indices, int mask, int *keys, int *ids) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    if (keys) keys[i] = indices[i] & mask;
    ids[i] = static_cast<int>(i);
}

__global__ void gather_rows_kernel(int64_t nnz, const int *rows_of_edge, const int *perm, int *t_rows) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < nnz) t_rows[i] = rows_of_edge[perm[i]];
}

template <typename P>
__global__ void col_ptr_kernel(int64_t n_cols, int64_t nnz, const int *sorted_keys, P *t_indptr) {
    const int64_t c = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (c > n_cols) return;
    int64_t lo = 0, hi = nnz;  // first position whose key >= c
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (sorted_keys[mid] >= c) hi = mid; else lo = mid + 1;
    }
    t_indptr[c] = static_cast<P>(lo);
}

static size_t sort_temp_bytes(int64_t nnz, int end_bit) {
    size_t bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, bytes, static_cast<const int *>(nullptr), static_cast<int *>(nullptr),
                                    static_cast<const int *>(nullptr), static_cast<int *>(nullptr), nnz, 0, end_bit);
    return bytes;
}

static int key_bits(int64_t n_cols) {
    int b = 1;
    while ((1ll << b) < n_cols && b < 31) ++b;
    return b;
}

// ------------------------------------------------------------------------------------------- partition
__global__ void partition_kernel(int64_t n_rows, const void *indptr, int is64, int n_parts, int64_t *bounds) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p > n_parts) return;
    if (p == 0) { bounds[0] = 0; return; }
    if (p == n_parts) { bounds[p] = n_rows; return; }
    const int64_t nnz = load_ptr(indptr, is64, n_rows);
    // ceil(p*nnz/P) without overflow: nnz < 2^40 and p < 2^16 in any real use
    const int64_t target = (static_cast<int64_t>(p) * nnz + n_parts - 1) / n_parts;
    int64_t lo = 0, hi = n_rows;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (load_ptr(indptr, is64, mid) >= target) hi = mid; else lo = mid + 1;
    }
    bounds[p] = lo;
}

// ------------------------------------------------------------------------------------------- segment mean
// One warp per row.  For every segment id present in the row: count its edges, then write 1/count to them.
__global__ void segment_mean_kernel(int64_t n_rows, const void *indptr, int is64, const int *indices, int mask,
                                    float *values) {
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= n_rows) return;
    const int64_t b = load_ptr(indptr, is64, row), e = load_ptr(indptr, is64, row + 1);
    if (mask == 0) {
        const float w = 1.0f / static_cast<float>(e - b);
        for (int64_t i = b + lane; i < e; i += 32) values[i] = w;
        return;
    }
    // segment ids are 8 bits: walk them in 8 groups of 32 with a presence mask per group
    for (int grp = 0; grp < 8; ++grp) {
        unsigned present = 0;
        for (int64_t i = b + lane; i < e; i += 32) {
            const unsigned s = static_cast<unsigned>(indices[i]) >> 24;
            if ((s >> 5) == static_cast<unsigned>(grp)) present |= 1u << (s & 31);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) present |= __shfl_xor_sync(0xffffffffu, present, o);
        while (present) {
            const unsigned s = grp * 32 + (__ffs(present) - 1);
            present &= present - 1;
            int cnt = 0;
            for (int64_t i = b + lane; i < e; i += 32) cnt += ((static_cast<unsigned>(indices[i]) >> 24) == s);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
            const float w = 1.0f / static_cast<float>(cnt);
            for (int64_t i = b + lane; i < e; i += 32)
                if ((static_cast<unsigned>(indices[i]) >> 24) == s) values[i] = w;
        }
    }
}


// ------------------------------------------------------------------------------------------- COO -> CSR
__global__ void pack_edges_kernel(int64_t n_edges, const int *src, const int *dst, int64_t n_loops, uint64_t *keys) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n_edges) {
        keys[i] = (static_cast<uint64_t>(static_cast<uint32_t>(dst[i])) << 32) | static_cast<uint32_t>(src[i]);
    } else if (i < n_edges + n_loops) {
        const uint64_t v = static_cast<uint64_t>(i - n_edges);
        keys[i] = (v << 32) | v;
    }
}

template <typename P>
__global__ void csr_from_keys_kernel(int64_t n_dst, const int64_t *nnz_dev, const uint64_t *keys, P *indptr, int *indices) {
    const int64_t nnz = *nnz_dev;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < nnz) indices[i] = static_cast<int>(keys[i] & 0xffffffffu);
    if (i <= n_dst) {  // first position whose destination >= i
        int64_t lo = 0, hi = nnz;
        while (lo < hi) {
            const int64_t mid = (lo + hi) >> 1;
            if (static_cast<int64_t>(keys[mid] >> 32) >= i) hi = mid; else lo = mid + 1;
        }
        indptr[i] = static_cast<P>(lo);
    }
}

__global__ void degree_norm_kernel(int64_t n, const void *indptr, int is64, int mode, float *out) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r >= n) return;
    const float d = fmaxf(static_cast<float>(load_ptr(indptr, is64, r + 1) - load_ptr(indptr, is64, r)), 1.0f);
    out[r] = mode == 0 ? sqrtf(d) : (mode == 1 ? 1.0f / sqrtf(d) : 1.0f / d);
}

// ------------------------------------------------------------------------------------------- stitch (device)
struct StitchParams {
    const int *indptr[16];
    const int *indices[16];
    int shift[16];
    int n_blocks;
    int64_t n_rows;
};

__global__ void stitch_ptr_kernel(const __grid_constant__ StitchParams p, int *out_indptr) {
    const int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (r > p.n_rows) return;
    int total = 0;
    for (int b = 0; b < p.n_blocks; ++b) total += p.indptr[b][r];
    out_indptr[r] = total;
}

__global__ void stitch_fill_kernel(const __grid_constant__ StitchParams p, const int *out_indptr, int *out_indices,
                                   int *overflow) {
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= p.n_rows) return;
    int w = out_indptr[row];
    for (int b = 0; b < p.n_blocks; ++b) {
        const int beg = p.indptr[b][row], end = p.indptr[b][row + 1];
        for (int i = beg + lane; i < end; i += 32) {
            const int col = p.shift[b] + p.indices[b][i];
            if (col >= (1 << 24)) *overflow = 1;  // would carry into the segment tag
            out_indices[w + (i - beg)] = (b << 24) + col;
        }
        w += end - beg;
    }
}

}  // namespace yitu

using namespace yitu;

extern "C" const char *yitu_status_string(int status) {
    switch (status) {
        case YITU_OK: return "ok";
        case YITU_ERR_INVALID_ARG: return "invalid argument";
        case YITU_ERR_CUDA: return "CUDA error";
        case YITU_ERR_WORKSPACE: return "workspace too small";
        case YITU_ERR_UNSUPPORTED: return "unsupported shape";
        case YITU_ERR_LIMIT: return "size limit exceeded";
        default: return "unknown status";
    }
}
extern "C" const char *yitu_last_error(void) { return g_error; }
extern "C" int yitu_version(void) { return 100; }

extern "C" int64_t yitu_hub_plan_workspace_bytes(int64_t n_rows) {
    return align_up((n_rows + 1) * 8, 256) + align_up(static_cast<int64_t>(scan_temp_bytes(n_rows + 1)), 256);
}

extern "C" int yitu_hub_plan_count(const yitu_csr_t *g, int32_t chunk_edges, void *workspace,
                                   int64_t workspace_bytes, int64_t *n_chunks_host, yitu_stream_t stream) {
    if (int rc = validate_csr(g)) return rc;
    YITU_REQUIRE(chunk_edges >= 32, YITU_ERR_INVALID_ARG, "chunk_edges must be >= 32");
    YITU_REQUIRE(workspace && workspace_bytes >= yitu_hub_plan_workspace_bytes(g->n_rows), YITU_ERR_WORKSPACE,
                 "hub plan workspace needs %lld bytes", (long long)yitu_hub_plan_workspace_bytes(g->n_rows));
    YITU_REQUIRE(n_chunks_host, YITU_ERR_INVALID_ARG, "n_chunks_host is NULL");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int64_t *counts = static_cast<int64_t *>(workspace);
    void *temp = static_cast<char *>(workspace) + align_up((g->n_rows + 1) * 8, 256);
    size_t temp_bytes = scan_temp_bytes(g->n_rows + 1);
    const int64_t n = g->n_rows + 1;
    hub_count_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(g->n_rows, g->indptr, g->indptr_is64,
                                                                            chunk_edges, counts);
    YITU_LAUNCH_CHECK();
    YITU_CUDA(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, counts, counts, n, st));
    YITU_CUDA(cudaMemcpyAsync(n_chunks_host, counts + g->n_rows, 8, cudaMemcpyDeviceToHost, st));
    YITU_CUDA(cudaStreamSynchronize(st));
    return YITU_OK;
}

extern "C" int yitu_hub_plan_fill(const yitu_csr_t *g, int32_t chunk_edges, const void *workspace, int64_t n_chunks,
                                  int32_t *chunk_row, int64_t *chunk_begin, yitu_stream_t stream) {
    if (int rc = validate_csr(g)) return rc;
    if (n_chunks == 0 || g->n_rows == 0) return YITU_OK;
    YITU_REQUIRE(workspace && chunk_row && chunk_begin, YITU_ERR_INVALID_ARG, "NULL table or workspace");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    hub_fill_kernel<<<static_cast<unsigned>((g->n_rows + 255) / 256), 256, 0, st>>>(
        g->n_rows, g->indptr, g->indptr_is64, chunk_edges, static_cast<const int64_t *>(workspace), chunk_row,
        chunk_begin);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

extern "C" int64_t yitu_csr_transpose_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t nnz) {
    (void)n_rows;
    const int64_t arr = align_up(nnz * 4 + 4, 256);
    return 4 * arr + align_up(static_cast<int64_t>(sort_temp_bytes(nnz, key_bits(n_cols))), 256) + 256;
}

extern "C" int yitu_csr_transpose(const yitu_csr_t *g, void *t_indptr, int32_t *t_rows, int32_t *t_perm,
                                  void *workspace, int64_t workspace_bytes, yitu_stream_t stream) {
    if (int rc = validate_csr(g)) return rc;
    YITU_REQUIRE(g->nnz < (1ll << 31), YITU_ERR_LIMIT, "transpose needs nnz < 2^31 (edge ids are int32)");
    YITU_REQUIRE(t_indptr, YITU_ERR_INVALID_ARG, "t_indptr is NULL");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int64_t nnz = g->nnz;
    if (nnz == 0) {
        YITU_CUDA(cudaMemsetAsync(t_indptr, 0, (g->n_cols + 1) * (g->indptr_is64 ? 8 : 4), st));
        return YITU_OK;
    }
    YITU_REQUIRE(t_rows && t_perm, YITU_ERR_INVALID_ARG, "t_rows / t_perm is NULL");
    YITU_REQUIRE(workspace && workspace_bytes >= yitu_csr_transpose_workspace_bytes(g->n_rows, g->n_cols, nnz),
                 YITU_ERR_WORKSPACE, "transpose workspace needs %lld bytes",
                 (long long)yitu_csr_transpose_workspace_bytes(g->n_rows, g->n_cols, nnz));
    const int64_t arr = align_up(nnz * 4 + 4, 256);
    char *ws = static_cast<char *>(workspace);
    int *rows_of_edge = reinterpret_cast<int *>(ws);
    int *keys_in = reinterpret_cast<int *>(ws + arr);
    int *keys_out = reinterpret_cast<int *>(ws + 2 * arr);
    int *ids = reinterpret_cast<int *>(ws + 3 * arr);
    void *temp = ws + 4 * arr;
    const int bits = key_bits(g->n_cols);
    size_t temp_bytes = sort_temp_bytes(nnz, bits);

    const unsigned eb = static_cast<unsigned>((nnz + 255) / 256);
    edge_rows_kernel<<<static_cast<unsigned>((g->n_rows * 32 + 255) / 256), 256, 0, st>>>(g->n_rows, g->indptr,
                                                                                          g->indptr_is64, rows_of_edge);
    YITU_LAUNCH_CHECK();
    const int *keys = g->indices;
    if (g->index_mask) {
        iota_mask_kernel<<<eb, 256, 0, st>>>(nnz, g->indices, g->index_mask, keys_in, ids);
        keys = keys_in;
    } else {
        iota_mask_kernel<<<eb, 256, 0, st>>>(nnz, g->indices, 0, nullptr, ids);
    }
    YITU_LAUNCH_CHECK();
    YITU_CUDA(cub::DeviceRadixSort::SortPairs(temp, temp_bytes, keys, keys_out, ids, t_perm, nnz, 0, bits, st));
    gather_rows_kernel<<<eb, 256, 0, st>>>(nnz, rows_of_edge, t_perm, t_rows);
    YITU_LAUNCH_CHECK();
    const unsigned cb = static_cast<unsigned>((g->n_cols + 1 + 255) / 256);
    if (g->indptr_is64)
        col_ptr_kernel<int64_t><<<cb, 256, 0, st>>>(g->n_cols, nnz, keys_out, static_cast<int64_t *>(t_indptr));
    else
        col_ptr_kernel<int><<<cb, 256, 0, st>>>(g->n_cols, nnz, keys_out, static_cast<int *>(t_indptr));
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

extern "C" int yitu_partition_rows(const yitu_csr_t *g, int32_t n_parts, int64_t *bounds, yitu_stream_t stream) {
    if (int rc = validate_csr(g)) return rc;
    YITU_REQUIRE(n_parts >= 1 && n_parts <= 65536 && bounds, YITU_ERR_INVALID_ARG, "bad n_parts or bounds");
    partition_kernel<<<(n_parts + 1 + 63) / 64, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        g->n_rows, g->indptr, g->indptr_is64, n_parts, bounds);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

static inline int64_t host_ptr(const void *p, int is64, int64_t i) {
    return is64 ? static_cast<const int64_t *>(p)[i] : static_cast<int64_t>(static_cast<const int32_t *>(p)[i]);
}

extern "C" int yitu_partition_rows_host(int64_t n_rows, const void *indptr_host, int32_t indptr_is64, int32_t n_parts,
                                        int64_t *bounds_host) {
    YITU_REQUIRE(indptr_host && bounds_host && n_parts >= 1 && n_rows >= 0, YITU_ERR_INVALID_ARG, "bad argument");
    const int64_t nnz = host_ptr(indptr_host, indptr_is64, n_rows);
    bounds_host[0] = 0;
    for (int p = 1; p < n_parts; ++p) {
        const int64_t target = (static_cast<int64_t>(p) * nnz + n_parts - 1) / n_parts;
        int64_t lo = 0, hi = n_rows;
        while (lo < hi) {
            const int64_t mid = (lo + hi) >> 1;
            if (host_ptr(indptr_host, indptr_is64, mid) >= target) hi = mid; else lo = mid + 1;
        }
        bounds_host[p] = lo;
    }
    bounds_host[n_parts] = n_rows;
    return YITU_OK;
}

extern "C" int yitu_segment_mean_weights_f32(const yitu_csr_t *g, float *values, yitu_stream_t stream) {
    if (int rc = validate_csr(g)) return rc;
    if (g->n_rows == 0 || g->nnz == 0) return YITU_OK;
    YITU_REQUIRE(values, YITU_ERR_INVALID_ARG, "values is NULL");
    segment_mean_kernel<<<static_cast<unsigned>((g->n_rows * 32 + 255) / 256), 256, 0,
                          reinterpret_cast<cudaStream_t>(stream)>>>(g->n_rows, g->indptr, g->indptr_is64, g->indices,
                                                                    g->index_mask, values);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}


// ------------------------------------------------------------------------------------------- COO -> CSR (device)
static int coo_key_bits(int64_t n_dst) { return 32 + key_bits(n_dst); }

static size_t coo_temp_bytes(int64_t m, int bits) {
    size_t a = 0, b = 0;
    cub::DeviceRadixSort::SortKeys(nullptr, a, static_cast<const uint64_t *>(nullptr), static_cast<uint64_t *>(nullptr), m, 0,
                                   bits);
    cub::DeviceSelect::Unique(nullptr, b, static_cast<const uint64_t *>(nullptr), static_cast<uint64_t *>(nullptr),
                              static_cast<int64_t *>(nullptr), m);
    return a > b ? a : b;
}

extern "C" int64_t yitu_coo_to_csr_workspace_bytes(int64_t n_edges, int64_t n_dst, int32_t add_self_loops) {
    const int64_t m = n_edges + (add_self_loops ? n_dst : 0);
    return 2 * align_up(m * 8 + 8, 256) + 256 + align_up(static_cast<int64_t>(coo_temp_bytes(m, coo_key_bits(n_dst))), 256);
}

extern "C" int yitu_coo_to_csr(int64_t n_src, int64_t n_dst, int64_t n_edges, const int32_t *src, const int32_t *dst,
                               int32_t add_self_loops, void *indptr_out, int32_t indptr_is64, int32_t *indices_out,
                               int64_t *nnz_host, void *workspace, int64_t workspace_bytes, yitu_stream_t stream) {
    YITU_REQUIRE(n_src >= 0 && n_dst >= 0 && n_edges >= 0 && n_src < (1ll << 31) && n_dst < (1ll << 31),
                 YITU_ERR_INVALID_ARG, "bad sizes");
    YITU_REQUIRE(!add_self_loops || n_src == n_dst, YITU_ERR_INVALID_ARG, "self-loops need a square graph");
    YITU_REQUIRE(indptr_out && nnz_host, YITU_ERR_INVALID_ARG, "NULL output");
    const int64_t m = n_edges + (add_self_loops ? n_dst : 0);
    YITU_REQUIRE(indptr_is64 || m < (1ll << 31), YITU_ERR_LIMIT, "%lld edges need int64 row pointers", (long long)m);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (m == 0) {
        YITU_CUDA(cudaMemsetAsync(indptr_out, 0, (n_dst + 1) * (indptr_is64 ? 8 : 4), st));
        *nnz_host = 0;
        return YITU_OK;
    }
    YITU_REQUIRE((n_edges == 0 || (src && dst)) && indices_out, YITU_ERR_INVALID_ARG, "NULL edge list or indices_out");
    YITU_REQUIRE(workspace && workspace_bytes >= yitu_coo_to_csr_workspace_bytes(n_edges, n_dst, add_self_loops),
                 YITU_ERR_WORKSPACE, "coo_to_csr workspace needs %lld bytes",
                 (long long)yitu_coo_to_csr_workspace_bytes(n_edges, n_dst, add_self_loops));
    const int64_t arr = align_up(m * 8 + 8, 256);
    char *ws = static_cast<char *>(workspace);
    uint64_t *keys_a = reinterpret_cast<uint64_t *>(ws);
    uint64_t *keys_b = reinterpret_cast<uint64_t *>(ws + arr);
    int64_t *nnz_dev = reinterpret_cast<int64_t *>(ws + 2 * arr);
    void *temp = ws + 2 * arr + 256;
    const int bits = coo_key_bits(n_dst);
    size_t temp_bytes = coo_temp_bytes(m, bits);
    pack_edges_kernel<<<static_cast<unsigned>((m + 255) / 256), 256, 0, st>>>(n_edges, src, dst,
                                                                             add_self_loops ? n_dst : 0, keys_a);
    YITU_LAUNCH_CHECK();
    YITU_CUDA(cub::DeviceRadixSort::SortKeys(temp, temp_bytes, keys_a, keys_b, m, 0, bits, st));
    YITU_CUDA(cub::DeviceSelect::Unique(temp, temp_bytes, keys_b, keys_a, nnz_dev, m, st));
    const int64_t work = (m > n_dst + 1 ? m : n_dst + 1);
    const unsigned blocks = static_cast<unsigned>((work + 255) / 256);
    if (indptr_is64)
        csr_from_keys_kernel<int64_t><<<blocks, 256, 0, st>>>(n_dst, nnz_dev, keys_a, static_cast<int64_t *>(indptr_out),
                                                              indices_out);
    else
        csr_from_keys_kernel<int><<<blocks, 256, 0, st>>>(n_dst, nnz_dev, keys_a, static_cast<int *>(indptr_out),
                                                          indices_out);
    YITU_LAUNCH_CHECK();
    YITU_CUDA(cudaMemcpyAsync(nnz_host, nnz_dev, 8, cudaMemcpyDeviceToHost, st));
    YITU_CUDA(cudaStreamSynchronize(st));
    return YITU_OK;
}

extern "C" int yitu_degree_norm_f32(int64_t n_rows, const void *indptr, int32_t indptr_is64, int32_t mode, float *out,
                                    yitu_stream_t stream) {
    YITU_REQUIRE(n_rows >= 0 && indptr && mode >= 0 && mode <= 2, YITU_ERR_INVALID_ARG, "bad argument");
    if (n_rows == 0) return YITU_OK;
    YITU_REQUIRE(out, YITU_ERR_INVALID_ARG, "out is NULL");
    degree_norm_kernel<<<static_cast<unsigned>((n_rows + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        n_rows, indptr, indptr_is64, mode, out);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

extern "C" int yitu_stitch_csr(int32_t n_blocks, int64_t n_rows, const int32_t *const *indptrs_host,
                               const int32_t *const *indices_host, const int64_t *n_cols_host, int32_t *out_indptr,
                               int32_t *out_indices, int32_t *overflow_flag, yitu_stream_t stream) {
    YITU_REQUIRE(n_blocks >= 0 && n_blocks <= 16, YITU_ERR_LIMIT, "stitch_csr takes at most 16 blocks, got %d", n_blocks);
    YITU_REQUIRE(out_indptr && overflow_flag && n_rows >= 0, YITU_ERR_INVALID_ARG, "bad argument");
    StitchParams p{};
    p.n_blocks = n_blocks;
    p.n_rows = n_rows;
    int64_t shift = 0;
    for (int b = 0; b < n_blocks; ++b) {
        YITU_REQUIRE(indptrs_host[b] != nullptr, YITU_ERR_INVALID_ARG, "block %d has no row pointers", b);
        p.indptr[b] = indptrs_host[b];
        p.indices[b] = indices_host[b];
        p.shift[b] = static_cast<int>(shift);
        shift += n_cols_host[b];
        // The reference asserts col <= 2**24 (xgnn_h/block.py:52), which lets column 2^24 through: added to the tag it
        // becomes column 0 of the next relation.  Deliberately stricter here: a stitched column must be below 2^24.
        YITU_REQUIRE(shift <= (1 << 24), YITU_ERR_LIMIT, "stitched blocks have %lld columns, more than 2^24", (long long)shift);
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    YITU_CUDA(cudaMemsetAsync(overflow_flag, 0, 4, st));
    stitch_ptr_kernel<<<static_cast<unsigned>((n_rows + 1 + 255) / 256), 256, 0, st>>>(p, out_indptr);
    YITU_LAUNCH_CHECK();
    if (n_rows > 0 && out_indices) {
        stitch_fill_kernel<<<static_cast<unsigned>((n_rows * 32 + 255) / 256), 256, 0, st>>>(p, out_indptr, out_indices,
                                                                                           overflow_flag);
        YITU_LAUNCH_CHECK();
    }
    return YITU_OK;
}

// ------------------------------------------------------------------------------------------- host tables
extern "C" int64_t yitu_build_part_count_host(int32_t part_size, const int32_t *indptr_host, int64_t n_nodes) {
    if (part_size < 1 || !indptr_host) return -1;
    int64_t groups = 0;
    for (int64_t i = 0; i < n_nodes; ++i) {
        const int64_t deg = static_cast<int64_t>(indptr_host[i + 1]) - indptr_host[i];
        groups += (deg + part_size - 1) / part_size;
    }
    return groups;
}

extern "C" int yitu_build_part_host(int32_t part_size, const int32_t *indptr_host, int64_t n_nodes,
                                    float *part_ptr_host, float *part2node_host) {
    YITU_REQUIRE(part_size >= 1 && indptr_host && part_ptr_host, YITU_ERR_INVALID_ARG, "bad build_part argument");
    int64_t g = 0;
    for (int64_t i = 0; i < n_nodes; ++i) {
        const int32_t first = indptr_host[i];
        const int64_t deg = static_cast<int64_t>(indptr_host[i + 1]) - first;
        const int64_t groups = (deg + part_size - 1) / part_size;
        for (int64_t k = 0; k < groups; ++k, ++g) {
            part_ptr_host[g] = static_cast<float>(first + static_cast<int32_t>(k) * part_size);
            part2node_host[g] = static_cast<float>(static_cast<int32_t>(i));
        }
    }
    // the reference writes the closing pointer while emitting the last node's final group, so it is the
    // edge count when that node has edges and stays 0 when it has none
    const bool last_has_edges = n_nodes > 0 && indptr_host[n_nodes] > indptr_host[n_nodes - 1];
    part_ptr_host[g] = last_has_edges ? static_cast<float>(indptr_host[n_nodes]) : 0.0f;
    return YITU_OK;
}

extern "C" int yitu_stitch_csr_host(int32_t n_blocks, int64_t n_rows, const int32_t *const *indptrs_host,
                                    const int32_t *const *indices_host, const int64_t *n_cols_host,
                                    int32_t *out_indptr_host, int32_t *out_indices_host) {
    YITU_REQUIRE(n_blocks >= 0 && n_blocks <= 16, YITU_ERR_LIMIT, "stitch_csr takes at most 16 blocks, got %d",
                 n_blocks);
    YITU_REQUIRE(out_indptr_host, YITU_ERR_INVALID_ARG, "out_indptr is NULL");
    // column offset of every block, then a row-major sweep that appends each block's slice of the row
    int64_t shift[16];
    int64_t total_cols = 0;
    for (int b = 0; b < n_blocks; ++b) {
        shift[b] = total_cols;
        total_cols += n_cols_host[b];
    }
    int64_t w = 0;
    for (int64_t r = 0; r < n_rows; ++r) {
        out_indptr_host[r] = static_cast<int32_t>(w);
        for (int b = 0; b < n_blocks; ++b) {
            const int32_t *ip = indptrs_host[b];
            const int32_t *id = indices_host[b];
            const int32_t tag = b << 24;
            for (int32_t i = ip[r]; i < ip[r + 1]; ++i) {
                const int64_t col = shift[b] + id[i];
                // stricter than the reference's `col <= 2**24` (xgnn_h/block.py:52): column 2^24 would carry into the tag
                YITU_REQUIRE(col < (1 << 24), YITU_ERR_LIMIT, "stitched column %lld exceeds 2^24 - 1", (long long)col);
                out_indices_host[w++] = tag + static_cast<int32_t>(col);
            }
        }
    }
    out_indptr_host[n_rows] = static_cast<int32_t>(w);
    return YITU_OK;
}
