// Locality reordering of node ids on the device: hierarchical community aggregation in the manner of Rabbit Order
// (ccsrc/reorder/rabbit_order.hpp:455-530: a vertex joins the neighbour with the largest modularity gain
// w(v,u) - str(v)*str(u)/tot_wgt), recast as synchronous rounds so that it runs as data-parallel kernels and gives
// the same permutation on every run:
//   * the edge list is symmetrised, self-loops dropped, parallel edges summed (reorder.cpp:32-80);
//   * per round every community v looks at its neighbours u of higher rank (str, then id) and picks the largest
//     positive gain; v joins u only if u itself stays in place this round (star merges: no chains, no cycles);
//   * the graph is contracted (relabel, 64-bit radix sort, reduce by key) and the next round runs on the coarser graph;
//   * new ids are the lexicographic order of (coarsest community, ..., finest community, old id): every community
//     of every level becomes a contiguous id range — the property Rabbit's dendrogram DFS gives
//     (rabbit_order.hpp:700-750).
// All arithmetic is integer (weights are edge counts; gains are compared as w*tot - str(v)*str(u) in 64 bits), so
// the result is reproducible and can be checked bit for bit against a CPU restatement.
//
// The reference runs the asynchronous, lock-based Rabbit Order on the host cores (Boost + libnuma); its result
// depends on thread timing.  This file shares its objective and merge criterion, not its schedule.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_reduce.cuh>
#include <cub/device/device_scan.cuh>

#include "common.cuh"

namespace yitu {

static inline int64_t up256(int64_t v) { return (v + 255) / 256 * 256; }

struct Carver {  // hands out 256-byte aligned pieces of the caller's workspace
    char *base;
    int64_t used, cap;
    template <typename T>
    T *take(int64_t n) {
        T *p = reinterpret_cast<T *>(base + used);
        used += up256(n * static_cast<int64_t>(sizeof(T)));
        return p;
    }
};

static int key_bits(int64_t n) {  // bits of a (community << 32 | community) key, sentinel community n included
    int b = 1;
    while ((1ll << b) <= n) ++b;
    return 32 + b;
}

// keys of both directions of every edge; self-loops become the sentinel (n << 32), which sorts last
__global__ void sym_keys_kernel(int64_t n_edges, int64_t n, const int *src, const int *dst, uint64_t *keys, int *w,
                                int *bad) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_edges) return;
    const int64_t s = src[i], d = dst[i];
    if (s < 0 || d < 0 || s >= n || d >= n) {
        *bad = 1;
        keys[2 * i] = keys[2 * i + 1] = static_cast<uint64_t>(n) << 32;
        w[2 * i] = w[2 * i + 1] = 0;
        return;
    }
    const uint64_t sentinel = static_cast<uint64_t>(n) << 32;
    keys[2 * i] = s != d ? (static_cast<uint64_t>(s) << 32 | static_cast<uint64_t>(d)) : sentinel;
    keys[2 * i + 1] = s != d ? (static_cast<uint64_t>(d) << 32 | static_cast<uint64_t>(s)) : sentinel;
    w[2 * i] = w[2 * i + 1] = s != d ? 1 : 0;
}

// first edge of every community in the sorted key array (binary search: no atomics)
__global__ void offsets_kernel(int64_t n_cur, int64_t n_edges, const uint64_t *keys, int *off) {
    const int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (v > n_cur) return;
    const uint64_t target = static_cast<uint64_t>(v) << 32;
    int64_t lo = 0, hi = n_edges;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (keys[mid] < target) lo = mid + 1;
        else hi = mid;
    }
    off[v] = static_cast<int>(lo);
}

__global__ void strength_kernel(int64_t n_cur, const int *off, const int *w, int64_t *str) {
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (warp >= n_cur) return;
    const int lane = threadIdx.x & 31;
    int64_t s = 0;
    for (int e = off[warp] + lane; e < off[warp + 1]; e += 32) s += w[e];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) str[warp] = s;
}

// parent[v] = the higher-ranked neighbour with the largest positive gain (ties: smaller id), else v.  Warp per community.
__global__ void best_neighbour_kernel(int64_t n_cur, const int *off, const uint64_t *keys, const int *w,
                                      const int64_t *str, const int64_t *tot_ptr, int *parent) {
    const int64_t v = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (v >= n_cur) return;
    const int lane = threadIdx.x & 31;
    const int64_t tot = *tot_ptr, sv = str[v];
    int64_t best_gain = 0;
    int best_u = static_cast<int>(v);
    for (int e = off[v] + lane; e < off[v + 1]; e += 32) {
        const int u = static_cast<int>(keys[e] & 0xffffffffu);
        const int64_t su = str[u];
        if (!(su > sv || (su == sv && u > v))) continue;
        const int64_t gain = static_cast<int64_t>(w[e]) * tot - sv * su;
        if (gain > best_gain || (gain == best_gain && gain > 0 && u < best_u)) {
            best_gain = gain;
            best_u = u;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const int64_t g2 = __shfl_xor_sync(0xffffffffu, best_gain, o);
        const int u2 = __shfl_xor_sync(0xffffffffu, best_u, o);
        if (g2 > best_gain || (g2 == best_gain && g2 > 0 && u2 < best_u)) {
            best_gain = g2;
            best_u = u2;
        }
    }
    if (lane == 0) parent[v] = best_gain > 0 ? best_u : static_cast<int>(v);
}

// star merges: v joins parent[v] only if that community stays in place; is_root marks the survivors
__global__ void star_kernel(int64_t n_cur, const int *parent, int *root, int *is_root) {
    const int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (v >= n_cur) return;
    const int u = parent[v];
    const int r = (parent[u] == u) ? u : static_cast<int>(v);
    root[v] = r;
    is_root[v] = r == v ? 1 : 0;
}

__global__ void label_kernel(int64_t n_cur, const int *root, const int *new_id, const int64_t *str, int *label,
                             unsigned long long *str_next) {
    const int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (v >= n_cur) return;
    const int c = new_id[root[v]];
    label[v] = c;
    atomicAdd(str_next + c, static_cast<unsigned long long>(str[v]));  // integer sum: order does not matter
}

__global__ void contract_kernel(int64_t n_edges, int64_t n_next, const int *label, const uint64_t *keys, uint64_t *out,
                                int *w) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_edges) return;
    const uint64_t k = keys[i];
    const int a = label[k >> 32], b = label[k & 0xffffffffu];
    if (a != b) {
        out[i] = static_cast<uint64_t>(a) << 32 | static_cast<uint64_t>(b);
    } else {
        out[i] = static_cast<uint64_t>(n_next) << 32;
        w[i] = 0;
    }
}

__global__ void descend_kernel(int64_t n, const int *label, int *cur, int *level_out) {
    const int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (v >= n) return;
    const int c = label[cur[v]];
    cur[v] = c;
    level_out[v] = c;
}

__global__ void iota_kernel(int64_t n, int *a) {
    const int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (v < n) a[v] = static_cast<int>(v);
}

__global__ void gather_kernel(int64_t n, const int *table, const int *idx, int *out) {
    const int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (v < n) out[v] = table[idx[v]];
}

__global__ void invert_kernel(int64_t n, const int *perm, int *new_id) {
    const int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (v < n) new_id[perm[v]] = static_cast<int>(v);
}

__global__ void relabel_edges_kernel(int64_t n_edges, const int *src, const int *dst, const int *new_id, int *out_src,
                                     int *out_dst) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n_edges) return;
    out_src[i] = new_id[src[i]];
    out_dst[i] = new_id[dst[i]];
}

__global__ void edge_span_kernel(int64_t n_edges, const int *src, const int *dst, unsigned long long *sum) {
    unsigned long long s = 0;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_edges; i += stride) {
        const int64_t d = static_cast<int64_t>(src[i]) - dst[i];
        s += static_cast<unsigned long long>(d < 0 ? -d : d);
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0 && s) atomicAdd(sum, s);
}

struct ReorderTemp {
    size_t sort_pairs, sort_ids, reduce_by_key, scan, reduce;
    size_t max() const {
        size_t m = sort_pairs;
        for (size_t v : {sort_ids, reduce_by_key, scan, reduce}) m = v > m ? v : m;
        return m;
    }
};

static ReorderTemp reorder_temp_bytes(int64_t n, int64_t e2) {
    ReorderTemp t{};
    const int n_e = static_cast<int>(e2), n_n = static_cast<int>(n);
    cub::DeviceRadixSort::SortPairs(nullptr, t.sort_pairs, static_cast<const uint64_t *>(nullptr),
                                    static_cast<uint64_t *>(nullptr), static_cast<const int *>(nullptr),
                                    static_cast<int *>(nullptr), n_e, 0, 64);
    cub::DeviceRadixSort::SortPairs(nullptr, t.sort_ids, static_cast<const int *>(nullptr), static_cast<int *>(nullptr),
                                    static_cast<const int *>(nullptr), static_cast<int *>(nullptr), n_n, 0, 32);
    cub::DeviceReduce::ReduceByKey(nullptr, t.reduce_by_key, static_cast<const uint64_t *>(nullptr),
                                   static_cast<uint64_t *>(nullptr), static_cast<const int *>(nullptr),
                                   static_cast<int *>(nullptr), static_cast<int *>(nullptr), cub::Sum(), n_e);
    cub::DeviceScan::ExclusiveSum(nullptr, t.scan, static_cast<const int *>(nullptr), static_cast<int *>(nullptr), n_n);
    cub::DeviceReduce::Sum(nullptr, t.reduce, static_cast<const int64_t *>(nullptr), static_cast<int64_t *>(nullptr), n_n);
    return t;
}

}  // namespace yitu

using namespace yitu;

static int64_t reorder_layout(int64_t n, int64_t n_edges, int32_t max_levels, Carver *c, ReorderTemp *tt) {
    const int64_t e2 = 2 * n_edges;
    const ReorderTemp t = reorder_temp_bytes(n, e2 > 0 ? e2 : 1);
    if (tt) *tt = t;
    Carver k{nullptr, 0, 0};
    k.take<uint64_t>(e2); k.take<uint64_t>(e2);          // keys, double buffered
    k.take<int>(e2); k.take<int>(e2);                    // weights, double buffered
    k.take<int64_t>(n + 1); k.take<int64_t>(n + 1);      // strengths, double buffered
    for (int i = 0; i < 8; ++i) k.take<int>(n + 1);      // offsets, parent, root, is_root, new ids, label, cur, keys of the final sorts
    k.take<int>(n); k.take<int>(n); k.take<int>(n);      // permutation (double buffered) and sorted keys
    k.take<int>(static_cast<int64_t>(max_levels) * n);   // community of every node at every level
    k.take<int64_t>(32);                                 // scalars
    k.used += up256(static_cast<int64_t>(t.max()));
    (void)c;
    return k.used;
}

extern "C" int64_t yitu_reorder_workspace_bytes(int64_t n_nodes, int64_t n_edges, int32_t max_levels) {
    if (n_nodes < 0 || n_edges < 0 || max_levels < 1 || n_edges >= (1ll << 30)) return -1;
    return reorder_layout(n_nodes, n_edges, max_levels, nullptr, nullptr);
}

extern "C" int yitu_reorder_communities(int64_t n_nodes, int64_t n_edges, const int32_t *src, const int32_t *dst,
                                        int32_t max_levels, int32_t *new_id, int32_t *n_levels_host,
                                        int64_t *n_top_host, void *workspace, int64_t workspace_bytes,
                                        yitu_stream_t stream) {
    YITU_REQUIRE(n_nodes >= 0 && n_nodes < (1ll << 31) - 1 && n_edges >= 0, YITU_ERR_INVALID_ARG, "bad sizes");
    YITU_REQUIRE(n_edges < (1ll << 30), YITU_ERR_LIMIT, "reordering takes fewer than 2^30 edges, got %lld",
                 (long long)n_edges);
    YITU_REQUIRE(max_levels >= 1 && max_levels <= 64, YITU_ERR_INVALID_ARG, "max_levels=%d (1..64)", max_levels);
    YITU_REQUIRE(n_nodes == 0 || new_id, YITU_ERR_INVALID_ARG, "new_id is NULL");
    YITU_REQUIRE(n_edges == 0 || (src && dst), YITU_ERR_INVALID_ARG, "NULL edge list");
    const int64_t need = yitu_reorder_workspace_bytes(n_nodes, n_edges, max_levels);
    YITU_REQUIRE(workspace && workspace_bytes >= need, YITU_ERR_WORKSPACE, "reorder workspace needs %lld bytes",
                 (long long)need);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (n_levels_host) *n_levels_host = 0;
    if (n_top_host) *n_top_host = n_nodes;
    if (n_nodes == 0) return YITU_OK;
    const int64_t n = n_nodes, e2 = 2 * n_edges;
    const auto blocks = [](int64_t items) { return static_cast<unsigned>((items + 255) / 256); };

    ReorderTemp tb = reorder_temp_bytes(n, e2 > 0 ? e2 : 1);
    Carver k{static_cast<char *>(workspace), 0, workspace_bytes};
    uint64_t *keys = k.take<uint64_t>(e2), *keys_alt = k.take<uint64_t>(e2);
    int *w = k.take<int>(e2), *w_alt = k.take<int>(e2);
    int64_t *str = k.take<int64_t>(n + 1), *str_alt = k.take<int64_t>(n + 1);
    int *off = k.take<int>(n + 1), *parent = k.take<int>(n + 1), *root = k.take<int>(n + 1);
    int *is_root = k.take<int>(n + 1), *new_ids = k.take<int>(n + 1), *label = k.take<int>(n + 1);
    int *cur = k.take<int>(n + 1), *sort_keys = k.take<int>(n + 1);
    int *perm = k.take<int>(n), *perm_alt = k.take<int>(n), *sort_keys_out = k.take<int>(n);
    int *levels = k.take<int>(static_cast<int64_t>(max_levels) * n);
    int64_t *scalars = k.take<int64_t>(32);  // [0] total weight, [1] runs (int), [2] bad-id flag (int), [3] last count
    void *temp = k.base + k.used;
    size_t temp_bytes = tb.max();

    int *runs_dev = reinterpret_cast<int *>(scalars + 1), *bad_dev = reinterpret_cast<int *>(scalars + 2);
    int64_t *tot_dev = scalars;
    YITU_CUDA(cudaMemsetAsync(scalars, 0, 32 * sizeof(int64_t), st));
    iota_kernel<<<blocks(n), 256, 0, st>>>(n, cur);
    YITU_LAUNCH_CHECK();

    int64_t e_cur = 0, n_cur = n;
    int n_levels = 0;
    // the reduce-by-key of a sorted key array, dropping the trailing sentinel run
    auto sort_and_merge = [&](int64_t items, int64_t sentinel_community) -> int {
        const int bits = key_bits(sentinel_community);
        YITU_CUDA(cub::DeviceRadixSort::SortPairs(temp, temp_bytes, keys, keys_alt, w, w_alt, static_cast<int>(items), 0,
                                                  bits, st));
        YITU_CUDA(cub::DeviceReduce::ReduceByKey(temp, temp_bytes, keys_alt, keys, w_alt, w, runs_dev, cub::Sum(),
                                                 static_cast<int>(items), st));
        int runs = 0;
        YITU_CUDA(cudaMemcpyAsync(&runs, runs_dev, sizeof(int), cudaMemcpyDeviceToHost, st));
        YITU_CUDA(cudaStreamSynchronize(st));
        e_cur = runs;
        if (runs > 0) {
            uint64_t last = 0;
            YITU_CUDA(cudaMemcpyAsync(&last, keys + (runs - 1), sizeof(uint64_t), cudaMemcpyDeviceToHost, st));
            YITU_CUDA(cudaStreamSynchronize(st));
            if ((last >> 32) == static_cast<uint64_t>(sentinel_community)) e_cur = runs - 1;
        }
        return YITU_OK;
    };

    if (e2 > 0) {
        sym_keys_kernel<<<blocks(n_edges), 256, 0, st>>>(n_edges, n, src, dst, keys, w, bad_dev);
        YITU_LAUNCH_CHECK();
        if (int rc = sort_and_merge(e2, n)) return rc;
        int bad = 0;
        YITU_CUDA(cudaMemcpyAsync(&bad, bad_dev, sizeof(int), cudaMemcpyDeviceToHost, st));
        YITU_CUDA(cudaStreamSynchronize(st));
        YITU_REQUIRE(bad == 0, YITU_ERR_INVALID_ARG, "edge list holds node ids outside [0, %lld)", (long long)n);
    }
    if (e_cur > 0) {
        offsets_kernel<<<blocks(n + 1), 256, 0, st>>>(n, e_cur, keys, off);
        YITU_LAUNCH_CHECK();
        strength_kernel<<<blocks(n * 32), 256, 0, st>>>(n, off, w, str);
        YITU_LAUNCH_CHECK();
        YITU_CUDA(cub::DeviceReduce::Sum(temp, temp_bytes, str, tot_dev, static_cast<int>(n), st));
    }

    while (n_levels < max_levels && e_cur > 0) {
        if (n_levels > 0) {
            offsets_kernel<<<blocks(n_cur + 1), 256, 0, st>>>(n_cur, e_cur, keys, off);
            YITU_LAUNCH_CHECK();
        }
        best_neighbour_kernel<<<blocks(n_cur * 32), 256, 0, st>>>(n_cur, off, keys, w, str, tot_dev, parent);
        YITU_LAUNCH_CHECK();
        star_kernel<<<blocks(n_cur), 256, 0, st>>>(n_cur, parent, root, is_root);
        YITU_LAUNCH_CHECK();
        YITU_CUDA(cudaMemsetAsync(is_root + n_cur, 0, sizeof(int), st));
        YITU_CUDA(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, is_root, new_ids, static_cast<int>(n_cur + 1), st));
        int n_next = 0;
        YITU_CUDA(cudaMemcpyAsync(&n_next, new_ids + n_cur, sizeof(int), cudaMemcpyDeviceToHost, st));
        YITU_CUDA(cudaStreamSynchronize(st));
        if (n_next == n_cur) break;  // no community moved: the hierarchy is complete
        YITU_CUDA(cudaMemsetAsync(str_alt, 0, (n_next + 1) * sizeof(int64_t), st));
        label_kernel<<<blocks(n_cur), 256, 0, st>>>(n_cur, root, new_ids, str, label,
                                                   reinterpret_cast<unsigned long long *>(str_alt));
        YITU_LAUNCH_CHECK();
        contract_kernel<<<blocks(e_cur), 256, 0, st>>>(e_cur, n_next, label, keys, keys, w);
        YITU_LAUNCH_CHECK();
        descend_kernel<<<blocks(n), 256, 0, st>>>(n, label, cur, levels + static_cast<int64_t>(n_levels) * n);
        YITU_LAUNCH_CHECK();
        if (int rc = sort_and_merge(e_cur, n_next)) return rc;
        int64_t *tmp = str; str = str_alt; str_alt = tmp;
        n_cur = n_next;
        ++n_levels;
    }

    // new ids: stable sorts from the finest level to the coarsest put every community of every level in one range
    iota_kernel<<<blocks(n), 256, 0, st>>>(n, perm);
    YITU_LAUNCH_CHECK();
    for (int l = 0; l < n_levels; ++l) {
        gather_kernel<<<blocks(n), 256, 0, st>>>(n, levels + static_cast<int64_t>(l) * n, perm, sort_keys);
        YITU_LAUNCH_CHECK();
        YITU_CUDA(cub::DeviceRadixSort::SortPairs(temp, temp_bytes, sort_keys, sort_keys_out, perm, perm_alt,
                                                  static_cast<int>(n), 0, 32, st));
        int *tmp = perm; perm = perm_alt; perm_alt = tmp;
    }
    invert_kernel<<<blocks(n), 256, 0, st>>>(n, perm, new_id);
    YITU_LAUNCH_CHECK();
    YITU_CUDA(cudaStreamSynchronize(st));
    if (n_levels_host) *n_levels_host = n_levels;
    if (n_top_host) *n_top_host = n_cur;
    return YITU_OK;
}

extern "C" int yitu_relabel_edges(int64_t n_edges, const int32_t *src, const int32_t *dst, const int32_t *new_id,
                                  int32_t *out_src, int32_t *out_dst, yitu_stream_t stream) {
    YITU_REQUIRE(n_edges >= 0, YITU_ERR_INVALID_ARG, "bad size");
    if (n_edges == 0) return YITU_OK;
    YITU_REQUIRE(src && dst && new_id && out_src && out_dst, YITU_ERR_INVALID_ARG, "NULL tensor");
    relabel_edges_kernel<<<static_cast<unsigned>((n_edges + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        n_edges, src, dst, new_id, out_src, out_dst);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

extern "C" int yitu_edge_span_sum(int64_t n_edges, const int32_t *src, const int32_t *dst, uint64_t *sum_device,
                                  yitu_stream_t stream) {
    YITU_REQUIRE(n_edges >= 0 && sum_device, YITU_ERR_INVALID_ARG, "bad argument");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    YITU_CUDA(cudaMemsetAsync(sum_device, 0, sizeof(uint64_t), st));
    if (n_edges == 0) return YITU_OK;
    YITU_REQUIRE(src && dst, YITU_ERR_INVALID_ARG, "NULL edge list");
    const int64_t want = (n_edges + 255) / 256;
    edge_span_kernel<<<static_cast<unsigned>(want < 148 * 8 ? want : 148 * 8), 256, 0, st>>>(
        n_edges, src, dst, reinterpret_cast<unsigned long long *>(sum_device));
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}
