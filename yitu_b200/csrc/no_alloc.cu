// SpMM entry point for callers that must not allocate device memory.
//
// Some callers of this library cannot call cudaMalloc at the moment they need an aggregation: code running
// inside a memory pool whose budget is fixed up front, plugins that are handed inputs and outputs by a
// framework and are forbidden to touch the allocator, or latency-critical loops where an allocation may
// synchronise the device.  The regular SpMM needs scratch memory (the partial sums of split hub rows) that
// the caller normally allocates; here that scratch is a fixed array that lives in the library image itself.
//
// Consequences of that choice, all part of the contract of yitu_spmm_csr_f32_static:
//   * every GPU that loads the library holds YITU_STATIC_SCRATCH_BYTES (16 MiB) until the process exits;
//   * a call whose hub schedule needs more (plan->n_chunks * H*F floats) is rejected with YITU_ERR_LIMIT;
//   * all calls on a device share the one array, so two calls that overlap on the GPU (different streams)
//     race on it — serialise them on one stream or with events;
//   * the array keeps whatever the previous call left.  Nothing has to be cleared: each chunk slot is fully
//     written by the aggregation kernel before the reduction kernel of the same call reads it;
//   * the first call on each device resolves the array's device address (one cudaGetSymbolAddress, no
//     allocation); make that first call before any stream capture begins.
#include <mutex>

#include "common.cuh"

#define YITU_STATIC_SCRATCH_BYTES (16ll << 20)

// The name below is a host-side handle in host code, not a device address: the address the kernels receive
// is looked up per device with cudaGetSymbolAddress.
static __device__ __align__(256) float g_static_scratch[YITU_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mutex;
float *g_scratch_addr[kMaxDevices] = {};

// Device address of the static scratch on the CURRENT device (resolved once per device).
int static_scratch(float **out) {
    int dev = -1;
    YITU_CUDA(cudaGetDevice(&dev));
    YITU_REQUIRE(dev >= 0 && dev < kMaxDevices, YITU_ERR_LIMIT, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        float *ptr = nullptr;
        YITU_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_scratch));
        YITU_REQUIRE(ptr != nullptr, YITU_ERR_CUDA, "static scratch has no device address on device %d", dev);
        g_scratch_addr[dev] = ptr;
    }
    *out = g_scratch_addr[dev];
    return YITU_OK;
}
}  // namespace

extern "C" int64_t yitu_static_scratch_bytes(void) { return YITU_STATIC_SCRATCH_BYTES; }

extern "C" int yitu_spmm_csr_f32_static(const yitu_spmm_args_t *args, yitu_stream_t stream) {
    YITU_REQUIRE(args != nullptr, YITU_ERR_INVALID_ARG, "args is NULL");
    yitu_spmm_args_t a = *args;
    a.scratch = nullptr;
    a.scratch_bytes = 0;
    if (a.plan != nullptr && a.plan->n_chunks > 0) {
        YITU_REQUIRE(a.n_heads >= 1 && a.n_feats >= 1, YITU_ERR_INVALID_ARG, "n_heads=%lld n_feats=%lld",
                     (long long)a.n_heads, (long long)a.n_feats);
        const int64_t need = a.plan->n_chunks * a.n_heads * a.n_feats * static_cast<int64_t>(sizeof(float));
        YITU_REQUIRE(need <= YITU_STATIC_SCRATCH_BYTES, YITU_ERR_LIMIT,
                     "hub partial sums need %lld bytes but the built-in scratch holds %lld: use a larger "
                     "plan chunk_edges, or yitu_spmm_csr_f32 with caller-allocated scratch",
                     (long long)need, (long long)YITU_STATIC_SCRATCH_BYTES);
        float *ptr = nullptr;
        if (int rc = static_scratch(&ptr)) return rc;
        a.scratch = ptr;
        a.scratch_bytes = YITU_STATIC_SCRATCH_BYTES;
    }
    return yitu_spmm_csr_f32(&a, stream);
}
