// Halo fetch for the row-partitioned SpMM: copies the listed rows of a feature matrix that is sharded over
// several GPUs into a dense local buffer, reading remote shards with ordinary loads through NVLink peer
// mappings.  One warp per row, 128-bit accesses; bound by NVLink bandwidth for remote rows.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace yitu {

struct HaloParams {
    const float *ptr[16];
    int64_t bound[17];
    int n_shards;
    const int *ids;
    int64_t n_ids, row_floats;
    int64_t stripes, per_stripe;  // visiting order: item j -> id position (j % stripes) * per_stripe + j / stripes
    float *dst;
};

// One warp moves ROWS rows at a time: all ROWS 128-bit loads of a lane are issued before the first store, so
// a warp keeps ROWS * 512 B in flight on the link.  The grid is small (two 8-warp CTAs per SM) so that an SpMM
// running on another stream keeps most of every SM.  The id list is sorted, hence grouped by owner; it is
// visited in a striped order so that at any moment the pulls are spread over all owners (all links busy)
// instead of every rank hammering owner 0 first, then owner 1, ...
template <int ROWS>
__global__ void __launch_bounds__(256) halo_gather_kernel(const __grid_constant__ HaloParams p) {
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
    const int64_t nvec = p.row_floats >> 2;
    const int64_t total = p.stripes * p.per_stripe;
    for (int64_t j0 = warp * ROWS; j0 < total; j0 += n_warps * ROWS) {
        const float4 *src[ROWS];
        float4 *dst[ROWS];
        bool ok[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int64_t j = j0 + r;
            const int64_t i = (j % p.stripes) * p.per_stripe + j / p.stripes;
            ok[r] = j < total && i < p.n_ids;
            src[r] = nullptr;
            dst[r] = nullptr;
            if (ok[r]) {
                const int64_t id = __ldg(p.ids + i);
                int s = 0;
                while (s + 1 < p.n_shards && id >= p.bound[s + 1]) ++s;
                src[r] = reinterpret_cast<const float4 *>(p.ptr[s] + (id - p.bound[s]) * p.row_floats);
                dst[r] = reinterpret_cast<float4 *>(p.dst + i * p.row_floats);
            }
        }
        for (int64_t v = lane; v < nvec; v += 32) {
            float4 val[ROWS];
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (ok[r]) val[r] = src[r][v];
#pragma unroll
            for (int r = 0; r < ROWS; ++r)
                if (ok[r]) dst[r][v] = val[r];
        }
    }
}

}  // namespace yitu

using namespace yitu;

extern "C" int yitu_halo_gather_f32(int32_t n_shards, const float *const *shard_ptrs_host,
                                    const int64_t *shard_bounds_host, const int32_t *ids, int64_t n_ids,
                                    int64_t row_floats, float *dst, yitu_stream_t stream) {
    YITU_REQUIRE(n_shards >= 1 && n_shards <= 16, YITU_ERR_LIMIT, "n_shards=%d (1..16)", n_shards);
    YITU_REQUIRE(shard_ptrs_host && shard_bounds_host, YITU_ERR_INVALID_ARG, "NULL shard table");
    YITU_REQUIRE(row_floats > 0 && row_floats % 4 == 0, YITU_ERR_INVALID_ARG, "row_floats must be a multiple of 4");
    if (n_ids == 0) return YITU_OK;
    YITU_REQUIRE(ids && dst && aligned16(dst), YITU_ERR_INVALID_ARG, "NULL or misaligned ids/dst");
    HaloParams p{};
    p.n_shards = n_shards;
    for (int s = 0; s < n_shards; ++s) {
        YITU_REQUIRE(shard_ptrs_host[s] && aligned16(shard_ptrs_host[s]), YITU_ERR_INVALID_ARG,
                     "shard %d pointer NULL or misaligned", s);
        p.ptr[s] = shard_ptrs_host[s];
        p.bound[s] = shard_bounds_host[s];
    }
    p.bound[n_shards] = shard_bounds_host[n_shards];
    p.ids = ids; p.n_ids = n_ids; p.row_floats = row_floats; p.dst = dst;
    p.stripes = n_ids >= (1 << 16) ? 1024 : 1;
    p.per_stripe = (n_ids + p.stripes - 1) / p.stripes;
    constexpr int kRows = 4;
    const int64_t blocks = (n_ids + 8 * kRows - 1) / (8 * kRows);
    const unsigned grid = static_cast<unsigned>(blocks < 148 * 2 ? blocks : 148 * 2);
    halo_gather_kernel<kRows><<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Owner-side push: the mirror image of the gather above.  The owner of a feature shard copies the rows that each
// peer needs straight into that peer's halo buffer with ordinary stores through the NVLink peer mapping.  Stores
// are posted (nothing waits for a round trip), the reads are local, and the owner paces its own egress - which
// is what bounds the exchange when one shard holds far more rows than the others.
// ---------------------------------------------------------------------------------------------------------
namespace yitu {

struct PushParams {
    float *dst[16];        // halo buffer of destination d (peer mapping), first row of this owner's slot range
    int64_t begin[17];     // items [begin[d], begin[d+1]) of the id list go to destination d
    int n_dests;
    const int *ids;        // local row ids, concatenated by destination, ascending within a destination
    const float *x;        // this rank's feature shard
    int64_t row_floats;
    int64_t stripes, per_stripe;
    unsigned long long *counter;  // next unclaimed item (zeroed before the launch)
};

// CTAs of 1024 threads at 64 registers per thread: each fills the register file of its SM, so the push kernel owns
// exactly gridDim.x SMs and nothing else runs on them.  That is on purpose.  Stores into a saturated NVLink back up
// into the memory pipeline of the SM that issued them, and every other warp on that SM then waits behind them:
// with two 256-thread push CTAs on EVERY SM an aggregation running beside the push crawled (the own-source pass of
// a rank took 4.8 ms beside its push and 0.6 ms alone).  About twenty SMs move more than one link direction
// carries; the other SMs keep a free memory pipeline for the aggregation.
template <int ROWS>
__global__ void __launch_bounds__(1024, 1) halo_push_kernel(const __grid_constant__ PushParams p) {
    static_assert(32 % ROWS == 0, "a claim of 32 items is copied in groups of ROWS");
    const int lane = threadIdx.x & 31;
    const int64_t nvec = p.row_floats >> 2;
    const int64_t n_items = p.begin[p.n_dests];
    const int64_t total = p.stripes * p.per_stripe;
    // A warp claims 32 items at a time from a global counter (not dealt out in advance: on B200 the warps of a
    // statically partitioned grid finished between 55 % and 100 % of the kernel's duration - SMs differ in their
    // distance to the NVLink ports - and the slowest decided when the shard had left).  Lane l resolves item l of the
    // claim (one coalesced read of the ids, the destination looked up once); the rows are then copied ROWS at a
    // time, source and destination addresses handed round by shuffles, all loads of a group issued before its stores.
    for (;;) {
        unsigned long long claim = 0;
        if (lane == 0) claim = atomicAdd(p.counter, 32ull);
        const int64_t j0 = static_cast<int64_t>(__shfl_sync(0xffffffffu, claim, 0));
        if (j0 >= total) break;
        // striped visiting order: consecutive items come from all over the list, hence from every destination, so
        // every link out of this GPU is busy from the first moment to the last
        const int64_t j = j0 + lane;
        const int64_t i = (j % p.stripes) * p.per_stripe + j / p.stripes;
        const bool mine = j < total && i < n_items;
        const float4 *my_src = nullptr;
        float4 *my_dst = nullptr;
        if (mine) {
            int d = 0;
            while (d + 1 < p.n_dests && i >= p.begin[d + 1]) ++d;
            my_src = reinterpret_cast<const float4 *>(p.x + static_cast<int64_t>(__ldg(p.ids + i)) * p.row_floats);
            my_dst = reinterpret_cast<float4 *>(p.dst[d] + (i - p.begin[d]) * p.row_floats);
        }
        const unsigned have = __ballot_sync(0xffffffffu, mine);
        for (int g = 0; g < 32; g += ROWS) {
            if (((have >> g) & ((1u << ROWS) - 1u)) == 0u) continue;
            const float4 *src[ROWS];
            float4 *dst[ROWS];
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                src[r] = reinterpret_cast<const float4 *>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_src), g + r));
                dst[r] = reinterpret_cast<float4 *>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_dst), g + r));
            }
            for (int64_t v = lane; v < nvec; v += 32) {
                float4 val[ROWS];
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (src[r]) val[r] = __ldg(src[r] + v);
#pragma unroll
                for (int r = 0; r < ROWS; ++r)
                    if (src[r]) dst[r][v] = val[r];
            }
        }
    }
}

}  // namespace yitu

extern "C" int yitu_halo_push_f32(int32_t n_dests, float *const *dst_ptrs_host, const int64_t *list_begin_host,
                                  const int32_t *ids, const float *x, int64_t row_floats, uint64_t *work_counter,
                                  int32_t n_sms, yitu_stream_t stream) {
    YITU_REQUIRE(n_dests >= 0 && n_dests <= 16, YITU_ERR_LIMIT, "n_dests=%d (0..16)", n_dests);
    YITU_REQUIRE(row_floats > 0 && row_floats % 4 == 0, YITU_ERR_INVALID_ARG, "row_floats must be a multiple of 4");
    if (n_dests == 0) return YITU_OK;
    YITU_REQUIRE(dst_ptrs_host && list_begin_host, YITU_ERR_INVALID_ARG, "NULL destination table");
    PushParams p{};
    p.n_dests = n_dests;
    YITU_REQUIRE(list_begin_host[0] == 0, YITU_ERR_INVALID_ARG, "list_begin[0] must be 0");
    for (int d = 0; d < n_dests; ++d) {
        YITU_REQUIRE(list_begin_host[d + 1] >= list_begin_host[d], YITU_ERR_INVALID_ARG, "list_begin must not decrease");
        YITU_REQUIRE(list_begin_host[d + 1] == list_begin_host[d] || (dst_ptrs_host[d] && aligned16(dst_ptrs_host[d])),
                     YITU_ERR_INVALID_ARG, "destination %d pointer NULL or misaligned", d);
        p.dst[d] = dst_ptrs_host[d];
        p.begin[d] = list_begin_host[d];
    }
    p.begin[n_dests] = list_begin_host[n_dests];
    const int64_t n_items = p.begin[n_dests];
    if (n_items == 0) return YITU_OK;
    YITU_REQUIRE(ids && x && aligned16(x), YITU_ERR_INVALID_ARG, "NULL or misaligned ids/x");
    YITU_REQUIRE(work_counter != nullptr, YITU_ERR_INVALID_ARG, "work_counter is NULL (8 bytes of device memory)");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    YITU_CUDA(cudaMemsetAsync(work_counter, 0, sizeof(uint64_t), st));
    p.ids = ids; p.x = x; p.row_floats = row_floats;
    p.counter = reinterpret_cast<unsigned long long *>(work_counter);
    p.stripes = n_items >= (1 << 16) ? 1024 : 1;
    p.per_stripe = (n_items + p.stripes - 1) / p.stripes;
    constexpr int kRows = 8;
    const int64_t blocks = (n_items + 32 * 32 - 1) / (32 * 32);
    // SMs given to the push (one CTA each).  Default 24: measured on B200, 3.0 GB to one peer took 9.5 / 4.7 / 4.24 /
    // 4.24 ms with 8 / 16 / 24 / 32 SMs (711 GB/s from 24 on: the link is full), and an aggregation running beside
    // it lost 4 % at 24 SMs.  YITU_PUSH_CTAS is a development switch that overrides the argument.
    YITU_REQUIRE(n_sms >= 0 && n_sms <= 1024, YITU_ERR_INVALID_ARG, "n_sms=%d (0 = default)", n_sms);
    const char *env = getenv("YITU_PUSH_CTAS");
    const int64_t max_blocks = (env && *env) ? atoll(env) : (n_sms > 0 ? n_sms : 24);
    const unsigned grid = static_cast<unsigned>(blocks < max_blocks ? blocks : (max_blocks > 0 ? max_blocks : 1));
    halo_push_kernel<kRows><<<grid, 1024, 0, st>>>(p);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

// ---------------------------------------------------------------------------------------------------------
// "My rows are with you": a 64-bit flag per (reader, owner) pair in the reader's memory.  The owner raises it, in
// stream order after its push kernel, by storing the step number through the peer mapping; the reader's stream
// waits for it with a one-warp kernel before the aggregation pass that needs those rows.  A collective cannot do
// this job while the push runs: its kernel needs a free SM, and the push kernel's resident CTAs occupy every SM until
// they are done (measured: a one-float all-reduce issued at the start of the exchange completed after 5.7 ms; the
// same all-reduce with half the SMs left free, after 0.19 ms).  The two kernels below need no shared memory and 32
// threads, and run beside anything.
// The wait is bounded: after `timeout_ns` the kernel records which flag was missing and returns, so a peer that
// never signals costs a wrong result that the host can see, not a hung GPU.
// ---------------------------------------------------------------------------------------------------------
namespace yitu {

struct SignalParams {
    unsigned long long *target[16];
    int n;
    unsigned long long value;
};

__global__ void flags_signal_kernel(const __grid_constant__ SignalParams p) {
    const int i = threadIdx.x;
    if (i < p.n) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p.target[i]), "l"(p.value) : "memory");
    }
}

__global__ void flags_wait_kernel(const unsigned long long *flags, unsigned mask, unsigned long long value,
                                  long long timeout_ns, int *error) {
    const int i = threadIdx.x;
    if (!((mask >> i) & 1u)) return;
    unsigned long long start;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
    for (;;) {
        unsigned long long v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flags + i) : "memory");
        if (v >= value) return;
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (static_cast<long long>(now - start) > timeout_ns) {
            atomicCAS(error, 0, 1 + i);  // first missing flag, 1-based
            return;
        }
        __nanosleep(200);
    }
}

}  // namespace yitu

extern "C" int yitu_flags_signal(int32_t n, uint64_t *const *targets_host, uint64_t value, yitu_stream_t stream) {
    YITU_REQUIRE(n >= 0 && n <= 16, YITU_ERR_LIMIT, "n=%d (0..16)", n);
    if (n == 0) return YITU_OK;
    YITU_REQUIRE(targets_host != nullptr, YITU_ERR_INVALID_ARG, "NULL target table");
    SignalParams p{};
    p.n = n;
    p.value = value;
    for (int i = 0; i < n; ++i) {
        YITU_REQUIRE(targets_host[i] && (reinterpret_cast<uintptr_t>(targets_host[i]) & 7) == 0, YITU_ERR_INVALID_ARG,
                     "target %d NULL or misaligned", i);
        p.target[i] = reinterpret_cast<unsigned long long *>(targets_host[i]);
    }
    flags_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

extern "C" int yitu_flags_wait(const uint64_t *flags, uint32_t mask, uint64_t value, int64_t timeout_ns,
                               int32_t *error_flag, yitu_stream_t stream) {
    if (mask == 0) return YITU_OK;
    YITU_REQUIRE(flags && error_flag, YITU_ERR_INVALID_ARG, "NULL flags / error_flag");
    YITU_REQUIRE(timeout_ns > 0 && timeout_ns <= 10000000000ll, YITU_ERR_INVALID_ARG,
                 "timeout_ns=%lld: the wait must be bounded (at most 10 s)", (long long)timeout_ns);
    flags_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const unsigned long long *>(flags), mask, value, timeout_ns, error_flag);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Peer-readable feature shards (CUDA IPC).  Allocation happens once per shard at set-up, never per step.
// ---------------------------------------------------------------------------------------------------------
static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");

extern "C" int yitu_shared_alloc(int64_t bytes, void **ptr_out, unsigned char *handle_out) {
    YITU_REQUIRE(bytes > 0 && ptr_out && handle_out, YITU_ERR_INVALID_ARG, "bad argument");
    void *p = nullptr;
    YITU_CUDA(cudaMalloc(&p, static_cast<size_t>(bytes)));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        set_error("cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
        return YITU_ERR_CUDA;
    }
    memcpy(handle_out, &h, sizeof(h));
    *ptr_out = p;
    return YITU_OK;
}

extern "C" int yitu_shared_open(const unsigned char *handle, void **ptr_out) {
    YITU_REQUIRE(handle && ptr_out, YITU_ERR_INVALID_ARG, "bad argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    YITU_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr_out = p;
    return YITU_OK;
}

extern "C" int yitu_shared_close(void *ptr) {
    if (ptr) YITU_CUDA(cudaIpcCloseMemHandle(ptr));
    return YITU_OK;
}

extern "C" int yitu_shared_free(void *ptr) {
    if (ptr) YITU_CUDA(cudaFree(ptr));
    return YITU_OK;
}
