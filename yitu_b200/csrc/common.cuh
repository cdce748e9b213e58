// Shared helpers of the yitu_b200 CUDA library (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/yitu_b200.h"

namespace yitu {

void set_error(const char *fmt, ...);

#define YITU_REQUIRE(cond, code, ...)      \
    do {                                   \
        if (!(cond)) {                     \
            ::yitu::set_error(__VA_ARGS__); \
            return (code);                 \
        }                                  \
    } while (0)

#define YITU_CUDA(expr)                                                                              \
    do {                                                                                             \
        cudaError_t e_ = (expr);                                                                     \
        if (e_ != cudaSuccess) {                                                                     \
            ::yitu::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
            return YITU_ERR_CUDA;                                                                    \
        }                                                                                            \
    } while (0)

#define YITU_LAUNCH_CHECK()                                                                      \
    do {                                                                                         \
        cudaError_t e_ = cudaGetLastError();                                                     \
        if (e_ != cudaSuccess) {                                                                 \
            ::yitu::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(e_), __FILE__, __LINE__); \
            return YITU_ERR_CUDA;                                                                \
        }                                                                                        \
    } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ int64_t load_ptr(const void *indptr, int is64, int64_t i) {
    return is64 ? __ldg(reinterpret_cast<const int64_t *>(indptr) + i)
                : static_cast<int64_t>(__ldg(reinterpret_cast<const int32_t *>(indptr) + i));
}

__device__ __forceinline__ float leaky_relu(float v, float slope) {
    return fmaxf(0.0f, v) + slope * fminf(0.0f, v);
}

__device__ __forceinline__ float activate(float v, int act) {
    if (act == YITU_ACT_RELU) return fmaxf(v, 0.0f);
    if (act == YITU_ACT_ELU) return v > 0.0f ? v : expm1f(v);
    return v;
}

// Loads of data that is streamed once (indices, edge values): kept out of L1, and marked evict-first in L2 through
// a cache-hint policy, so that they do not push the gathered feature rows out of the 126 MB L2.
__device__ __forceinline__ uint64_t stream_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ int ld_stream(const int *p) {
    int v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.b32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(stream_policy()));
    return v;
}
__device__ __forceinline__ float ld_stream(const float *p) {
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(stream_policy()));
    return v;
}

// Row slices of VEC floats: 128-bit or (new with sm_100) 256-bit global loads; streaming stores for outputs.
template <int VEC>
__device__ __forceinline__ void load_vec(float (&r)[VEC], const float *p) {
    if constexpr (VEC == 8) {
        // 256-bit global load (new with sm_100): one request moves 32 bytes per lane, 1 KiB per warp
        asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7])
                     : "l"(p));
    } else if constexpr (VEC == 4) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(p));
        r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
    } else {
        r[0] = __ldg(p);
    }
}

template <int VEC>
__device__ __forceinline__ void store_vec(float *p, const float (&r)[VEC]) {
    // output rows are written once and not read again by this kernel: streaming stores (evict-first)
    if constexpr (VEC == 8) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(r[0], r[1], r[2], r[3]));
        __stcs(reinterpret_cast<float4 *>(p) + 1, make_float4(r[4], r[5], r[6], r[7]));
    } else if constexpr (VEC == 4) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(r[0], r[1], r[2], r[3]));
    } else {
        __stcs(p, r[0]);
    }
}

inline int validate_csr(const yitu_csr_t *g) {
    YITU_REQUIRE(g != nullptr, YITU_ERR_INVALID_ARG, "graph is NULL");
    YITU_REQUIRE(g->n_rows >= 0 && g->n_cols >= 0 && g->nnz >= 0, YITU_ERR_INVALID_ARG,
                 "negative graph size (n_rows=%lld n_cols=%lld nnz=%lld)", (long long)g->n_rows,
                 (long long)g->n_cols, (long long)g->nnz);
    YITU_REQUIRE(g->indptr != nullptr, YITU_ERR_INVALID_ARG, "graph.indptr is NULL");
    YITU_REQUIRE(g->nnz == 0 || g->indices != nullptr, YITU_ERR_INVALID_ARG, "graph.indices is NULL");
    YITU_REQUIRE(g->n_rows < (1ll << 31) && g->n_cols < (1ll << 31), YITU_ERR_LIMIT,
                 "node ids must fit int32 (n_rows=%lld n_cols=%lld)", (long long)g->n_rows, (long long)g->n_cols);
    YITU_REQUIRE(g->indptr_is64 || g->nnz < (1ll << 31), YITU_ERR_LIMIT,
                 "nnz=%lld needs int64 row pointers", (long long)g->nnz);
    YITU_REQUIRE(g->index_mask == 0 || g->index_mask == 0xffffff, YITU_ERR_INVALID_ARG,
                 "index_mask must be 0 or 0xffffff");
    return YITU_OK;
}

}  // namespace yitu
