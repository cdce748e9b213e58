// GAT attention kernels for sm_100a.
//
//   edge_softmax_{fwd,bwd}  stand-alone "SDDMM" of the reference (u_add_v -> LeakyReLU -> per-segment edge
//                           softmax) with [nnz,H] attention in memory — the drop-in operator path;
//   edge_dot                grad of the per-edge values of a multi-head SpMM;
//   edge_gather_sum         per-source sum of per-edge gradients over the transposed graph (replaces the
//                           reference's atomicAdd scatter);
//   gat_fwd / gat_bwd       the fused layer core: one pass over a row's edges computes scores, an online
//                           max/sum softmax and the weighted aggregation; the backward is one pass over the
//                           transposed graph that reuses every gathered gradient row for grad_x and for d attn
//                           (attention rebuilt per edge from the forward's row statistics);
//   hub rows                every kernel takes the optional hub schedule: long rows are cut into chunks with an ordered
//                           merge, or handed to a whole CTA.
//
// All of them are bound by gather bandwidth (HBM/L2); none uses float atomics.
#include <math_constants.h>

#include <type_traits>

#include "common.cuh"

namespace yitu {

__device__ __forceinline__ int pow2_shift(int v) { return 31 - __clz(v); }

// ---------------------------------------------------------------------------------------------------------
// Stand-alone edge softmax.  One warp per row; a lane is (edge slot, head): HB = pow2 >= min(H,32) lanes
// span the heads (coalesced key / attn accesses), 32/HB edges advance together.
// ---------------------------------------------------------------------------------------------------------
struct SoftmaxParams {
    int64_t n_rows;
    const void *indptr;
    const int *indices;
    int is64, mask, B, H, HB;
    float slope;
    const float *q, *k, *attn_in, *grad_attn;
    float *attn_out, *grad_q, *edge_grad;
    // optional hub schedule: rows longer than chunk_edges are left to the CTA-per-row variants below
    int64_t n_chunks;
    int chunk_edges;
    const int *chunk_row;
    const int64_t *chunk_begin;
};

// Row assignment shared by the stand-alone kernels.  CTA = false: one warp per row, hub rows skipped when a schedule
// is given.  CTA = true: one 256-thread CTA per hub row (launched with one CTA per chunk; the CTAs of a row's later
// chunks leave at once), its 256/HB edge slots advancing together.
template <bool CTA>
__device__ __forceinline__ bool softmax_row(const SoftmaxParams &p, int64_t &row, int64_t &eb, int64_t &ee) {
    if constexpr (CTA) {
        row = __ldg(p.chunk_row + blockIdx.x);
        eb = load_ptr(p.indptr, p.is64, row);
        if (__ldg(p.chunk_begin + blockIdx.x) != eb) return false;
        ee = load_ptr(p.indptr, p.is64, row + 1);
        return true;
    } else {
        row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
        if (row >= p.n_rows) return false;
        eb = load_ptr(p.indptr, p.is64, row);
        ee = load_ptr(p.indptr, p.is64, row + 1);
        return !(p.n_chunks > 0 && ee - eb > p.chunk_edges);
    }
}

// Sum over the edge slots that share a head lane: shuffles inside the warp, then (CTA) across the 8 warps through
// shared memory, every thread adding the 8 values in the same order.
template <bool CTA>
__device__ __forceinline__ float slot_sum(float v, int HB, float *s_red) {
    for (int o = HB; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if constexpr (CTA) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, hs = lane & (HB - 1);
        __syncthreads();
        if (lane < HB) s_red[warp * 32 + hs] = v;
        __syncthreads();
        v = 0.0f;
        for (int w = 0; w < 8; ++w) v += s_red[w * 32 + hs];
    }
    return v;
}

template <bool CTA>
__global__ void __launch_bounds__(256) edge_softmax_fwd_kernel(const __grid_constant__ SoftmaxParams p) {
    __shared__ float s_red[CTA ? 2 * 8 * 32 : 1];
    int64_t row, eb, ee;
    if (!softmax_row<CTA>(p, row, eb, ee)) return;
    const int lane = threadIdx.x & 31;
    const int hs = lane & (p.HB - 1);
    const int slot = (CTA ? threadIdx.x : lane) >> pow2_shift(p.HB);
    const int ES = (CTA ? 256 : 32) / p.HB;
    for (int s = 0; s < p.B; ++s) {
        for (int hc = 0; hc < p.H; hc += p.HB) {
            const int h = hc + hs;
            const bool hv = h < p.H;
            const float qv = hv ? __ldg(p.q + (static_cast<int64_t>(s) * p.n_rows + row) * p.H + h) : 0.0f;
            float m = -CUDART_INF_F, l = 0.0f;
            for (int64_t e = eb + slot; e < ee; e += ES) {
                const int raw = __ldg(p.indices + e);
                const int bid = p.mask ? static_cast<int>(static_cast<unsigned>(raw) >> 24) : 0;
                if (bid != s || !hv) continue;
                const int col = p.mask ? (raw & p.mask) : raw;
                const float z = leaky_relu(qv + __ldg(p.k + static_cast<int64_t>(col) * p.H + h), p.slope);
                if (z > m) {
                    l = l * expf(m - z) + 1.0f;
                    m = z;
                } else {
                    l += expf(z - m);
                }
            }
            for (int o = p.HB; o < 32; o <<= 1) {
                const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
                const float l2 = __shfl_xor_sync(0xffffffffu, l, o);
                const float M = fmaxf(m, m2);
                if (M > -CUDART_INF_F) l = l * expf(m - M) + l2 * expf(m2 - M);
                m = M;
            }
            if constexpr (CTA) {
                const int warp = threadIdx.x >> 5;
                __syncthreads();
                if (lane < p.HB) {
                    s_red[warp * 32 + hs] = m;
                    s_red[256 + warp * 32 + hs] = l;
                }
                __syncthreads();
                float M = -CUDART_INF_F;
                for (int w = 0; w < 8; ++w) M = fmaxf(M, s_red[w * 32 + hs]);
                float L = 0.0f;
                if (M > -CUDART_INF_F)
                    for (int w = 0; w < 8; ++w) L += s_red[256 + w * 32 + hs] * expf(s_red[w * 32 + hs] - M);
                m = M;
                l = L;
            }
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            for (int64_t e = eb + slot; e < ee; e += ES) {
                const int raw = __ldg(p.indices + e);
                const int bid = p.mask ? static_cast<int>(static_cast<unsigned>(raw) >> 24) : 0;
                if (bid != s || !hv) continue;
                const int col = p.mask ? (raw & p.mask) : raw;
                const float z = leaky_relu(qv + __ldg(p.k + static_cast<int64_t>(col) * p.H + h), p.slope);
                p.attn_out[e * p.H + h] = expf(z - m) * inv;
            }
        }
    }
}

template <bool CTA>
__global__ void __launch_bounds__(256) edge_softmax_bwd_kernel(const __grid_constant__ SoftmaxParams p) {
    __shared__ float s_red[CTA ? 8 * 32 : 1];
    int64_t row, eb, ee;
    if (!softmax_row<CTA>(p, row, eb, ee)) return;
    const int lane = threadIdx.x & 31;
    const int hs = lane & (p.HB - 1);
    const int slot = (CTA ? threadIdx.x : lane) >> pow2_shift(p.HB);
    const int ES = (CTA ? 256 : 32) / p.HB;
    for (int s = 0; s < p.B; ++s) {
        for (int hc = 0; hc < p.H; hc += p.HB) {
            const int h = hc + hs;
            const bool hv = h < p.H;
            const float qv = hv ? __ldg(p.q + (static_cast<int64_t>(s) * p.n_rows + row) * p.H + h) : 0.0f;
            float t = 0.0f;  // sum over the segment of attn * grad
            for (int64_t e = eb + slot; e < ee; e += ES) {
                const int raw = __ldg(p.indices + e);
                const int bid = p.mask ? static_cast<int>(static_cast<unsigned>(raw) >> 24) : 0;
                if (bid != s || !hv) continue;
                t = fmaf(__ldg(p.attn_in + e * p.H + h), __ldg(p.grad_attn + e * p.H + h), t);
            }
            t = slot_sum<CTA>(t, p.HB, s_red);
            float gq = 0.0f;
            for (int64_t e = eb + slot; e < ee; e += ES) {
                const int raw = __ldg(p.indices + e);
                const int bid = p.mask ? static_cast<int>(static_cast<unsigned>(raw) >> 24) : 0;
                if (bid != s || !hv) continue;
                const int col = p.mask ? (raw & p.mask) : raw;
                const float a = __ldg(p.attn_in + e * p.H + h);
                const float gs = a * (__ldg(p.grad_attn + e * p.H + h) - t);
                const float z = qv + __ldg(p.k + static_cast<int64_t>(col) * p.H + h);
                const float gv = gs * (z < 0.0f ? p.slope : 1.0f);
                p.edge_grad[e * p.H + h] = gv;
                gq += gv;
            }
            gq = slot_sum<CTA>(gq, p.HB, s_red);
            if (slot == 0 && hv) p.grad_q[(static_cast<int64_t>(s) * p.n_rows + row) * p.H + h] = gq;
        }
    }
}

// out[c,h] = sum over column c of the transposed graph of vals[perm[j], h]
struct GatherSumParams {
    int64_t n_cols;
    const void *t_indptr;
    int is64;
    const int *perm;
    int H, HB;
    const float *vals;
    float *out;
    int64_t n_chunks;
    int chunk_edges;
    const int *chunk_row;
    const int64_t *chunk_begin;
};

template <bool CTA>
__global__ void __launch_bounds__(256) edge_gather_sum_kernel(const __grid_constant__ GatherSumParams p) {
    __shared__ float s_red[CTA ? 8 * 32 : 1];
    int64_t c, b, e;
    if constexpr (CTA) {
        c = __ldg(p.chunk_row + blockIdx.x);
        b = load_ptr(p.t_indptr, p.is64, c);
        if (__ldg(p.chunk_begin + blockIdx.x) != b) return;
        e = load_ptr(p.t_indptr, p.is64, c + 1);
    } else {
        c = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
        if (c >= p.n_cols) return;
        b = load_ptr(p.t_indptr, p.is64, c);
        e = load_ptr(p.t_indptr, p.is64, c + 1);
        if (p.n_chunks > 0 && e - b > p.chunk_edges) return;
    }
    const int lane = threadIdx.x & 31;
    const int H = p.H, HB = p.HB;
    const int hs = lane & (HB - 1);
    const int slot = (CTA ? threadIdx.x : lane) >> pow2_shift(HB);
    const int ES = (CTA ? 256 : 32) / HB;
    const int *perm = p.perm;
    const float *vals = p.vals;
    for (int hc = 0; hc < H; hc += HB) {
        const int h = hc + hs;
        float a = 0.0f;
        if (h < H) {
            int64_t j = b + slot;
            // four permutation loads (none when perm is NULL: the identity), then four value loads, in flight together
            for (; j + 3 * ES < e; j += 4 * ES) {
                int64_t p0 = j, p1 = j + ES, p2 = j + 2 * ES, p3 = j + 3 * ES;
                if (perm != nullptr) {
                    p0 = __ldg(perm + j); p1 = __ldg(perm + j + ES); p2 = __ldg(perm + j + 2 * ES); p3 = __ldg(perm + j + 3 * ES);
                }
                const float v0 = __ldg(vals + p0 * H + h), v1 = __ldg(vals + p1 * H + h), v2 = __ldg(vals + p2 * H + h),
                            v3 = __ldg(vals + p3 * H + h);
                a += v0; a += v1; a += v2; a += v3;
            }
            for (; j < e; j += ES) a += __ldg(vals + (perm ? static_cast<int64_t>(__ldg(perm + j)) : j) * H + h);
        }
        a = slot_sum<CTA>(a, HB, s_red);
        if (slot == 0 && h < H) p.out[c * H + h] = a;
    }
}

// grad_a[e,h] = <g[row,h,:], x[col,h,:]>.  A group of LP = pow2 >= min(F,32) lanes owns one (edge, head) pair.
__global__ void __launch_bounds__(256)
edge_dot_kernel(int64_t n_rows, const void *indptr, int is64, const int *indices, int mask, int H, int F, int LP,
                const float *g, int g_shared, float g_scale, const float *x, float *grad_a) {
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const int gl = lane & (LP - 1);
    const int grp = lane >> pow2_shift(LP);
    const int G = 32 / LP;
    const int64_t eb = load_ptr(indptr, is64, row), ee = load_ptr(indptr, is64, row + 1);
    const int64_t D = static_cast<int64_t>(H) * F;
    const int64_t pairs = (ee - eb) * H;
    const float *gr = g + row * (g_shared ? F : D);  // g_shared: one F-wide gradient row serves every head
    for (int64_t pb = 0; pb < pairs; pb += G) {  // uniform trip count: every lane joins the shuffles
        const int64_t pi = pb + grp;
        float a = 0.0f;
        int64_t e = 0;
        int h = 0;
        if (pi < pairs) {
            e = eb + pi / H;
            h = static_cast<int>(pi % H);
            const int raw = __ldg(indices + e);
            const int col = mask ? (raw & mask) : raw;
            const float *xr = x + static_cast<int64_t>(col) * D + static_cast<int64_t>(h) * F;
            const float *gh = g_shared ? gr : gr + static_cast<int64_t>(h) * F;
            for (int k = gl; k < F; k += LP) a = fmaf(__ldg(gh + k), __ldg(xr + k), a);
        }
        for (int o = LP >> 1; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (pi < pairs && gl == 0) grad_a[e * H + h] = a * g_scale;
    }
}

// Fast path of edge_dot for F a multiple of 4 with F/4 a power of two and H*F <= 512: one warp per row keeps the
// row of g in registers, gathers the source rows with 128-bit loads (two edges in flight), reduces each head's
// partial products with log2(F/4) shuffles, and writes the [32 edges, H] tile of results coalesced.
template <int NV>
__global__ void __launch_bounds__(256)
edge_dot_rows_kernel(int64_t n_rows, const void *indptr, int is64, const int *indices, int mask, int H, int F,
                     const float *g, int g_shared, float g_scale, const float *x, float *grad_a, int64_t n_chunks,
                     int chunk_edges, const int *chunk_row, const int64_t *chunk_begin) {
    extern __shared__ float smem[];
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the first n_chunks warps take the chunks of the hub rows (every edge is independent: nothing to merge)
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + wib;
    int64_t row, eb, ee;
    if (gid < n_chunks) {
        row = __ldg(chunk_row + gid);
        eb = __ldg(chunk_begin + gid);
        ee = min(eb + static_cast<int64_t>(chunk_edges), load_ptr(indptr, is64, row + 1));
    } else {
        row = gid - n_chunks;
        if (row >= n_rows) return;
        eb = load_ptr(indptr, is64, row);
        ee = load_ptr(indptr, is64, row + 1);
        if (n_chunks > 0 && ee - eb > chunk_edges) return;
    }
    float *base = smem + wib * (32 + 32 * H);
    int *s_col = reinterpret_cast<int *>(base);
    float *s_out = base + 32;
    const int64_t D = static_cast<int64_t>(H) * F;
    const int LPH = F >> 2;
    int hd[NV];
    bool valid[NV];
    int64_t off[NV];
    float4 gr[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        off[i] = static_cast<int64_t>(i * 32 + lane) * 4;
        valid[i] = off[i] < D;
        hd[i] = valid[i] ? static_cast<int>(off[i] / F) : 0;
        gr[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (valid[i]) {
            const float *gp = g_shared ? g + row * F + (off[i] - static_cast<int64_t>(hd[i]) * F) : g + row * D + off[i];
            gr[i] = __ldg(reinterpret_cast<const float4 *>(gp));
            gr[i].x *= g_scale; gr[i].y *= g_scale; gr[i].z *= g_scale; gr[i].w *= g_scale;
        }
    }
    for (int64_t e0 = eb; e0 < ee; e0 += 32) {
        const int n = static_cast<int>(min(static_cast<int64_t>(32), ee - e0));
        int my_col = lane < n ? ld_stream(indices + e0 + lane) : 0;
        if (mask) my_col &= mask;
        const int c_first = __shfl_sync(0xffffffffu, my_col, 0);
        s_col[lane] = lane < n ? my_col : c_first;
        __syncwarp();
        const int n2 = (n + 1) & ~1;
        for (int j = 0; j < n2; j += 2) {
            float4 v[2][NV];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const float *xr = x + static_cast<int64_t>(s_col[j + u]) * D;
#pragma unroll
                for (int i = 0; i < NV; ++i)
                    v[u][i] = valid[i] ? __ldg(reinterpret_cast<const float4 *>(xr + off[i]))
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    float d = gr[i].x * v[u][i].x + gr[i].y * v[u][i].y + gr[i].z * v[u][i].z + gr[i].w * v[u][i].w;
                    for (int s = LPH >> 1; s > 0; s >>= 1) d += __shfl_xor_sync(0xffffffffu, d, s);
                    if (valid[i] && (lane & (LPH - 1)) == 0 && j + u < n) s_out[(j + u) * H + hd[i]] = d;
                }
        }
        __syncwarp();
        for (int idx = lane; idx < n * H; idx += 32) grad_a[e0 * H + idx] = s_out[idx];
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------------------------
// Fused GAT forward.  One warp per destination row, tiles of 32 edges.
//   per tile: lanes fetch 32 column ids; (edge, head) pairs are spread over the lanes to compute the scores
//   with coalesced key reads; lane h folds the tile into head h's running (max, sum); then every lane
//   gathers its NV 128-bit slices of each source row and accumulates p * x.  Accumulators are rescaled when
//   the running maximum moves (online softmax), and divided by the sum once at the end.
// Shared memory per warp: 32 column ids, 32*H scores/probabilities, H-sized scale / max / sum / query rows.
// ---------------------------------------------------------------------------------------------------------
struct GatParams {
    int64_t n_rows;
    const void *indptr;
    const int *indices;
    int is64, H, F, hshift;  // hshift = log2(H) if H is a power of two, else -1
    float slope;
    const float *q, *k, *x;
    float *out, *row_max, *row_sum;
    int head_mean, act, stage;  // stage = floats of per-warp staging for the head mean (H*F or 0)
    float *out_heads;           // head_mean: optional per-head result [n_rows,H,F]
    // hub rows: chunk c covers edges [chunk_begin[c], +chunk_edges) of row chunk_row[c]; its unnormalised sums, running
    // maxima and sums go to partial[c] = {H*F, H, H} floats and gat_fwd_merge_kernel finishes the row
    int64_t n_chunks;
    int chunk_edges;
    const int *chunk_row;
    const int64_t *chunk_begin;
    float *partial;
};

// edges per tile of the fused forward (64: 6.52 against 6.56 ms on the uniform 8x32 layer, but 5.87 against 5.16 ms on the
// power-law graph, whose many short rows pay for the larger shared-memory footprint)
constexpr int FWD_TILE = 32;
__host__ __device__ __forceinline__ int warp_smem_floats_fwd(int H, int stage) {
    return FWD_TILE + FWD_TILE * H + 4 * 32 + stage;
}

// floats of one hub chunk's partial result: H*F sums, then H maxima and H sums (padded so that chunks stay 16-byte aligned)
__host__ __device__ __forceinline__ int64_t fwd_partial_stride(int64_t H, int64_t F) { return H * F + ((2 * H + 3) & ~3ll); }

template <int NV, bool MEAN, bool PLAN>
__device__ __forceinline__ void gat_fwd_body(const GatParams &p) {
    extern __shared__ float smem[];
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + wib;
    int64_t row, eb, ee;
    bool chunk = false;  // PLAN = false is the kernel for graphs without hub rows: no schedule logic at all
    if constexpr (PLAN) {
        chunk = gid < p.n_chunks;
        if (chunk) {
            row = __ldg(p.chunk_row + gid);
            eb = __ldg(p.chunk_begin + gid);
            ee = min(eb + static_cast<int64_t>(p.chunk_edges), load_ptr(p.indptr, p.is64, row + 1));
        } else {
            row = gid - p.n_chunks;
            if (row >= p.n_rows) return;
            eb = load_ptr(p.indptr, p.is64, row);
            ee = load_ptr(p.indptr, p.is64, row + 1);
            if (ee - eb > p.chunk_edges) return;  // hub row: done by its chunks
        }
    } else {
        row = gid;
        if (row >= p.n_rows) return;
        eb = load_ptr(p.indptr, p.is64, row);
        ee = load_ptr(p.indptr, p.is64, row + 1);
    }
    const int H = p.H;
    float *base = smem + wib * warp_smem_floats_fwd(H, p.stage);
    int *s_col = reinterpret_cast<int *>(base);
    float *s_p = base + FWD_TILE;
    float *s_scale = s_p + FWD_TILE * H;
    float *s_m = s_scale + 32;
    float *s_q = s_m + 32;
    float *s_l = s_q + 32;

    const int64_t D = static_cast<int64_t>(H) * p.F;
    int hd[NV];
    bool valid[NV];
    int64_t off[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        off[i] = static_cast<int64_t>(i * 32 + lane) * 4;
        valid[i] = off[i] < D;
        hd[i] = valid[i] ? static_cast<int>(off[i] / p.F) : 0;
    }
    float acc[NV][4];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

    if (lane < H) s_q[lane] = __ldg(p.q + row * H + lane);
    float m_run = -CUDART_INF_F, l_run = 0.0f;  // lane h owns head h
    __syncwarp();

    for (int64_t e0 = eb; e0 < ee; e0 += FWD_TILE) {
        const int n = static_cast<int>(min(static_cast<int64_t>(FWD_TILE), ee - e0));
        int my_col[FWD_TILE / 32];
#pragma unroll
        for (int t = 0; t < FWD_TILE / 32; ++t) my_col[t] = t * 32 + lane < n ? ld_stream(p.indices + e0 + t * 32 + lane) : 0;
        const int c_first = __shfl_sync(0xffffffffu, my_col[0], 0);
#pragma unroll
        for (int t = 0; t < FWD_TILE / 32; ++t) s_col[t * 32 + lane] = t * 32 + lane < n ? my_col[t] : c_first;
        __syncwarp();
        const int npairs = n * H;
        for (int idx = lane; idx < npairs; idx += 32) {
            const int e = p.hshift >= 0 ? (idx >> p.hshift) : (idx / H);
            const int h = idx - e * H;
            s_p[idx] = leaky_relu(s_q[h] + __ldg(p.k + static_cast<int64_t>(s_col[e]) * H + h), p.slope);
        }
        __syncwarp();
        const int n4 = (n + 3) & ~3;
        if (p.hshift >= 0) {
            // H a power of two: a lane's pairs idx = lane + 32t all belong to head lane % H, so the tile's maximum and
            // sum are butterflies over the lanes of equal lane % H; every lane keeps the running statistics of that head
            float tm = -CUDART_INF_F;
            for (int idx = lane; idx < npairs; idx += 32) tm = fmaxf(tm, s_p[idx]);
            for (int o = H; o < 32; o <<= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
            const float m_new = fmaxf(m_run, tm);
            const float sc = expf(m_run - m_new);  // 0 on the first tile (m_run = -inf)
            if (lane < H) s_scale[lane] = sc;
            float ls = 0.0f;
            for (int idx = lane; idx < n4 * H; idx += 32) {
                const float v = idx < npairs ? expf(s_p[idx] - m_new) : 0.0f;
                s_p[idx] = v;
                ls += v;
            }
            for (int o = H; o < 32; o <<= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
            l_run = l_run * sc + ls;
            m_run = m_new;
            __syncwarp();
        } else {
            if (lane < H) {
                float tm = -CUDART_INF_F;
                for (int e = 0; e < n; ++e) tm = fmaxf(tm, s_p[e * H + lane]);
                const float m_new = fmaxf(m_run, tm);
                const float sc = expf(m_run - m_new);  // 0 on the first tile (m_run = -inf)
                s_scale[lane] = sc;
                s_m[lane] = m_new;
                l_run *= sc;
                m_run = m_new;
            }
            __syncwarp();
            for (int idx = lane; idx < n4 * H; idx += 32) {
                const int e = idx / H;
                const int h = idx - e * H;
                s_p[idx] = idx < npairs ? expf(s_p[idx] - s_m[h]) : 0.0f;
            }
            __syncwarp();
            if (lane < H) {
                float ls = 0.0f;
                for (int e = 0; e < n; ++e) ls += s_p[e * H + lane];
                l_run += ls;
            }
        }
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float sc = s_scale[hd[i]];
            acc[i][0] *= sc; acc[i][1] *= sc; acc[i][2] *= sc; acc[i][3] *= sc;
        }
        for (int j = 0; j < n4; j += 4) {
            float4 v[4][NV];
            float w[4][NV];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float *xr = p.x + static_cast<int64_t>(s_col[j + u]) * D;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    if (valid[i]) {
                        v[u][i] = __ldg(reinterpret_cast<const float4 *>(xr + off[i]));
                        w[u][i] = s_p[(j + u) * H + hd[i]];
                    } else {
                        v[u][i] = make_float4(0.f, 0.f, 0.f, 0.f);
                        w[u][i] = 0.0f;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    acc[i][0] = fmaf(w[u][i], v[u][i].x, acc[i][0]);
                    acc[i][1] = fmaf(w[u][i], v[u][i].y, acc[i][1]);
                    acc[i][2] = fmaf(w[u][i], v[u][i].z, acc[i][2]);
                    acc[i][3] = fmaf(w[u][i], v[u][i].w, acc[i][3]);
                }
        }
        __syncwarp();
    }
    if (PLAN && chunk) {
        float *part = p.partial + gid * fwd_partial_stride(H, p.F);
#pragma unroll
        for (int i = 0; i < NV; ++i)
            if (valid[i])
                *reinterpret_cast<float4 *>(part + off[i]) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        if (lane < H) {
            part[D + lane] = m_run;
            part[D + H + lane] = l_run;
        }
        return;
    }
    if (lane < H) {
        s_l[lane] = l_run;
        p.row_max[row * H + lane] = m_run;
        p.row_sum[row * H + lane] = l_run;
    }
    __syncwarp();
    if constexpr (MEAN) {
        // the layer's mean over heads: stage the H*F results, then lane f adds the H values of feature f in head
        // order (fixed order: deterministic) — the [n_rows,H,F] tensor is never written
        float *s_o = s_l + 32;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (!valid[i]) continue;
            const float l = s_l[hd[i]];
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            const float4 r = make_float4(acc[i][0] * inv, acc[i][1] * inv, acc[i][2] * inv, acc[i][3] * inv);
            *reinterpret_cast<float4 *>(s_o + off[i]) = r;
            if (p.out_heads) *reinterpret_cast<float4 *>(p.out_heads + row * D + off[i]) = r;
        }
        __syncwarp();
        const float inv_h = 1.0f / static_cast<float>(H);
        for (int f = lane; f < p.F; f += 32) {
            float a = 0.0f;
            for (int h = 0; h < H; ++h) a += s_o[h * p.F + f];
            p.out[row * p.F + f] = activate(a * inv_h, p.act);
        }
    } else {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            if (!valid[i]) continue;
            const float l = s_l[hd[i]];
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            *reinterpret_cast<float4 *>(p.out + row * D + off[i]) =
                make_float4(activate(acc[i][0] * inv, p.act), activate(acc[i][1] * inv, p.act),
                            activate(acc[i][2] * inv, p.act), activate(acc[i][3] * inv, p.act));
        }
    }
}

template <int NV, bool MEAN, bool PLAN>
__global__ void __launch_bounds__(256) gat_fwd_kernel(const __grid_constant__ GatParams p) {
    gat_fwd_body<NV, MEAN, PLAN>(p);
}

// The same body held to 64 registers (four 256-thread CTAs per SM).  Left to itself the compiler settles on 48
// registers for the two-slice head-mean variant and serialises the gathers: 7.2 ms against 6.5 ms on the 8x32 layer.
template <int NV, bool MEAN, bool PLAN>
__global__ void __launch_bounds__(256, 4) gat_fwd_kernel_r64(const __grid_constant__ GatParams p) {
    gat_fwd_body<NV, MEAN, PLAN>(p);
}

// Finishes the hub rows of the fused forward: combines the chunks' (maximum, sum, unnormalised aggregate) in chunk
// order.  One CTA per chunk; only the first chunk of a row works.
__global__ void __launch_bounds__(128) gat_fwd_merge_kernel(const __grid_constant__ GatParams p) {
    __shared__ float s_m[32], s_inv[32], s_o[512];
    const int64_t c0 = blockIdx.x;
    const int64_t row = __ldg(p.chunk_row + c0);
    const int64_t rb = load_ptr(p.indptr, p.is64, row);
    if (__ldg(p.chunk_begin + c0) != rb) return;
    const int64_t re = load_ptr(p.indptr, p.is64, row + 1);
    const int nch = static_cast<int>((re - rb + p.chunk_edges - 1) / p.chunk_edges);
    const int H = p.H, F = p.F, D = H * F;
    const int64_t stride = fwd_partial_stride(H, F);
    const float *part = p.partial + c0 * stride;
    if (threadIdx.x < H) {
        const int h = threadIdx.x;
        float m = -CUDART_INF_F;
        for (int c = 0; c < nch; ++c) m = fmaxf(m, part[c * stride + D + h]);
        float l = 0.0f;
        for (int c = 0; c < nch; ++c) l += part[c * stride + D + H + h] * expf(part[c * stride + D + h] - m);
        s_m[h] = m;
        s_inv[h] = l > 0.0f ? 1.0f / l : 0.0f;
        p.row_max[row * H + h] = m;
        p.row_sum[row * H + h] = l;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const int h = d / F;
        float a = 0.0f;
        for (int c = 0; c < nch; ++c) a = fmaf(part[c * stride + d], expf(part[c * stride + D + h] - s_m[h]), a);
        const float v = a * s_inv[h];
        if (p.head_mean) {
            s_o[d] = v;
            if (p.out_heads) p.out_heads[row * D + d] = v;
        } else {
            p.out[row * D + d] = activate(v, p.act);
        }
    }
    if (!p.head_mean) return;
    __syncthreads();
    const float inv_h = 1.0f / static_cast<float>(H);
    for (int f = threadIdx.x; f < F; f += blockDim.x) {
        float a = 0.0f;
        for (int h = 0; h < H; ++h) a += s_o[h * F + f];
        p.out[row * F + f] = activate(a * inv_h, p.act);
    }
}

// ---------------------------------------------------------------------------------------------------------
// Fused GAT backward, destination side.  With the forward's row statistics (max M, sum L) the attention of an edge
// is p = exp(LeakyReLU(q+k) - M) / L on its own, and sum_e p_e * dp_e over a row equals Dv = <grad_out, out> of that
// row, so every edge is independent:
//   dp = <grad_out[row,h,:], x[col,h,:]>   (edge_dot_rows_kernel: the gather pass, at the DRAM roofline)
//   d score = p * (dp - Dv) * LeakyReLU'(q+k)   (gat_bwd_score_kernel: streams dp, writes attention and d score in
//                                                place, sums d score per row into grad_query)
// A single kernel doing both passes was measured slower (9.0 ms against 5.6 + 2.2 ms on the 8x32 layer): its register
// count costs the gather pass a fifth of its warps.  The score pass is latency bound (a short dependent chain per row),
// so it is held to 48 registers for five CTAs per SM (2.9 ms at 64 registers).  Hub rows are processed as chunks; chunk_sum_kernel adds the
// chunks' grad_query partials in order.
// ---------------------------------------------------------------------------------------------------------
struct GatBwdParams {
    int64_t n_rows;
    const void *indptr;
    const int *indices;
    int is64, H, F, hshift;
    float slope;
    const float *q, *k, *out_heads, *row_max, *row_sum;
    const float *g;  // upstream gradient: [n_rows,H,F], or [n_rows,F] shared by the heads (g_shared), times g_scale
    int g_shared;
    float g_scale;
    float *edge_attn, *edge_grad, *grad_q;  // edge_grad holds dp on entry, d score on exit
    int64_t n_chunks;
    int chunk_edges;
    const int *chunk_row;
    const int64_t *chunk_begin;
    float *q_partial;  // [n_chunks, H]
};

__global__ void __launch_bounds__(256, 5) gat_bwd_score_kernel(const __grid_constant__ GatBwdParams p) {
    extern __shared__ float smem[];
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t gid = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + wib;
    int64_t row, eb, ee;
    const bool chunk = gid < p.n_chunks;
    if (chunk) {
        row = __ldg(p.chunk_row + gid);
        eb = __ldg(p.chunk_begin + gid);
        ee = min(eb + static_cast<int64_t>(p.chunk_edges), load_ptr(p.indptr, p.is64, row + 1));
    } else {
        row = gid - p.n_chunks;
        if (row >= p.n_rows) return;
        eb = load_ptr(p.indptr, p.is64, row);
        ee = load_ptr(p.indptr, p.is64, row + 1);
        if (p.n_chunks > 0 && ee - eb > p.chunk_edges) return;
    }
    const int H = p.H, F = p.F;
    const int64_t D = static_cast<int64_t>(H) * F;
    const bool pow2 = p.hshift >= 0;  // then a lane always meets the same head: idx % H == lane % H
    float *base = smem + wib * (32 + 32 * H + 4 * 32);
    int *s_col = reinterpret_cast<int *>(base);
    float *s_v = base + 32;
    float *s_q = s_v + 32 * H, *s_m = s_q + 32, *s_il = s_m + 32, *s_d = s_il + 32;
    if (lane < H) {
        s_q[lane] = __ldg(p.q + row * H + lane);
        s_m[lane] = __ldg(p.row_max + row * H + lane);
        const float l = __ldg(p.row_sum + row * H + lane);
        s_il[lane] = l > 0.0f ? 1.0f / l : 0.0f;
    }
    // Dv[h] = <grad_out[row,h,:], out[row,h,:]>
    const int LPH = F >> 2;
    if ((F & 3) == 0 && LPH <= 32 && (LPH & (LPH - 1)) == 0 && D <= 512) {
        // 128-bit slices, all requested before the first use; a head's lanes are adjacent: butterfly inside the head
        float d[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t off = static_cast<int64_t>(i * 32 + lane) * 4;
            d[i] = 0.0f;
            if (off < D) {
                const int64_t goff = p.g_shared ? off % F : off;
                const float4 gv = __ldg(reinterpret_cast<const float4 *>(p.g + row * (p.g_shared ? F : D) + goff));
                const float4 ov = __ldg(reinterpret_cast<const float4 *>(p.out_heads + row * D + off));
                d[i] = gv.x * ov.x + gv.y * ov.y + gv.z * ov.z + gv.w * ov.w;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t off = static_cast<int64_t>(i * 32 + lane) * 4;
            for (int o = LPH >> 1; o > 0; o >>= 1) d[i] += __shfl_xor_sync(0xffffffffu, d[i], o);
            if (off < D && (lane & (LPH - 1)) == 0) s_d[off / F] = d[i] * p.g_scale;
        }
    } else {
        for (int h = 0; h < H; ++h) {
            const float *gp = p.g_shared ? p.g + row * F : p.g + row * D + static_cast<int64_t>(h) * F;
            const float *op = p.out_heads + row * D + static_cast<int64_t>(h) * F;
            float d = 0.0f;
            for (int k = lane; k < F; k += 32) d = fmaf(__ldg(gp + k), __ldg(op + k), d);
            for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            if (lane == 0) s_d[h] = d * p.g_scale;
        }
    }
    __syncwarp();
    float gq = 0.0f;  // pow2: the lane's own pairs (head lane % H); otherwise lane h owns head h
    for (int64_t e0 = eb; e0 < ee; e0 += 32) {
        const int n = static_cast<int>(min(static_cast<int64_t>(32), ee - e0));
        s_col[lane] = lane < n ? ld_stream(p.indices + e0 + lane) : 0;
        __syncwarp();
        const int npairs = n * H;
        // eight (edge, head) pairs per lane and step: their dp and key loads are all issued before the first result is
        // stored (the stores go to the array the dp values come from, which would otherwise order every load behind them)
        for (int idx0 = lane; idx0 < npairs; idx0 += 256) {
            float dpv[8], kv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = idx0 + 32 * u;
                dpv[u] = kv[u] = 0.0f;
                if (idx < npairs) {
                    const int e = pow2 ? (idx >> p.hshift) : (idx / H);
                    dpv[u] = p.edge_grad[e0 * H + idx];
                    kv[u] = __ldg(p.k + static_cast<int64_t>(s_col[e]) * H + (idx - e * H));
                }
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int idx = idx0 + 32 * u;
                if (idx < npairs) {
                    const int e = pow2 ? (idx >> p.hshift) : (idx / H);
                    const int h = idx - e * H;
                    const float sc = s_q[h] + kv[u];
                    const float pr = expf(leaky_relu(sc, p.slope) - s_m[h]) * s_il[h];
                    const float ds = pr * (dpv[u] - s_d[h]) * (sc < 0.0f ? p.slope : 1.0f);
                    p.edge_attn[e0 * H + idx] = pr;
                    p.edge_grad[e0 * H + idx] = ds;
                    if (pow2) gq += ds;
                    else s_v[idx] = ds;
                }
            }
        }
        if (!pow2) {
            __syncwarp();
            if (lane < H)
                for (int e = 0; e < n; ++e) gq += s_v[e * H + lane];
        }
        __syncwarp();
    }
    if (pow2)  // lanes lane, lane + H, lane + 2H, ... hold partial sums of head lane % H
        for (int o = H; o < 32; o <<= 1) gq += __shfl_xor_sync(0xffffffffu, gq, o);
    if (lane < H) {
        if (chunk) p.q_partial[gid * H + lane] = gq;
        else p.grad_q[row * H + lane] = gq;
    }
}

// ---------------------------------------------------------------------------------------------------------
// Fused GAT backward, source side: the whole backward in ONE pass over the transposed graph.
// For source c and each of its out-edges e = (c -> r) the row of the upstream gradient g[r] has to be gathered anyway
// (grad_x[c] = sum_e p_e g[r_e]); with x[c] held in registers the same row gives dp_e = <g[r_e], x[c]>, and with the
// per-destination constants (query, log-sum statistics, D = <g[r], out[r]>) packed into one 16-byte record per
// (row, head) the edge's attention p_e and score gradient ds_e follow on the spot:
//     p = exp(LeakyReLU(q[r] + k[c]) - M[r]) / L[r],   ds = p (dp - D[r]) LeakyReLU'(q[r] + k[c]).
// grad_key[c] = sum_e ds_e is local to the warp; ds_e is scattered to the edge's CSR position so that grad_query
// is a plain row sum afterwards.  No pass over the forward graph gathers features, and no [nnz,H] attention array
// exists.  One warp per source row or hub chunk (chunks leave partial grad_x / grad_key rows); EU edges in flight.
// ---------------------------------------------------------------------------------------------------------
struct GatSrcParams {
    int64_t n_cols;      // rows of the transposed graph
    const void *t_indptr;
    int is64;
    const int *t_rows, *t_perm;
    int H, F;
    float slope;
    int hshift;             // log2(H) if H is a power of two, else -1
    const float4 *rowpack;  // [n_rows, H]: (query, row max + log row sum, D, unused)
    const float *k, *x;
    const float *g;
    int g_shared;
    float g_scale;
    float *grad_x, *grad_k, *edge_grad;
    int64_t n_chunks;
    int chunk_edges;
    const int *chunk_row;
    const int64_t *chunk_begin;
    float *x_partial, *k_partial;  // [n_chunks, H*F], [n_chunks, H]
    const float *values;           // GIVEN: per-edge weights [nnz, H] in CSR order instead of attention
    float *grad_values;            // GIVEN: d weight [nnz, H] in CSR order
};

// rowpack[r,h] = (q, M + log L, <g[r,h,:], out[r,h,:]>, 0); warp per row, 128-bit slices, butterfly inside a head
__global__ void __launch_bounds__(256)
gat_rowpack_kernel(int64_t n_rows, int H, int F, const float *q, const float *row_max, const float *row_sum,
                   const float *g, int g_shared, float g_scale, const float *out_heads, float4 *rowpack) {
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const int64_t D = static_cast<int64_t>(H) * F;
    const int LPH = F >> 2;
    float d[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t off = static_cast<int64_t>(i * 32 + lane) * 4;
        d[i] = 0.0f;
        if (off < D) {
            const int64_t goff = g_shared ? off % F : off;
            const float4 gv = __ldg(reinterpret_cast<const float4 *>(g + row * (g_shared ? F : D) + goff));
            const float4 ov = __ldg(reinterpret_cast<const float4 *>(out_heads + row * D + off));
            d[i] = gv.x * ov.x + gv.y * ov.y + gv.z * ov.z + gv.w * ov.w;
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t off = static_cast<int64_t>(i * 32 + lane) * 4;
        for (int o = LPH >> 1; o > 0; o >>= 1) d[i] += __shfl_xor_sync(0xffffffffu, d[i], o);
        if (off < D && (lane & (LPH - 1)) == 0) {
            const int64_t h = off / F;
            // p = exp(score - M) / L = exp(score - (M + log L)); rows without edges are never looked up
            const float l = __ldg(row_sum + row * H + h);
            rowpack[row * H + h] = make_float4(__ldg(q + row * H + h), __ldg(row_max + row * H + h) + logf(fmaxf(l, 1e-38f)),
                                               d[i] * g_scale, 0.0f);
        }
    }
}

// Edges are taken in tiles of SRC_TILE.  Shared memory per warp: SRC_TILE destination ids and CSR positions, H keys of
// the source, and per (edge, head) of the tile the attention p, p * LeakyReLU' and the destination's D.  (Tiles of 64,
// which spare rows of 33..64 edges a second chain of dependent loads, were measured slower on the 8x32 layer, 10.5 ms
// against 8.95 ms: the doubled shared memory costs more than the shorter chain gains.)
constexpr int SRC_TILE = 32;
__host__ __device__ __forceinline__ int src_smem_floats(int H) { return 2 * SRC_TILE + 32 + 3 * SRC_TILE * H; }

// GIVEN = true is the backward of a multi-head SpMM with stored edge values (graph_ext.spmm_backward): the weights are
// read instead of rebuilt, and the by-product is d value = <g[r], x[c]> per edge and head.
template <int NV, int VEC, int EU, bool GIVEN>
__device__ __forceinline__ void gat_bwd_src_body(const GatSrcParams &p) {
    extern __shared__ float smem[];
    const int wib = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t gid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    int64_t c, eb, ee;
    const bool chunk = gid < p.n_chunks;
    if (chunk) {
        c = __ldg(p.chunk_row + gid);
        eb = __ldg(p.chunk_begin + gid);
        ee = min(eb + static_cast<int64_t>(p.chunk_edges), load_ptr(p.t_indptr, p.is64, c + 1));
    } else {
        c = gid - p.n_chunks;
        if (c >= p.n_cols) return;
        eb = load_ptr(p.t_indptr, p.is64, c);
        ee = load_ptr(p.t_indptr, p.is64, c + 1);
        if (p.n_chunks > 0 && ee - eb > p.chunk_edges) return;
    }
    const int H = p.H, F = p.F;
    const int D = H * F;
    const int LPH = F / VEC;  // lanes per head: a power of two <= 32
    const bool leader = (lane & (LPH - 1)) == 0;
    const int64_t gstride = p.g_shared ? F : D;
    float *base = smem + wib * src_smem_floats(H);
    int *s_r = reinterpret_cast<int *>(base), *s_pos = s_r + SRC_TILE;
    float *s_k = base + 2 * SRC_TILE, *s_p = s_k + 32, *s_pf = s_p + SRC_TILE * H, *s_d = s_pf + SRC_TILE * H;
    if (!GIVEN && lane < H) s_k[lane] = __ldg(p.k + c * H + lane);
    int hd[NV], off[NV], goff[NV];  // offsets inside a row: H*F <= 512
    bool valid[NV];
    float xr[NV][VEC], acc[NV][VEC];
    float gk_lane = 0.0f;  // partial sum of the score gradients of head lane % H (lane h of head h when H is not 2^k)
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        off[i] = (i * 32 + lane) * VEC;
        valid[i] = off[i] < D;
        hd[i] = valid[i] ? off[i] / F : 0;
        goff[i] = p.g_shared ? off[i] - hd[i] * F : off[i];
        if (valid[i]) {
            load_vec<VEC>(xr[i], p.x + c * D + off[i]);
        } else {
#pragma unroll
            for (int v = 0; v < VEC; ++v) xr[i][v] = 0.0f;
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[i][v] = 0.0f;
    }
    for (int64_t e0 = eb; e0 < ee; e0 += SRC_TILE) {
        const int n = static_cast<int>(min(static_cast<int64_t>(SRC_TILE), ee - e0));
        int my_r[SRC_TILE / 32], my_pos[SRC_TILE / 32];
#pragma unroll
        for (int t = 0; t < SRC_TILE / 32; ++t) {
            my_r[t] = my_pos[t] = 0;
            if (t * 32 + lane < n) {
                my_r[t] = ld_stream(p.t_rows + e0 + t * 32 + lane);
                my_pos[t] = ld_stream(p.t_perm + e0 + t * 32 + lane);
            }
        }
        const int r_first = __shfl_sync(0xffffffffu, my_r[0], 0);
#pragma unroll
        for (int t = 0; t < SRC_TILE / 32; ++t) {
            s_r[t * 32 + lane] = t * 32 + lane < n ? my_r[t] : r_first;  // padding edges repeat the first one, attention 0
            s_pos[t * 32 + lane] = my_pos[t];
        }
        __syncwarp();
        // attention and its factors for the tile's (edge, head) pairs: one 16-byte record of the destination each
        const int n_up = (n + EU - 1) & ~(EU - 1);
        for (int idx = lane; idx < n_up * H; idx += 32) {
            const int e = p.hshift >= 0 ? (idx >> p.hshift) : (idx / H);
            const int h = idx - e * H;
            float pr = 0.0f, pf = 0.0f, dv = 0.0f;
            if constexpr (GIVEN) {
                if (e < n) pr = __ldg(p.values + static_cast<int64_t>(s_pos[e]) * H + h);
            } else if (e < n) {
                const float4 rp = __ldg(p.rowpack + static_cast<int64_t>(s_r[e]) * H + h);
                const float sc = rp.x + s_k[h];
                pr = expf(leaky_relu(sc, p.slope) - rp.y);
                pf = sc < 0.0f ? pr * p.slope : pr;
                dv = rp.z;
            }
            s_p[idx] = pr;
            if constexpr (!GIVEN) {
                s_pf[idx] = pf;
                s_d[idx] = dv;
            }
        }
        __syncwarp();
        for (int j = 0; j < n_up; j += EU) {
            float gv[EU][NV][VEC];
#pragma unroll
            for (int u = 0; u < EU; ++u) {
                const float *gr = p.g + static_cast<int64_t>(s_r[j + u]) * gstride;
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    if (valid[i]) {
                        load_vec<VEC>(gv[u][i], gr + goff[i]);
                    } else {
#pragma unroll
                        for (int v = 0; v < VEC; ++v) gv[u][i][v] = 0.0f;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < EU; ++u) {
#pragma unroll
                for (int i = 0; i < NV; ++i) {
                    float dp = 0.0f;
#pragma unroll
                    for (int v = 0; v < VEC; ++v) dp = fmaf(gv[u][i][v], xr[i][v], dp);
                    for (int o = LPH >> 1; o > 0; o >>= 1) dp += __shfl_xor_sync(0xffffffffu, dp, o);
                    const int slot = (j + u) * H + hd[i];
                    const float w = valid[i] ? s_p[slot] * p.g_scale : 0.0f;
#pragma unroll
                    for (int v = 0; v < VEC; ++v) acc[i][v] = fmaf(w, gv[u][i][v], acc[i][v]);
                    // the head's leader lane leaves dp (minus the destination's D) for the pass over the pairs below
                    if (leader && valid[i]) s_d[slot] = dp * p.g_scale - (GIVEN ? 0.0f : s_d[slot]);
                }
            }
        }
        __syncwarp();
        // score gradients (or d value) of the tile, spread over (edge, head) pairs: scattered to the edges' CSR positions
        for (int idx = lane; idx < n * H; idx += 32) {
            const int e = p.hshift >= 0 ? (idx >> p.hshift) : (idx / H);
            const int h = idx - e * H;
            if constexpr (GIVEN) {
                p.grad_values[static_cast<int64_t>(s_pos[e]) * H + h] = s_d[idx];
            } else {
                const float ds = s_pf[idx] * s_d[idx];
                p.edge_grad[static_cast<int64_t>(s_pos[e]) * H + h] = ds;
                if (p.hshift >= 0) gk_lane += ds;  // H a power of two: this lane always meets head lane % H
                else s_pf[idx] = ds;
            }
        }
        if (!GIVEN && p.hshift < 0) {
            __syncwarp();
            if (lane < H)
                for (int e = 0; e < n; ++e) gk_lane += s_pf[e * H + lane];
        }
        __syncwarp();
    }
    float *xdst = chunk ? p.x_partial + gid * D : p.grad_x + c * D;
    float *kdst = chunk ? p.k_partial + gid * H : p.grad_k + c * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        if (!valid[i]) continue;
        store_vec<VEC>(xdst + off[i], acc[i]);
    }
    if constexpr (!GIVEN) {
        if (p.hshift >= 0)
            for (int o = H; o < 32; o <<= 1) gk_lane += __shfl_xor_sync(0xffffffffu, gk_lane, o);
        if (lane < H) kdst[lane] = gk_lane;
    }
}

template <int NV, int VEC, int EU, bool GIVEN>
__global__ void __launch_bounds__(256) gat_bwd_src_kernel(const __grid_constant__ GatSrcParams p) {
    gat_bwd_src_body<NV, VEC, EU, GIVEN>(p);
}

// the same body held to 64 registers, four CTAs per SM: 8.95 ms against 9.58 ms at 80 registers for the backward of the
// 8x32 layer (the few spilled values cost less than the lost warps)
template <int NV, int VEC, int EU, bool GIVEN>
__global__ void __launch_bounds__(256, 4) gat_bwd_src_kernel_r64(const __grid_constant__ GatSrcParams p) {
    gat_bwd_src_body<NV, VEC, EU, GIVEN>(p);
}

// out[row, :W] = sum of the row's chunk partials, in chunk order (one CTA per chunk, the row's first chunk works)
__global__ void __launch_bounds__(128)
chunk_sum_kernel(const void *indptr, int is64, int chunk_edges, const int *chunk_row, const int64_t *chunk_begin, int W,
                 const float *partial, float *out) {
    const int64_t c0 = blockIdx.x;
    const int64_t row = __ldg(chunk_row + c0);
    const int64_t rb = load_ptr(indptr, is64, row);
    if (__ldg(chunk_begin + c0) != rb) return;
    const int64_t nch = (load_ptr(indptr, is64, row + 1) - rb + chunk_edges - 1) / chunk_edges;
    for (int d = threadIdx.x; d < W; d += blockDim.x) {
        float a = 0.0f;
        for (int64_t c = 0; c < nch; ++c) a += partial[(c0 + c) * W + d];
        out[row * W + d] = a;
    }
}

static int head_block(int64_t H) {
    int hb = 1;
    while (hb < H && hb < 32) hb <<= 1;
    return hb;
}

}  // namespace yitu

using namespace yitu;

static int fill_plan(const yitu_hub_plan_t *plan, int64_t *n_chunks, int *chunk_edges, const int **chunk_row,
                     const int64_t **chunk_begin) {
    *n_chunks = 0;
    *chunk_edges = 0;
    *chunk_row = nullptr;
    *chunk_begin = nullptr;
    if (plan == nullptr || plan->n_chunks == 0) return YITU_OK;
    YITU_REQUIRE(plan->chunk_edges >= 32 && plan->chunk_row && plan->chunk_begin, YITU_ERR_INVALID_ARG,
                 "hub plan needs chunk_edges >= 32 and its two tables");
    *n_chunks = plan->n_chunks;
    *chunk_edges = plan->chunk_edges;
    *chunk_row = plan->chunk_row;
    *chunk_begin = plan->chunk_begin;
    return YITU_OK;
}

static int check_softmax_args(const yitu_csr_t *g, int32_t n_segments, int64_t H) {
    if (int rc = validate_csr(g)) return rc;
    YITU_REQUIRE(n_segments >= 1 && n_segments <= 256, YITU_ERR_INVALID_ARG, "n_segments=%d", n_segments);
    YITU_REQUIRE(n_segments == 1 || g->index_mask != 0, YITU_ERR_INVALID_ARG,
                 "several segments need stitched indices (index_mask=0xffffff)");
    YITU_REQUIRE(H >= 1 && H < (1 << 20), YITU_ERR_INVALID_ARG, "n_heads=%lld", (long long)H);
    return YITU_OK;
}

extern "C" int yitu_edge_softmax_fwd_f32(const yitu_csr_t *g, int32_t n_segments, int64_t n_heads, float slope,
                                         const float *query, const float *key, float *attn,
                                         const yitu_hub_plan_t *plan, yitu_stream_t stream) {
    if (int rc = check_softmax_args(g, n_segments, n_heads)) return rc;
    if (g->n_rows == 0 || g->nnz == 0) return YITU_OK;
    YITU_REQUIRE(query && key && attn, YITU_ERR_INVALID_ARG, "NULL tensor");
    SoftmaxParams p{};
    p.n_rows = g->n_rows; p.indptr = g->indptr; p.indices = g->indices; p.is64 = g->indptr_is64;
    p.mask = g->index_mask; p.B = n_segments; p.H = static_cast<int>(n_heads); p.HB = head_block(n_heads);
    p.slope = slope; p.q = query; p.k = key; p.attn_out = attn;
    if (int rc = fill_plan(plan, &p.n_chunks, &p.chunk_edges, &p.chunk_row, &p.chunk_begin)) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    edge_softmax_fwd_kernel<false><<<static_cast<unsigned>((g->n_rows + 7) / 8), 256, 0, st>>>(p);
    YITU_LAUNCH_CHECK();
    if (p.n_chunks > 0) {  // hub rows: one CTA each
        edge_softmax_fwd_kernel<true><<<static_cast<unsigned>(p.n_chunks), 256, 0, st>>>(p);
        YITU_LAUNCH_CHECK();
    }
    return YITU_OK;
}

extern "C" int yitu_edge_softmax_bwd_f32(const yitu_csr_t *g, int32_t n_segments, int64_t n_heads, float slope,
                                         const float *query, const float *key, const float *attn,
                                         const float *grad_attn, float *grad_query, float *edge_grad,
                                         const yitu_hub_plan_t *plan, yitu_stream_t stream) {
    if (int rc = check_softmax_args(g, n_segments, n_heads)) return rc;
    if (g->n_rows == 0) return YITU_OK;
    YITU_REQUIRE(query && grad_query, YITU_ERR_INVALID_ARG, "NULL tensor");
    YITU_REQUIRE(g->nnz == 0 || (key && attn && grad_attn && edge_grad), YITU_ERR_INVALID_ARG, "NULL tensor");
    SoftmaxParams p{};
    p.n_rows = g->n_rows; p.indptr = g->indptr; p.indices = g->indices; p.is64 = g->indptr_is64;
    p.mask = g->index_mask; p.B = n_segments; p.H = static_cast<int>(n_heads); p.HB = head_block(n_heads);
    p.slope = slope; p.q = query; p.k = key; p.attn_in = attn; p.grad_attn = grad_attn;
    p.grad_q = grad_query; p.edge_grad = edge_grad;
    if (int rc = fill_plan(plan, &p.n_chunks, &p.chunk_edges, &p.chunk_row, &p.chunk_begin)) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    edge_softmax_bwd_kernel<false><<<static_cast<unsigned>((g->n_rows + 7) / 8), 256, 0, st>>>(p);
    YITU_LAUNCH_CHECK();
    if (p.n_chunks > 0) {
        edge_softmax_bwd_kernel<true><<<static_cast<unsigned>(p.n_chunks), 256, 0, st>>>(p);
        YITU_LAUNCH_CHECK();
    }
    return YITU_OK;
}

extern "C" int yitu_edge_gather_sum_f32(int64_t n_cols, const void *t_indptr, int32_t indptr_is64,
                                        const int32_t *t_perm, int64_t n_heads, const float *edge_vals, float *out,
                                        const yitu_hub_plan_t *t_plan, yitu_stream_t stream) {
    YITU_REQUIRE(n_cols >= 0 && n_heads >= 1 && t_indptr, YITU_ERR_INVALID_ARG, "bad argument");
    if (n_cols == 0) return YITU_OK;
    YITU_REQUIRE(out, YITU_ERR_INVALID_ARG, "out is NULL");
    GatherSumParams p{};
    p.n_cols = n_cols; p.t_indptr = t_indptr; p.is64 = indptr_is64; p.perm = t_perm;
    p.H = static_cast<int>(n_heads); p.HB = head_block(n_heads); p.vals = edge_vals; p.out = out;
    if (int rc = fill_plan(t_plan, &p.n_chunks, &p.chunk_edges, &p.chunk_row, &p.chunk_begin)) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    edge_gather_sum_kernel<false><<<static_cast<unsigned>((n_cols + 7) / 8), 256, 0, st>>>(p);
    YITU_LAUNCH_CHECK();
    if (p.n_chunks > 0) {
        edge_gather_sum_kernel<true><<<static_cast<unsigned>(p.n_chunks), 256, 0, st>>>(p);
        YITU_LAUNCH_CHECK();
    }
    return YITU_OK;
}

// grad_shared: grad_out is [n_rows,F] and stands for every head (scaled by grad_scale) — the gradient of a mean
// over heads.
static int edge_dot_impl(const yitu_csr_t *g, int64_t n_heads, int64_t n_feats, const float *grad_out, int grad_shared,
                         float grad_scale, const float *x, float *grad_a, yitu_stream_t stream, int64_t n_chunks = 0,
                         int chunk_edges = 0, const int *chunk_row = nullptr, const int64_t *chunk_begin = nullptr) {
    if (int rc = validate_csr(g)) return rc;
    YITU_REQUIRE(n_heads >= 1 && n_feats >= 1, YITU_ERR_INVALID_ARG, "bad shape");
    if (g->n_rows == 0 || g->nnz == 0) return YITU_OK;
    YITU_REQUIRE(grad_out && x && grad_a, YITU_ERR_INVALID_ARG, "NULL tensor");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int64_t lph = n_feats / 4, D = n_heads * n_feats;
    const bool fast = n_feats % 4 == 0 && lph <= 32 && (lph & (lph - 1)) == 0 && D <= 512 && n_heads <= 128 &&
                      aligned16(grad_out) && aligned16(x);
    const unsigned blocks = static_cast<unsigned>((g->n_rows + 7) / 8);
    if (fast) {
        const int H = static_cast<int>(n_heads), F = static_cast<int>(n_feats);
        const size_t smem = 8 * (32 + 32 * static_cast<size_t>(H)) * sizeof(float);
        const unsigned blocks_plan = static_cast<unsigned>((g->n_rows + n_chunks + 7) / 8);
        auto run = [&](auto kernel) -> int {
            if (smem > 48 * 1024)
                YITU_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
            kernel<<<blocks_plan, 256, smem, st>>>(g->n_rows, g->indptr, g->indptr_is64, g->indices, g->index_mask, H, F,
                                                   grad_out, grad_shared, grad_scale, x, grad_a, n_chunks, chunk_edges,
                                                   chunk_row, chunk_begin);
            YITU_LAUNCH_CHECK();
            return YITU_OK;
        };
        if (D <= 128) return run(edge_dot_rows_kernel<1>);
        if (D <= 256) return run(edge_dot_rows_kernel<2>);
        return run(edge_dot_rows_kernel<4>);
    }
    edge_dot_kernel<<<blocks, 256, 0, st>>>(g->n_rows, g->indptr, g->indptr_is64, g->indices, g->index_mask,
                                            static_cast<int>(n_heads), static_cast<int>(n_feats), head_block(n_feats),
                                            grad_out, grad_shared, grad_scale, x, grad_a);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

extern "C" int yitu_edge_dot_f32(const yitu_csr_t *g, int64_t n_heads, int64_t n_feats, const float *grad_out,
                                 const float *x, float *grad_a, const yitu_hub_plan_t *plan, yitu_stream_t stream) {
    int64_t n_chunks;
    int chunk_edges;
    const int *chunk_row;
    const int64_t *chunk_begin;
    if (int rc = fill_plan(plan, &n_chunks, &chunk_edges, &chunk_row, &chunk_begin)) return rc;
    return edge_dot_impl(g, n_heads, n_feats, grad_out, 0, 1.0f, x, grad_a, stream, n_chunks, chunk_edges, chunk_row,
                         chunk_begin);
}

static int check_gat(const yitu_gat_args_t *a, bool backward) {
    YITU_REQUIRE(a != nullptr, YITU_ERR_INVALID_ARG, "args is NULL");
    if (int rc = validate_csr(&a->graph)) return rc;
    const int64_t H = a->n_heads, F = a->n_feats;
    YITU_REQUIRE(H >= 1 && F >= 1, YITU_ERR_INVALID_ARG, "bad shape");
    YITU_REQUIRE(a->graph.index_mask == 0, YITU_ERR_UNSUPPORTED, "fused GAT takes plain (unstitched) graphs");
    YITU_REQUIRE(H <= 32 && F % 4 == 0 && H * F <= 512, YITU_ERR_UNSUPPORTED,
                 "fused GAT needs H <= 32, F %% 4 == 0, H*F <= 512 (H=%lld F=%lld)", (long long)H, (long long)F);
    (void)backward;
    YITU_REQUIRE(a->activation >= YITU_ACT_NONE && a->activation <= YITU_ACT_ELU, YITU_ERR_INVALID_ARG,
                 "unknown activation %d", a->activation);
    YITU_REQUIRE(a->graph.n_rows == 0 || (a->query && a->out && a->row_max && a->row_sum), YITU_ERR_INVALID_ARG,
                 "NULL tensor");
    YITU_REQUIRE(a->graph.nnz == 0 || (a->key && a->x), YITU_ERR_INVALID_ARG, "NULL tensor");
    YITU_REQUIRE(aligned16(a->x) && aligned16(a->out), YITU_ERR_INVALID_ARG, "x / out must be 16-byte aligned");
    return YITU_OK;
}

static void fill_gat(GatParams &p, const yitu_gat_args_t *a) {
    p.n_rows = a->graph.n_rows; p.indptr = a->graph.indptr; p.indices = a->graph.indices;
    p.is64 = a->graph.indptr_is64; p.H = static_cast<int>(a->n_heads); p.F = static_cast<int>(a->n_feats);
    p.hshift = (p.H & (p.H - 1)) == 0 ? 31 - __builtin_clz(p.H) : -1;
    p.slope = a->slope; p.q = a->query; p.k = a->key; p.x = a->x;
    p.out = a->out; p.row_max = a->row_max; p.row_sum = a->row_sum;
    p.head_mean = a->head_mean ? 1 : 0; p.act = a->activation;
    p.stage = p.head_mean ? p.H * p.F : 0;
    p.out_heads = p.head_mean ? a->out_heads : nullptr;
}

template <typename K>
static int launch_rows(K kernel, const GatParams &p, int smem_floats_per_warp, cudaStream_t st) {
    const int warps = 8;
    const size_t smem = static_cast<size_t>(warps) * smem_floats_per_warp * sizeof(float);
    if (smem > 48 * 1024)
        YITU_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    const int64_t groups = p.n_rows + p.n_chunks;
    kernel<<<static_cast<unsigned>((groups + warps - 1) / warps), warps * 32, smem, st>>>(p);
    YITU_LAUNCH_CHECK();
    return YITU_OK;
}

extern "C" int64_t yitu_gat_fwd_scratch_bytes(int64_t n_chunks, int64_t n_heads, int64_t n_feats) {
    if (n_chunks < 0 || n_heads < 1 || n_feats < 1) return -1;
    return n_chunks * fwd_partial_stride(n_heads, n_feats) * static_cast<int64_t>(sizeof(float));
}

static inline int64_t up256f(int64_t floats) { return (floats + 63) / 64 * 64; }  // 256-byte pieces, counted in floats

extern "C" int64_t yitu_gat_bwd_scratch_bytes(int64_t n_rows, int64_t n_chunks, int64_t t_n_chunks, int64_t n_heads,
                                              int64_t n_feats) {
    if (n_rows < 0 || n_chunks < 0 || t_n_chunks < 0 || n_heads < 1 || n_feats < 1) return -1;
    return (up256f(n_rows * n_heads * 4) + up256f(n_chunks * n_heads) + up256f(t_n_chunks * n_heads) +
            up256f(t_n_chunks * n_heads * n_feats)) *
           static_cast<int64_t>(sizeof(float));
}

extern "C" int yitu_gat_fwd_f32(const yitu_gat_args_t *a, yitu_stream_t stream) {
    if (int rc = check_gat(a, false)) return rc;
    if (a->graph.n_rows == 0) return YITU_OK;
    GatParams p{};
    fill_gat(p, a);
    if (int rc = fill_plan(a->plan, &p.n_chunks, &p.chunk_edges, &p.chunk_row, &p.chunk_begin)) return rc;
    const int64_t D = a->n_heads * a->n_feats;
    if (p.n_chunks > 0) {
        const int64_t need = yitu_gat_fwd_scratch_bytes(p.n_chunks, a->n_heads, a->n_feats);
        YITU_REQUIRE(a->scratch && a->scratch_bytes >= need && aligned16(a->scratch), YITU_ERR_WORKSPACE, "fused GAT forward with a hub plan needs %lld bytes of 16-byte aligned scratch",
                     (long long)need);
        p.partial = a->scratch;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int sm = warp_smem_floats_fwd(p.H, p.stage);
    const auto pick = [&](auto mean, auto plan) -> int {
        constexpr bool M = decltype(mean)::value, P = decltype(plan)::value;
        if (D <= 128) return launch_rows(gat_fwd_kernel<1, M, P>, p, sm, st);
        if (D <= 256) return launch_rows(gat_fwd_kernel_r64<2, M, P>, p, sm, st);
        return launch_rows(gat_fwd_kernel<4, M, P>, p, sm, st);
    };
    using T = std::true_type;
    using Fl = std::false_type;
    const int rc = p.head_mean ? (p.n_chunks > 0 ? pick(T{}, T{}) : pick(T{}, Fl{}))
                               : (p.n_chunks > 0 ? pick(Fl{}, T{}) : pick(Fl{}, Fl{}));
    if (rc) return rc;
    if (p.n_chunks > 0) {
        gat_fwd_merge_kernel<<<static_cast<unsigned>(p.n_chunks), 128, 0, st>>>(p);
        YITU_LAUNCH_CHECK();
    }
    return YITU_OK;
}

// Launches the source-side pass (attention rebuilt, or GIVEN edge values); the caller merges hub chunks afterwards.
template <bool GIVEN>
static int launch_src(GatSrcParams &sp, int64_t t_chunks, const float *x, const float *grad_out, float *grad_x,
                      float *x_partial, cudaStream_t st) {
    const int D = sp.H * sp.F;
    sp.hshift = (sp.H & (sp.H - 1)) == 0 ? 31 - __builtin_clz(sp.H) : -1;
    const unsigned blocks = static_cast<unsigned>((sp.n_cols + t_chunks + 7) / 8);
    const size_t smem = 8 * static_cast<size_t>(src_smem_floats(sp.H)) * sizeof(float);
    auto run = [&](auto kernel) -> int {
        if (smem > 48 * 1024)
            YITU_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kernel<<<blocks, 256, smem, st>>>(sp);
        YITU_LAUNCH_CHECK();
        return YITU_OK;
    };
    // 256-bit gathers when a head spans whole 32-byte slices and every row starts on a 32-byte boundary
    const auto a32 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 31) == 0; };
    const bool wide = sp.F % 8 == 0 && a32(x) && a32(grad_out) && a32(grad_x) && a32(x_partial);
    if (wide && D > 128)
        return D <= 256 ? run(gat_bwd_src_kernel_r64<1, 8, 4, GIVEN>) : run(gat_bwd_src_kernel<2, 8, 2, GIVEN>);
    if (D <= 128) return run(gat_bwd_src_kernel<1, 4, 4, GIVEN>);
    if (D <= 256) return run(gat_bwd_src_kernel<2, 4, 4, GIVEN>);
    return run(gat_bwd_src_kernel<4, 4, 2, GIVEN>);
}

extern "C" int yitu_gat_bwd_f32(const yitu_gat_bwd_args_t *b, yitu_stream_t stream) {
    YITU_REQUIRE(b != nullptr, YITU_ERR_INVALID_ARG, "args is NULL");
    const yitu_gat_args_t *a = &b->fwd;
    if (int rc = check_gat(a, true)) return rc;
    const yitu_csr_t &g = a->graph;
    YITU_REQUIRE(g.nnz < (1ll << 31), YITU_ERR_LIMIT, "fused GAT backward needs nnz < 2^31");
    YITU_REQUIRE(b->grad_out && b->grad_query && b->grad_key && b->grad_x && b->t_indptr, YITU_ERR_INVALID_ARG,
                 "NULL tensor");
    YITU_REQUIRE(g.nnz == 0 || (b->t_rows && b->t_perm && b->edge_grad), YITU_ERR_INVALID_ARG,
                 "NULL transposed graph or scratch");
    YITU_REQUIRE(aligned16(b->grad_out) && aligned16(b->grad_x), YITU_ERR_INVALID_ARG,
                 "grad_out / grad_x must be 16-byte aligned");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int64_t H = a->n_heads, F = a->n_feats, D = H * F;
    const int shared = a->head_mean ? 1 : 0;
    const float gscale = shared ? 1.0f / static_cast<float>(H) : 1.0f;
    const float *out_heads = shared ? a->out_heads : a->out;
    YITU_REQUIRE(g.n_rows == 0 || out_heads, YITU_ERR_INVALID_ARG,
                 "the backward of a head-mean forward needs fwd.out_heads (the per-head result)");

    GatBwdParams p{};
    int64_t t_chunks = 0;
    int t_chunk_edges = 0;
    const int *t_chunk_row = nullptr;
    const int64_t *t_chunk_begin = nullptr;
    if (int rc = fill_plan(a->plan, &p.n_chunks, &p.chunk_edges, &p.chunk_row, &p.chunk_begin)) return rc;
    if (int rc = fill_plan(b->t_plan, &t_chunks, &t_chunk_edges, &t_chunk_row, &t_chunk_begin)) return rc;
    const int64_t need = yitu_gat_bwd_scratch_bytes(g.n_rows, p.n_chunks, t_chunks, H, F);
    YITU_REQUIRE(b->scratch && b->scratch_bytes >= need && aligned16(b->scratch), YITU_ERR_WORKSPACE,
                 "fused GAT backward needs %lld bytes of 16-byte aligned scratch", (long long)need);
    float *rowpack = b->scratch;
    float *q_partial = rowpack + up256f(g.n_rows * H * 4);
    float *k_partial = q_partial + up256f(p.n_chunks * H);
    float *x_partial = k_partial + up256f(t_chunks * H);
    const int64_t lph = F / 4;
    const bool one_pass = lph <= 32 && (lph & (lph - 1)) == 0 && aligned16(a->x) && aligned16(out_heads);

    if (one_pass) {
        // (1) per-destination constants, (2) everything else in one pass over the transposed graph, (3) grad_query as
        // the row sum of the scattered score gradients
        if (g.n_rows > 0) {
            gat_rowpack_kernel<<<static_cast<unsigned>((g.n_rows + 7) / 8), 256, 0, st>>>(
                g.n_rows, static_cast<int>(H), static_cast<int>(F), a->query, a->row_max, a->row_sum, b->grad_out, shared,
                gscale, out_heads, reinterpret_cast<float4 *>(rowpack));
            YITU_LAUNCH_CHECK();
        }
        if (g.n_cols > 0) {
            GatSrcParams sp{};
            sp.n_cols = g.n_cols; sp.t_indptr = b->t_indptr; sp.is64 = g.indptr_is64;
            sp.t_rows = b->t_rows; sp.t_perm = b->t_perm; sp.H = static_cast<int>(H); sp.F = static_cast<int>(F);
            sp.slope = a->slope; sp.rowpack = reinterpret_cast<const float4 *>(rowpack); sp.k = a->key; sp.x = a->x;
            sp.g = b->grad_out; sp.g_shared = shared; sp.g_scale = gscale;
            sp.grad_x = b->grad_x; sp.grad_k = b->grad_key; sp.edge_grad = b->edge_grad;
            sp.n_chunks = t_chunks; sp.chunk_edges = t_chunk_edges; sp.chunk_row = t_chunk_row;
            sp.chunk_begin = t_chunk_begin; sp.x_partial = x_partial; sp.k_partial = k_partial;
            int rc = launch_src<false>(sp, t_chunks, a->x, b->grad_out, b->grad_x, x_partial, st);
            if (rc) return rc;
            if (t_chunks > 0) {
                chunk_sum_kernel<<<static_cast<unsigned>(t_chunks), 128, 0, st>>>(
                    b->t_indptr, g.indptr_is64, t_chunk_edges, t_chunk_row, t_chunk_begin, static_cast<int>(D), x_partial,
                    b->grad_x);
                YITU_LAUNCH_CHECK();
                chunk_sum_kernel<<<static_cast<unsigned>(t_chunks), 128, 0, st>>>(
                    b->t_indptr, g.indptr_is64, t_chunk_edges, t_chunk_row, t_chunk_begin, static_cast<int>(H), k_partial,
                    b->grad_key);
                YITU_LAUNCH_CHECK();
            }
        }
        return yitu_edge_gather_sum_f32(g.n_rows, g.indptr, g.indptr_is64, nullptr, H, b->edge_grad, b->grad_query,
                                        p.n_chunks > 0 ? a->plan : nullptr, stream);
    }

    // Head widths whose lanes-per-head count is not a power of two (or exceeds a warp): destination side as a gather
    // pass (dp) and a score pass over the forward graph, source side as a per-head SpMM and a per-source sum.
    YITU_REQUIRE(g.nnz == 0 || b->edge_attn, YITU_ERR_INVALID_ARG,
                 "this head width takes the two-sided backward, which needs the edge_attn scratch");
    float *spmm_scratch = x_partial;
    if (g.n_rows > 0) {
        if (int rc = edge_dot_impl(&g, H, F, b->grad_out, shared, gscale, a->x, b->edge_grad, stream, p.n_chunks,
                                   p.chunk_edges, p.chunk_row, p.chunk_begin))
            return rc;
        p.n_rows = g.n_rows; p.indptr = g.indptr; p.indices = g.indices; p.is64 = g.indptr_is64;
        p.H = static_cast<int>(H); p.F = static_cast<int>(F);
        p.hshift = (p.H & (p.H - 1)) == 0 ? 31 - __builtin_clz(p.H) : -1;
        p.slope = a->slope; p.q = a->query; p.k = a->key; p.out_heads = out_heads;
        p.row_max = a->row_max; p.row_sum = a->row_sum;
        p.g = b->grad_out; p.g_shared = shared; p.g_scale = gscale;
        p.edge_attn = b->edge_attn; p.edge_grad = b->edge_grad; p.grad_q = b->grad_query;
        p.q_partial = q_partial;
        const int warps = 8;
        const size_t smem = static_cast<size_t>(warps) * (32 + 32 * p.H + 4 * 32) * sizeof(float);
        if (smem > 48 * 1024)
            YITU_CUDA(cudaFuncSetAttribute(gat_bwd_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem)));
        gat_bwd_score_kernel<<<static_cast<unsigned>((g.n_rows + p.n_chunks + warps - 1) / warps), warps * 32, smem, st>>>(p);
        YITU_LAUNCH_CHECK();
        if (p.n_chunks > 0) {
            chunk_sum_kernel<<<static_cast<unsigned>(p.n_chunks), 128, 0, st>>>(
                g.indptr, g.indptr_is64, p.chunk_edges, p.chunk_row, p.chunk_begin, p.H, q_partial, b->grad_query);
            YITU_LAUNCH_CHECK();
        }
    }
    yitu_hub_plan_t tp{};
    yitu_spmm_args_t s{};
    s.graph.n_rows = g.n_cols; s.graph.n_cols = g.n_rows; s.graph.nnz = g.nnz;
    s.graph.indptr = b->t_indptr; s.graph.indptr_is64 = g.indptr_is64; s.graph.index_mask = 0;
    s.graph.indices = b->t_rows;
    s.n_heads = H; s.n_feats = F; s.weight_mode = YITU_W_EDGE_HEAD;
    s.edge_values = b->edge_attn; s.edge_perm = b->t_perm; s.alpha = gscale;
    s.x = b->grad_out; s.x_stride = shared ? F : D; s.x_shared_heads = shared; s.out = b->grad_x; s.out_stride = D;
    if (t_chunks > 0) {
        tp = *b->t_plan;
        s.plan = &tp;
        s.scratch = spmm_scratch;
        s.scratch_bytes = t_chunks * D * static_cast<int64_t>(sizeof(float));
    }
    if (int rc = yitu_spmm_csr_f32(&s, stream)) return rc;
    if (g.n_cols == 0) return YITU_OK;
    return yitu_edge_gather_sum_f32(g.n_cols, b->t_indptr, g.indptr_is64, b->t_perm, H, b->edge_grad, b->grad_key,
                                    t_chunks > 0 ? b->t_plan : nullptr, stream);
}

extern "C" int yitu_spmm_bwd_f32(const yitu_spmm_bwd_args_t *a, yitu_stream_t stream) {
    YITU_REQUIRE(a != nullptr, YITU_ERR_INVALID_ARG, "args is NULL");
    if (int rc = validate_csr(&a->graph)) return rc;
    const yitu_csr_t &g = a->graph;
    const int64_t H = a->n_heads, F = a->n_feats, D = H * F, lph = F / 4;
    YITU_REQUIRE(H >= 1 && F >= 1, YITU_ERR_INVALID_ARG, "bad shape");
    YITU_REQUIRE(H <= 32 && F % 4 == 0 && D <= 512 && lph <= 32 && (lph & (lph - 1)) == 0, YITU_ERR_UNSUPPORTED,
                 "one-pass SpMM backward needs H <= 32, H*F <= 512 and F/4 a power of two <= 32 (H=%lld F=%lld)",
                 (long long)H, (long long)F);
    YITU_REQUIRE(g.nnz < (1ll << 31), YITU_ERR_LIMIT, "one-pass SpMM backward needs nnz < 2^31");
    YITU_REQUIRE(a->t_indptr && (g.n_cols == 0 || a->grad_x), YITU_ERR_INVALID_ARG, "NULL tensor");
    YITU_REQUIRE(g.nnz == 0 || (a->edge_values && a->x && a->grad_out && a->t_rows && a->t_perm && a->grad_values),
                 YITU_ERR_INVALID_ARG, "NULL tensor");
    YITU_REQUIRE(aligned16(a->x) && aligned16(a->grad_out) && aligned16(a->grad_x), YITU_ERR_INVALID_ARG,
                 "x / grad_out / grad_x must be 16-byte aligned");
    if (g.n_cols == 0) return YITU_OK;
    GatSrcParams sp{};
    int64_t t_chunks = 0;
    if (int rc = fill_plan(a->t_plan, &t_chunks, &sp.chunk_edges, &sp.chunk_row, &sp.chunk_begin)) return rc;
    if (t_chunks > 0)
        YITU_REQUIRE(a->scratch && aligned16(a->scratch) && a->scratch_bytes >= t_chunks * D * 4, YITU_ERR_WORKSPACE,
                     "one-pass SpMM backward with a hub plan needs %lld bytes of scratch", (long long)(t_chunks * D * 4));
    sp.n_cols = g.n_cols; sp.t_indptr = a->t_indptr; sp.is64 = g.indptr_is64; sp.t_rows = a->t_rows; sp.t_perm = a->t_perm;
    sp.H = static_cast<int>(H); sp.F = static_cast<int>(F); sp.x = a->x; sp.g = a->grad_out; sp.g_shared = 0;
    sp.g_scale = 1.0f; sp.grad_x = a->grad_x; sp.n_chunks = t_chunks; sp.x_partial = a->scratch;
    sp.values = a->edge_values; sp.grad_values = a->grad_values;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (int rc = launch_src<true>(sp, t_chunks, a->x, a->grad_out, a->grad_x, a->scratch, st)) return rc;
    if (t_chunks > 0) {
        chunk_sum_kernel<<<static_cast<unsigned>(t_chunks), 128, 0, st>>>(a->t_indptr, g.indptr_is64, sp.chunk_edges,
                                                                          sp.chunk_row, sp.chunk_begin,
                                                                          static_cast<int>(D), a->scratch, a->grad_x);
        YITU_LAUNCH_CHECK();
    }
    return YITU_OK;
}
